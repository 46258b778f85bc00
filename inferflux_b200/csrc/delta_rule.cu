// A recurrence with a matrix of state per head that every token decays, partly erases along its own key, and writes to:
//
//   decay_t = exp(-exp(-1/2) * sigmoid(w_raw_t + w0))            per head and key channel
//   a_t     = sigmoid(a_raw_t + a_bias)                          per head and key channel
//   u_t     = k_t / sqrt(sum k_t^2 + 1e-6)                       the unit key of the head
//   S       = diag(decay_t) S - (a_t u_t) (u_t^T S) + k_t v_t^T   both products of the old S  [key channel, value channel]
//   o_t     = S^T r_t                                            of the new S
//   y_t     = o_t / rms(o_t) per head * norm_w * sigmoid(g_t)
//
// Three kernels.  delta_prepare (a warp per token and head) makes decay, a * u and u in float32.  delta_scan walks a
// request's tokens: a column of S (one value channel, all key channels) never meets another column, so the grid is
// (requests, heads, groups of columns); a column's key channels are cut into slices of 8 that neighbouring lanes keep
// in registers, and the two sums over key channels are added across a column's lanes by shuffles.  The step's vectors
// of a stretch of tokens arrive by cp.async in one of two buffers while the other is worked on.  delta_finish (a warp
// per token and head) norms and gates.  Everything is float32, and every sum's order is a function of the head size
// alone, so a token's result does not depend on how its request's tokens were cut into steps or on what else is in the
// batch.
#include "common.cuh"

namespace ifx {

constexpr float kDecayFloor = 0.6065306597126334f;       // exp(-1/2)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// proj: [T, ld] with r, k, v, g, a at column blocks 0..4 of heads * dim.  Out: decay, au, u, r * decay [T, heads * dim]
// and, per token and head, c = (sum r a u, sum r k): with them the output needs the old state only,
//   S_t^T r = (r * decay)^T S_(t-1) - (sum r a u) (u^T S_(t-1)) + (sum r k) v.
__global__ void delta_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ w_raw,
                                     const float* __restrict__ w0, const float* __restrict__ a_bias,
                                     float* __restrict__ decay, float* __restrict__ au, float* __restrict__ unit,
                                     float* __restrict__ rw, float2* __restrict__ c, int num_tokens, int heads, int dim) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int HD = heads * dim;
  const float* r = proj + (size_t)t * ld + h * dim;
  const float* k = proj + (size_t)t * ld + HD + h * dim;
  const float* a = proj + (size_t)t * ld + 4 * HD + h * dim;
  float ss = 0.0f;
  for (int i = lane; i < dim; i += 32) ss = fmaf(k[i], k[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + 1e-6f);
  const size_t base = (size_t)t * HD + h * dim;
  float c1 = 0.0f, c2 = 0.0f;
  for (int i = lane; i < dim; i += 32) {
    const float u = k[i] * inv;
    const float e = sigmoid_f(a[i] + a_bias[h * dim + i]) * u;
    const float d = expf(-kDecayFloor * sigmoid_f(w_raw[base + i] + w0[h * dim + i]));
    unit[base + i] = u;
    au[base + i] = e;
    decay[base + i] = d;
    rw[base + i] = r[i] * d;
    c1 = fmaf(r[i], e, c1);
    c2 = fmaf(r[i], k[i], c2);
  }
  c1 = warp_sum(c1);
  c2 = warp_sum(c2);
  if (lane == 0) c[item] = make_float2(c1, c2);
}

__device__ __forceinline__ void delta_cp_async_4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void delta_cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void delta_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void delta_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kDeltaR = 8;            // key channels a thread keeps
constexpr int kDeltaPad = 4;          // floats between the slices of a staged row: their float4 reads meet no bank twice
constexpr int kDeltaThreads = 128;
constexpr int kDeltaNC = 2;           // columns a thread keeps: one's shuffles run under the other's multiply-adds

// Thread (c, s) = threadIdx.x / KS, threadIdx.x % KS keeps the key channels s * 8 .. s * 8 + 7 of the columns
// j0 + 2 c and j0 + 2 c + 1 of S in registers; the KS threads of a column lie in neighbouring lanes and add their parts of both sums by shuffles, in
// an order that the head size alone decides.  Both sums of a token, u^T S and (r * decay)^T S, are taken of the state
// before the token, so they run side by side and their shuffles overlap.  Block: 128 threads, of which the first cols * KS (whole warps) compute;
// all of them bring the vectors of the next `stage` tokens into the other buffer by cp.async while these are worked on.
template <int KS>
__global__ void __launch_bounds__(kDeltaThreads) delta_scan_kernel(
    const float* __restrict__ proj, int ld, const float* __restrict__ decay, const float* __restrict__ au,
    const float* __restrict__ unit, const float* __restrict__ rw, const float2* __restrict__ c12,
    float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_seqlens,
    const int* __restrict__ req_slot, float* __restrict__ o, int heads, int dim, int cols, int stage, int vec) {
  constexpr int R = kDeltaR;
  constexpr int DP = KS * (R + kDeltaPad);               // a staged row: slice s at s * (R + pad), zeros beyond dim
  extern __shared__ __align__(16) float smem[];          // 2 x ([stage][5][DP]: r * decay, k, decay, au, u ; [stage][cols]: v ; [stage][2])
  const int buf_floats = stage * (5 * DP + cols + 2);
  const int req = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * cols;
  constexpr int NC = kDeltaNC;
  const int tid = threadIdx.x, c = tid / KS, sl = tid % KS;
  const int j = j0 + c * NC;                             // this thread's first column
  const bool computes = (tid & ~31) < cols / NC * KS;    // this warp has columns
  bool live[NC];
#pragma unroll
  for (int cc = 0; cc < NC; ++cc) live[cc] = c * NC + cc < cols && j + cc < dim;
  const int HD = heads * dim;
  const int lo = cu_seqlens[req], hi = cu_seqlens[req + 1];
  float* S_mem = state + (long long)req_slot[req] * slot_stride + (size_t)h * dim * dim;
  float S[NC][R];
#pragma unroll
  for (int cc = 0; cc < NC; ++cc)
#pragma unroll
    for (int i = 0; i < R; ++i) S[cc][i] = (live[cc] && sl * R + i < dim) ? S_mem[(size_t)(sl * R + i) * dim + j + cc] : 0.0f;
  for (int e = tid; e < 2 * buf_floats; e += kDeltaThreads) smem[e] = 0.0f;
  __syncthreads();

  auto fetch = [&](int b, int t0) {
    float* dst = smem + (size_t)b * buf_floats;
    float* v_s = dst + stage * 5 * DP;
    float* c_s = v_s + stage * cols;
    const int n = min(stage, hi - t0);
    for (int e = tid; e < 2 * n; e += kDeltaThreads)
      delta_cp_async_4(c_s + e, reinterpret_cast<const float*>(c12 + (size_t)(t0 + (e >> 1)) * heads + h) + (e & 1));
    if (vec) {                                           // dim, ld and cols in whole float4, rows on 16-byte boundaries
      const int q4 = dim >> 2;
      for (int e = tid; e < n * q4; e += kDeltaThreads) {
        const int tt = e / q4, i = (e % q4) << 2;
        const size_t row = (size_t)(t0 + tt);
        float* d = dst + (size_t)tt * 5 * DP + i + kDeltaPad * (i / R);
        delta_cp_async_16(d, rw + row * HD + h * dim + i);
        delta_cp_async_16(d + DP, proj + row * ld + HD + h * dim + i);
        delta_cp_async_16(d + 2 * DP, decay + row * HD + h * dim + i);
        delta_cp_async_16(d + 3 * DP, au + row * HD + h * dim + i);
        delta_cp_async_16(d + 4 * DP, unit + row * HD + h * dim + i);
      }
      const int c4 = cols >> 2;
      for (int e = tid; e < n * c4; e += kDeltaThreads) {
        const int tt = e / c4, i = (e % c4) << 2;
        if (j0 + i < dim) delta_cp_async_16(v_s + tt * cols + i, proj + (size_t)(t0 + tt) * ld + 2 * HD + h * dim + j0 + i);
      }
    } else {
      for (int e = tid; e < n * dim; e += kDeltaThreads) {
        const int tt = e / dim, i = e % dim;
        const size_t row = (size_t)(t0 + tt);
        float* d = dst + (size_t)tt * 5 * DP + i + kDeltaPad * (i / R);
        delta_cp_async_4(d, rw + row * HD + h * dim + i);
        delta_cp_async_4(d + DP, proj + row * ld + HD + h * dim + i);
        delta_cp_async_4(d + 2 * DP, decay + row * HD + h * dim + i);
        delta_cp_async_4(d + 3 * DP, au + row * HD + h * dim + i);
        delta_cp_async_4(d + 4 * DP, unit + row * HD + h * dim + i);
      }
      for (int e = tid; e < n * cols; e += kDeltaThreads) {
        const int tt = e / cols, i = e % cols;
        if (j0 + i < dim) delta_cp_async_4(v_s + tt * cols + i, proj + (size_t)(t0 + tt) * ld + 2 * HD + h * dim + j0 + i);
      }
    }
  };

  if (lo < hi) fetch(0, lo);
  delta_cp_async_commit();
  int b = 0;
  for (int t0 = lo; t0 < hi; t0 += stage, b ^= 1) {
    if (t0 + stage < hi) fetch(b ^ 1, t0 + stage);
    delta_cp_async_commit();
    delta_cp_async_wait<1>();                            // everything but the copies just asked for has landed
    __syncthreads();
    if (computes) {
      const int n = min(stage, hi - t0);
      const float* cur = smem + (size_t)b * buf_floats;
      const float* v_s = cur + stage * 5 * DP;
      const float2* c_s = reinterpret_cast<const float2*>(v_s + stage * cols);
#pragma unroll 2
      for (int tt = 0; tt < n; ++tt) {
        const float4* g_s = reinterpret_cast<const float4*>(cur + (size_t)tt * 5 * DP + sl * (R + kDeltaPad));
        constexpr int Q = DP / 4;
        const float4 *k_s = g_s + Q, *w_s = g_s + 2 * Q, *au_s = g_s + 3 * Q, *u_s = g_s + 4 * Q;
        const float2 c12v = c_s[tt];
        float vj[NC], along[NC], kept[NC];
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) {
          vj[cc] = v_s[tt * cols + c * NC + cc];
          float al[4] = {0.0f, 0.0f, 0.0f, 0.0f}, ql[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // partial sums over channels i % 4
#pragma unroll
          for (int i = 0; i < R; i += 4) {
            const float4 u4 = u_s[i >> 2], g4 = g_s[i >> 2];
            al[0] = fmaf(u4.x, S[cc][i], al[0]);
            al[1] = fmaf(u4.y, S[cc][i + 1], al[1]);
            al[2] = fmaf(u4.z, S[cc][i + 2], al[2]);
            al[3] = fmaf(u4.w, S[cc][i + 3], al[3]);
            ql[0] = fmaf(g4.x, S[cc][i], ql[0]);
            ql[1] = fmaf(g4.y, S[cc][i + 1], ql[1]);
            ql[2] = fmaf(g4.z, S[cc][i + 2], ql[2]);
            ql[3] = fmaf(g4.w, S[cc][i + 3], ql[3]);
          }
          along[cc] = (al[0] + al[1]) + (al[2] + al[3]);
          kept[cc] = (ql[0] + ql[1]) + (ql[2] + ql[3]);
        }
#pragma unroll
        for (int m = 1; m < KS; m <<= 1) {
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) {
            along[cc] += __shfl_xor_sync(0xffffffffu, along[cc], m);
            kept[cc] += __shfl_xor_sync(0xffffffffu, kept[cc], m);
          }
        }
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 k4 = k_s[i >> 2], w4 = w_s[i >> 2], a4 = au_s[i >> 2];
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) {
            S[cc][i] = fmaf(-a4.x, along[cc], fmaf(k4.x, vj[cc], w4.x * S[cc][i]));
            S[cc][i + 1] = fmaf(-a4.y, along[cc], fmaf(k4.y, vj[cc], w4.y * S[cc][i + 1]));
            S[cc][i + 2] = fmaf(-a4.z, along[cc], fmaf(k4.z, vj[cc], w4.z * S[cc][i + 2]));
            S[cc][i + 3] = fmaf(-a4.w, along[cc], fmaf(k4.w, vj[cc], w4.w * S[cc][i + 3]));
          }
        }
        if (sl == 0) {
#pragma unroll
          for (int cc = 0; cc < NC; ++cc)
            if (live[cc]) o[(size_t)(t0 + tt) * HD + h * dim + j + cc] = fmaf(c12v.y, vj[cc], fmaf(-c12v.x, along[cc], kept[cc]));
        }
      }
    }
    __syncthreads();                                     // the buffer is filled again two stretches on
  }
  delta_cp_async_wait<0>();
#pragma unroll
  for (int cc = 0; cc < NC; ++cc) {
    if (!live[cc]) continue;
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (sl * R + i < dim) S_mem[(size_t)(sl * R + i) * dim + j + cc] = S[cc][i];
  }
}

// y = o / rms(o) per head * norm_w * sigmoid(g): a warp per (token, head).
template <typename TO>
__global__ void delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj, int ld,
                                    const float* __restrict__ norm_w, float eps, TO* __restrict__ y, int num_tokens,
                                    int heads, int dim) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int HD = heads * dim;
  const float* orow = o + (size_t)t * HD + h * dim;
  const float* g = proj + (size_t)t * ld + 3 * HD + h * dim;
  float ss = 0.0f;
  for (int i = lane; i < dim; i += 32) ss = fmaf(orow[i], orow[i], ss);
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
  for (int i = lane; i < dim; i += 32)
    y[(size_t)t * HD + h * dim + i] = from_f32<TO>(orow[i] * r * norm_w[h * dim + i] * sigmoid_f(g[i]));
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// Floats of scratch the scan needs for T tokens: decay, a * u, u, o and r * decay, [T, heads * dim] each, and two numbers per
// token and head.
long long ifx_delta_rule_scratch_floats(int T, int heads, int dim) { return 5LL * T * heads * dim + 2LL * T * heads + 4; }

// proj: float32 [T, ld], the projections r, k, v, g, a in column blocks of heads * dim; w_raw: float32 [T, heads * dim];
// state: float32, slot s at state + s * slot_stride holds [heads, dim, dim]; y: [T, heads * dim] in out_dtype.
int ifx_delta_rule_scan(const float* proj, int ld, const float* w_raw, const float* w0, const float* a_bias,
                        const float* norm_w, float eps, float* state, long long slot_stride, const int* cu_seqlens,
                        const int* req_slot, float* scratch, void* y, int num_requests, int T, int heads, int dim,
                        int out_dtype, cudaStream_t stream) {
  if (T <= 0 || num_requests <= 0) return 0;
  if (heads <= 0 || dim <= 0 || ld < 5 * heads * dim || slot_stride < (long long)heads * dim * dim) return IFX_E_BADARG;
  if (dim > 256) return IFX_E_TOOBIG;
  const size_t n = (size_t)T * heads * dim;
  float *decay = scratch, *au = scratch + n, *unit = scratch + 2 * n, *o = scratch + 3 * n, *rw = scratch + 4 * n;
  float2* c12 = reinterpret_cast<float2*>(scratch + ((5 * n + 1) & ~(size_t)1));
  const long long items = (long long)T * heads;
  delta_prepare_kernel<<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(proj, ld, w_raw, w0, a_bias, decay, au, unit, rw, c12, T, heads,
                                                                        dim);
  IFX_CHECK_LAUNCH();
  // slices of 8 key channels: a function of the head size alone, so that no sum's order depends on anything else
  const int KS = dim <= 8 ? 1 : dim <= 16 ? 2 : dim <= 32 ? 4 : dim <= 64 ? 8 : dim <= 128 ? 16 : 32;
  // columns a block: as many as its 128 threads take, then fewer (whole warps) as long as all blocks still run at once
  const int least = 32 / KS * kDeltaNC > 4 ? 32 / KS * kDeltaNC : 4;      // whole warps, and whole float4 of values
  const int stage = KS <= 8 ? 16 : 8;                    // tokens a buffer: 62 KB of shared memory at most, 123 KB for KS = 32
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 1;
  }
  auto bytes_for = [&](int c) { return (size_t)2 * stage * (5 * KS * (kDeltaR + kDeltaPad) + c + 2) * sizeof(float); };
  auto blocks_for = [&](int c) { return (long long)num_requests * heads * ((dim + c - 1) / c); };
  auto room_for = [&](int c) {                           // blocks that run at once: shared memory, and 80 registers a thread
    const long long by_smem = (long long)(227 * 1024 / (bytes_for(c) + 1024));
    return (long long)sms * (by_smem < 1 ? 1 : by_smem > 6 ? 6 : by_smem);
  };
  int cols = kDeltaThreads / KS * kDeltaNC;
  while (cols > least && (cols / 2 >= dim || blocks_for(cols / 2) <= room_for(cols / 2))) cols /= 2;
  dim3 grid(num_requests, heads, (dim + cols - 1) / cols);
  const int vec = (dim % 4 == 0 && ld % 4 == 0 && cols % 4 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)scratch % 16 == 0) ? 1 : 0;
  const size_t smem = bytes_for(cols);
#define IFX_SCAN(KK)                                                                                              \
  do {                                                                                                            \
    auto kern = delta_scan_kernel<KK>;                                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    kern<<<grid, kDeltaThreads, smem, stream>>>(proj, ld, decay, au, unit, rw, c12, state, slot_stride, cu_seqlens,  \
                                                req_slot, o, heads, dim, cols, stage, vec);                       \
  } while (0)
  if (KS == 1) IFX_SCAN(1);
  else if (KS == 2) IFX_SCAN(2);
  else if (KS == 4) IFX_SCAN(4);
  else if (KS == 8) IFX_SCAN(8);
  else if (KS == 16) IFX_SCAN(16);
  else IFX_SCAN(32);
#undef IFX_SCAN
  IFX_CHECK_LAUNCH();
  if (out_dtype == IFX_DT_F32)
    delta_finish_kernel<float><<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(o, proj, ld, norm_w, eps, (float*)y, T, heads, dim);
  else if (out_dtype == IFX_DT_BF16)
    delta_finish_kernel<__nv_bfloat16><<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(o, proj, ld, norm_w, eps,
                                                                                       (__nv_bfloat16*)y, T, heads, dim);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
