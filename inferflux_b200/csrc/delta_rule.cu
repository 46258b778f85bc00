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
// request's tokens: a column of S (one value channel, all key channels) never meets another column, so a thread keeps
// one column in registers, a block a group of columns, and the grid is (requests, heads, column groups); the step's
// vectors of a stretch of tokens are staged in shared memory (rows padded with zeros to whole float4, read as such),
// and both sums over key channels run as four interleaved partial sums (channels i % 4) so that their additions do not
// wait for each other.  delta_finish (a warp per token and head) norms and gates.  Everything is float32, and every
// sum's order is a function of the head size alone, so a token's result does not depend on how its request's tokens
// were cut into steps or on what else is in the batch.
#include "common.cuh"

namespace ifx {

constexpr float kDecayFloor = 0.6065306597126334f;       // exp(-1/2)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// proj: [T, ld] with r, k, v, g, a at column blocks 0..4 of heads * dim.  Out: decay, au, u [T, heads * dim].
__global__ void delta_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ w_raw,
                                     const float* __restrict__ w0, const float* __restrict__ a_bias,
                                     float* __restrict__ decay, float* __restrict__ au, float* __restrict__ unit,
                                     int num_tokens, int heads, int dim) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int HD = heads * dim;
  const float* k = proj + (size_t)t * ld + HD + h * dim;
  const float* a = proj + (size_t)t * ld + 4 * HD + h * dim;
  float ss = 0.0f;
  for (int i = lane; i < dim; i += 32) ss = fmaf(k[i], k[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + 1e-6f);
  const size_t base = (size_t)t * HD + h * dim;
  for (int i = lane; i < dim; i += 32) {
    const float u = k[i] * inv;
    unit[base + i] = u;
    au[base + i] = sigmoid_f(a[i] + a_bias[h * dim + i]) * u;
    decay[base + i] = expf(-kDecayFloor * sigmoid_f(w_raw[base + i] + w0[h * dim + i]));
  }
}

constexpr int kDeltaStage = 16;       // tokens staged at a time

// D: key channels a thread keeps (>= dim).  Block: `cols` threads, one value channel each.
template <int D>
__global__ void __launch_bounds__(128) delta_scan_kernel(
    const float* __restrict__ proj, int ld, const float* __restrict__ decay, const float* __restrict__ au,
    const float* __restrict__ unit, float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_seqlens,
    const int* __restrict__ req_slot, float* __restrict__ o, int heads, int dim, int cols) {
  extern __shared__ __align__(16) float stage[];         // [kDeltaStage][5][dp]: r, k, decay, au, u ; then v [kDeltaStage][cols]
  const int dp = (dim + 3) & ~3;                         // a staged row, padded with zeros to whole float4
  const int req = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * cols;
  const int j = j0 + threadIdx.x;
  const bool live = threadIdx.x < cols && j < dim;
  const int HD = heads * dim;
  const int lo = cu_seqlens[req], hi = cu_seqlens[req + 1];
  float* S_mem = state + (long long)req_slot[req] * slot_stride + (size_t)h * dim * dim;
  float S[D];
#pragma unroll
  for (int i = 0; i < D; ++i) S[i] = (live && i < dim) ? S_mem[(size_t)i * dim + j] : 0.0f;
  float* v_s = stage + kDeltaStage * 5 * dp;
  for (int t0 = lo; t0 < hi; t0 += kDeltaStage) {
    const int n = min(kDeltaStage, hi - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < n * dp; e += blockDim.x) {
      const int tt = e / dp, i = e % dp;
      const size_t row = (size_t)(t0 + tt);
      float* dst = stage + (size_t)tt * 5 * dp;
      const bool in = i < dim;
      dst[i] = in ? proj[row * ld + h * dim + i] : 0.0f;
      dst[dp + i] = in ? proj[row * ld + HD + h * dim + i] : 0.0f;
      dst[2 * dp + i] = in ? decay[row * HD + h * dim + i] : 0.0f;
      dst[3 * dp + i] = in ? au[row * HD + h * dim + i] : 0.0f;
      dst[4 * dp + i] = in ? unit[row * HD + h * dim + i] : 0.0f;
    }
    for (int e = threadIdx.x; e < n * cols; e += blockDim.x) {
      const int tt = e / cols, c = e % cols;
      v_s[tt * cols + c] = j0 + c < dim ? proj[(size_t)(t0 + tt) * ld + 2 * HD + h * dim + j0 + c] : 0.0f;
    }
    __syncthreads();
    if (!live) continue;
    for (int tt = 0; tt < n; ++tt) {
      const float4* r_s = reinterpret_cast<const float4*>(stage + (size_t)tt * 5 * dp);
      const int q4 = dp >> 2;
      const float4 *k_s = r_s + q4, *w_s = r_s + 2 * q4, *au_s = r_s + 3 * q4, *u_s = r_s + 4 * q4;
      const float vj = v_s[tt * cols + threadIdx.x];
      float al[4] = {0.0f, 0.0f, 0.0f, 0.0f};                          // partial sums over channels i % 4
#pragma unroll
      for (int i = 0; i < D; i += 4)
        if (i < dp) {
          const float4 u4 = u_s[i >> 2];
          al[0] = fmaf(u4.x, S[i], al[0]);
          al[1] = fmaf(u4.y, S[i + 1], al[1]);
          al[2] = fmaf(u4.z, S[i + 2], al[2]);
          al[3] = fmaf(u4.w, S[i + 3], al[3]);
        }
      const float along = (al[0] + al[1]) + (al[2] + al[3]);
      float ou[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < D; i += 4)
        if (i < dp) {
          const float4 k4 = k_s[i >> 2], w4 = w_s[i >> 2], a4 = au_s[i >> 2], r4 = r_s[i >> 2];
          S[i] = fmaf(k4.x, vj, fmaf(-a4.x, along, w4.x * S[i]));
          S[i + 1] = fmaf(k4.y, vj, fmaf(-a4.y, along, w4.y * S[i + 1]));
          S[i + 2] = fmaf(k4.z, vj, fmaf(-a4.z, along, w4.z * S[i + 2]));
          S[i + 3] = fmaf(k4.w, vj, fmaf(-a4.w, along, w4.w * S[i + 3]));
          ou[0] = fmaf(S[i], r4.x, ou[0]);
          ou[1] = fmaf(S[i + 1], r4.y, ou[1]);
          ou[2] = fmaf(S[i + 2], r4.z, ou[2]);
          ou[3] = fmaf(S[i + 3], r4.w, ou[3]);
        }
      o[(size_t)(t0 + tt) * HD + h * dim + j] = (ou[0] + ou[1]) + (ou[2] + ou[3]);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < D; ++i)
      if (i < dim) S_mem[(size_t)i * dim + j] = S[i];
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

// Floats of scratch the scan needs for T tokens: decay, a * u, u and o, [T, heads * dim] each.
long long ifx_delta_rule_scratch_floats(int T, int heads, int dim) { return 4LL * T * heads * dim; }

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
  float *decay = scratch, *au = scratch + n, *unit = scratch + 2 * n, *o = scratch + 3 * n;
  const long long items = (long long)T * heads;
  delta_prepare_kernel<<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(proj, ld, w_raw, w0, a_bias, decay, au, unit, T, heads, dim);
  IFX_CHECK_LAUNCH();
  // columns a block: all of a head's while (requests x heads) fills the SMs, fewer (at least 32) while it does not
  int cols = dim < 128 ? ((dim + 31) / 32) * 32 : 128;
  while (cols > 32 && (long long)num_requests * heads * ((dim + cols - 1) / cols) < 296) cols /= 2;
  if (cols > 128) cols = 128;
  dim3 grid(num_requests, heads, (dim + cols - 1) / cols);
  const size_t smem = (size_t)kDeltaStage * (5 * ((dim + 3) & ~3) + cols) * sizeof(float);
#define IFX_SCAN(DD)                                                                                              \
  do {                                                                                                            \
    auto kern = delta_scan_kernel<DD>;                                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    kern<<<grid, cols, smem, stream>>>(proj, ld, decay, au, unit, state, slot_stride, cu_seqlens, req_slot, o,    \
                                       heads, dim, cols);                                                         \
  } while (0)
  if (dim <= 16) IFX_SCAN(16);
  else if (dim <= 32) IFX_SCAN(32);
  else if (dim <= 64) IFX_SCAN(64);
  else if (dim <= 128) IFX_SCAN(128);
  else IFX_SCAN(256);
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
