// A scan with a matrix of state per (request, head) that every token decays and writes to:
//
//   S <- diag(w_t) S + k_t v_t^T        S: [key channel, value channel], float32
//   o_t = S^T (q_scale q_t)             of the new S        (+ skip[h] v_t)
//
// q and k hold `groups` heads of dk channels; head h reads group h / (heads / groups).  v holds `heads` heads of dv.
// The decay comes from raw inputs, turned into w inside the kernel, in float32:
//
//   DECAY_CHANNEL   raw [T, heads dk]:  w = sigmoid(raw)^(1 / tau) = exp(logsigmoid(raw) / tau), one per key channel
//   DECAY_STEP      raw [T, heads]:     dt = softplus(raw + step_bias[h]);  w = exp(-exp(log_rate[h]) dt) for the
//                                       whole head;  k_t is multiplied by dt
//
// All inputs are float32 rows that may be wider than what is read (row strides in elements, pointers already at the
// first column).  The state lives in a slot per request, [head, value channel, key channel] (a column of S is
// contiguous), state_slot_stride floats from slot to slot; a new request finds it zeroed.
//
// Work split: grid (request, head, slice of value channels).  A value channel j is a column of S; KS neighbouring
// lanes share it, lane s keeping key channels s R ... s R + R - 1 in registers.  Per token a lane
// does R multiply-adds for the update and R for the read-out, and the KS partial sums meet through shuffles.  A
// stretch of tokens' q, k, raw decay and v arrives in shared memory by cp.async, one stretch ahead of the one being
// worked on (the exponentials are taken there, once per token and channel).  Every sum's order depends on (dk, R, KS)
// only, never on how the tokens were cut into steps or which other requests are in the batch.
#include "common.cuh"

namespace ifx {

enum { DECAY_CHANNEL = 0, DECAY_STEP = 1 };

struct DecayScanArgs {
  const float* q; long long q_stride;
  const float* k; long long k_stride;
  const float* v; long long v_stride;
  const float* raw; long long raw_stride;
  float* state; long long state_slot_stride;
  const int* req_slot; const int* cu_seqlens;
  float* out;                                  // [T, heads dv]
  const float* step_bias; const float* log_rate; const float* skip;     // per head, DECAY_STEP (skip: either mode)
  int heads, groups, dk, dv;
  int ks, cols, chunk;                         // lanes per column, columns per block, staged tokens
  float inv_tau, q_scale;
  // ready: `raw` already holds the decays (DECAY_CHANNEL: [T, heads dk]; DECAY_STEP: [T, 2 heads], a head's decays in
  // front, its step sizes behind), made by decay_prepare_kernel for steps with long spans
  int ready;
  int vec;                                     // rows, strides and sizes allow copies of four floats at a time
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

__device__ __forceinline__ void cp_async_f32(float* dst_shared, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_shared);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_f32x4(float* dst_shared, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_shared);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One stretch of staged tokens: [CH][ROW] q, [CH][ROW] k, the decay's raw input ([CH][ROW], or [CH] and room for [CH]
// decays), [CH][CB] v.  Two such buffers take turns: while one is worked on, the next stretch's rows arrive in the other
// by cp.async; what has to be made of the raw numbers (the exponentials, q's scale, k's step) is made in place, once per
// token and channel, when a buffer's turn comes.  A lane's R key channels lie side by side and are read four at a time;
// four floats of padding behind every 32 keep the KS lanes of a column on banks of their own.
__device__ __forceinline__ int padded(int c) { return c + ((c >> 5) << 2); }

template <int R, int MODE>
__global__ void __launch_bounds__(256) decay_scan_kernel(const DecayScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  static_assert(R % 4 == 0, "a lane reads its key channels four at a time");
  const int r = blockIdx.x, h = blockIdx.y;
  const int KS = a.ks, CB = a.cols, CH = a.chunk;
  const int DKP = R * KS;                                    // key channels, padded to the lanes (a power of two)
  const int lg = 31 - __clz(DKP);
  const int ROW = padded(DKP);                               // floats from one token's row to the next
  const size_t w_floats = MODE == DECAY_CHANNEL ? (size_t)CH * ROW : (size_t)2 * CH;
  const size_t buf_floats = ((size_t)2 * CH * ROW + w_floats + (size_t)CH * CB + 3) / 4 * 4;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int s = tid % KS, jl = tid / KS;
  const int j = blockIdx.z * CB + jl;
  const bool live = jl < CB && j < a.dv;
  const int dk = a.dk, dv = a.dv;
  const int g = h / (a.heads / a.groups);
  const int first = a.cu_seqlens[r], n = a.cu_seqlens[r + 1] - first;
  float* st = a.state + (long long)a.req_slot[r] * a.state_slot_stride + ((size_t)h * dv + (live ? j : 0)) * dk;
  const int c0 = s * R;                                      // this lane's first key channel

  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (live && c0 + i < dk) ? st[c0 + i] : 0.0f;
  const float skip = a.skip ? a.skip[h] : 0.0f;
  const float rate = MODE == DECAY_STEP ? expf(a.log_rate[h]) : 0.0f;
  const float sbias = MODE == DECAY_STEP ? a.step_bias[h] : 0.0f;

  auto fetch = [&](int t0, float* buf) {                     // the raw rows of tokens t0 .. t0 + m - 1 on their way
    const int m = min(CH, n - t0);
    float* sq = buf;
    float* sk = sq + (size_t)CH * ROW;
    float* sw = sk + (size_t)CH * ROW;
    float* sv = sw + w_floats;
    if (a.vec) {
      for (int e = tid * 4; e < (m << lg); e += nthreads * 4) {
        const int tt = e >> lg, c = e & (DKP - 1);
        const size_t t = (size_t)(first + t0 + tt);
        const int at = tt * ROW + padded(c);
        if (c < dk) {
          cp_async_f32x4(sq + at, a.q + t * a.q_stride + (size_t)g * dk + c);
          cp_async_f32x4(sk + at, a.k + t * a.k_stride + (size_t)g * dk + c);
          if (MODE == DECAY_CHANNEL) cp_async_f32x4(sw + at, a.raw + t * a.raw_stride + (size_t)h * dk + c);
        }
      }
    } else {
      for (int e = tid; e < (m << lg); e += nthreads) {
        const int tt = e >> lg, c = e & (DKP - 1);
        const size_t t = (size_t)(first + t0 + tt);
        const int at = tt * ROW + padded(c);
        if (c < dk) {
          cp_async_f32(sq + at, a.q + t * a.q_stride + (size_t)g * dk + c);
          cp_async_f32(sk + at, a.k + t * a.k_stride + (size_t)g * dk + c);
          if (MODE == DECAY_CHANNEL) cp_async_f32(sw + at, a.raw + t * a.raw_stride + (size_t)h * dk + c);
        }
      }
    }
    if (MODE == DECAY_STEP)
      for (int tt = tid; tt < m; tt += nthreads) {
        cp_async_f32(sw + tt, a.raw + (size_t)(first + t0 + tt) * a.raw_stride + h);
        if (a.ready) cp_async_f32(sw + CH + tt, a.raw + (size_t)(first + t0 + tt) * a.raw_stride + a.heads + h);
      }
    for (int e = tid; e < m * CB; e += nthreads) {
      const int tt = e / CB, c = e % CB;
      const int col = blockIdx.z * CB + c;
      if (col < dv) cp_async_f32(sv + e, a.v + (size_t)(first + t0 + tt) * a.v_stride + (size_t)h * dv + col);
    }
    cp_async_commit();
  };

  if (n > 0) fetch(0, smem);
  int turn = 0;
  for (int t0 = 0; t0 < n; t0 += CH, turn ^= 1) {
    const int m = min(CH, n - t0);
    float* buf = smem + (size_t)turn * buf_floats;
    float* sq = buf;
    float* sk = sq + (size_t)CH * ROW;
    float* sw = sk + (size_t)CH * ROW;
    float* sv = sw + w_floats;
    cp_async_wait_all();
    __syncthreads();                                         // this stretch has arrived; the one before has been read
    if (t0 + CH < n) fetch(t0 + CH, smem + (size_t)(turn ^ 1) * buf_floats);
    if (MODE == DECAY_STEP && !a.ready) {
      for (int tt = tid; tt < m; tt += nthreads) {
        const float dt = softplus(sw[tt] + sbias);
        sw[tt] = expf(-rate * dt);
        sw[CH + tt] = dt;
      }
      __syncthreads();
    }
    for (int e = tid; e < (m << lg); e += nthreads) {
      const int tt = e >> lg, c = e & (DKP - 1);
      const int at = tt * ROW + padded(c);
      if (c < dk) {
        sq[at] *= a.q_scale;
        if (MODE == DECAY_CHANNEL) {
          if (!a.ready) sw[at] = expf(log_sigmoid(sw[at]) * a.inv_tau);
        } else {
          sk[at] *= sw[CH + tt];
        }
      } else {                                               // padding: nothing is written, nothing is read out
        sq[at] = 0.0f;
        sk[at] = 0.0f;
        if (MODE == DECAY_CHANNEL) sw[at] = 1.0f;
      }
    }
    __syncthreads();
    const int lane_at = padded(c0);
    // Every thread walks the stretch (whole warps meet in the shuffles), U tokens at a time: their loads, their read-out
    // sums and their shuffles are independent of one another (only S passes from token to token, one multiply-add
    // each), so one token's latencies hide behind the others' work.
    constexpr int U = 4;
    for (int tt = 0; tt < m; tt += U) {
      const int cnt = min(U, m - tt);
      float vv[U], acc[U], wall[U];
      int rowat[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int tu = tt + min(u, cnt - 1);
        vv[u] = (live && u < cnt) ? sv[tu * CB + jl] : 0.0f;
        wall[u] = MODE == DECAY_STEP ? sw[tu] : 0.0f;
        rowat[u] = tu * ROW + lane_at;
        acc[u] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        float4 qv[U], kv[U], wv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          qv[u] = *reinterpret_cast<const float4*>(sq + rowat[u] + i);
          kv[u] = *reinterpret_cast<const float4*>(sk + rowat[u] + i);
          if (MODE == DECAY_CHANNEL) wv[u] = *reinterpret_cast<const float4*>(sw + rowat[u] + i);
          else wv[u] = make_float4(wall[u], wall[u], wall[u], wall[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (u < cnt) {
            S[i] = fmaf(wv[u].x, S[i], kv[u].x * vv[u]);
            S[i + 1] = fmaf(wv[u].y, S[i + 1], kv[u].y * vv[u]);
            S[i + 2] = fmaf(wv[u].z, S[i + 2], kv[u].z * vv[u]);
            S[i + 3] = fmaf(wv[u].w, S[i + 3], kv[u].w * vv[u]);
            acc[u] = fmaf(S[i], qv[u].x, acc[u]);
            acc[u] = fmaf(S[i + 1], qv[u].y, acc[u]);
            acc[u] = fmaf(S[i + 2], qv[u].z, acc[u]);
            acc[u] = fmaf(S[i + 3], qv[u].w, acc[u]);
          }
        }
      }
      for (int o = KS >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < U; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
      }
      if (s == 0 && live) {
        float* o0 = a.out + (size_t)(first + t0 + tt) * ((size_t)a.heads * dv) + (size_t)h * dv + j;
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (u < cnt) o0[(size_t)u * a.heads * dv] = fmaf(skip, vv[u], acc[u]);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (c0 + i < dk) st[c0 + i] = S[i];
  }
}

// The decays of a whole step ahead of the scan, for steps with long spans: every SM takes part, and the scan's blocks,
// which then stage ready numbers, can be small and many.
__global__ void decay_prepare_kernel(const float* __restrict__ raw, long long raw_stride, float* __restrict__ out, int T,
                                     int per_row, int heads, int mode, float inv_tau, const float* __restrict__ step_bias,
                                     const float* __restrict__ log_rate) {
  const size_t total = (size_t)T * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row;
    const int c = (int)(i % per_row);
    const float x = raw[t * raw_stride + c];
    if (mode == DECAY_CHANNEL) {
      out[i] = expf(log_sigmoid(x) * inv_tau);
    } else {                                                 // per_row = heads: the decay in front, the step behind
      const float dt = softplus(x + step_bias[c]);
      out[t * 2 * heads + c] = expf(-expf(log_rate[c]) * dt);
      out[t * 2 * heads + heads + c] = dt;
    }
  }
}

template <int MODE>
static int launch_decay_scan(const DecayScanArgs& a, int R, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
#define IFX_SCAN(RR)                                                                                          \
  do {                                                                                                        \
    auto kern = decay_scan_kernel<RR, MODE>;                                                                  \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    kern<<<grid, threads, smem, stream>>>(a);                                                                 \
  } while (0)
  switch (R) {
    case 4: IFX_SCAN(4); break;
    case 8: IFX_SCAN(8); break;
    case 16: IFX_SCAN(16); break;
    default: return IFX_E_BADARG;
  }
#undef IFX_SCAN
  return 0;
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// How the kernel splits dk key channels: R per lane (4, 8 or 16) times KS lanes (a power of two up to 32), the pair
// with the least padding, 8 before 4 before 16 on a tie.  dk <= 512.
int ifx_decay_scan_split(int dk, int* R_out, int* KS_out) {
  if (dk <= 0 || dk > 512) return IFX_E_TOOBIG;
  const int Rs[3] = {8, 4, 16};
  int best_R = 0, best_KS = 0, best_pad = 1 << 30;
  for (int i = 0; i < 3; ++i) {
    int ks = 1;
    while (ks * Rs[i] < dk) ks *= 2;
    if (ks > 32) continue;
    const int pad = ks * Rs[i] - dk;
    if (pad < best_pad) { best_pad = pad; best_R = Rs[i]; best_KS = ks; }
  }
  if (best_R == 0) return IFX_E_TOOBIG;
  *R_out = best_R;
  *KS_out = best_KS;
  return 0;
}

// mode 0: a decay per key channel (raw [T, heads dk], tau); mode 1: a decay per head from a step size (raw [T, heads],
// step_bias, log_rate per head; k is multiplied by the step).  skip (per head, may be null): out += skip v.
// blocks_wanted: how many blocks the caller would like at least (the SMs to fill); value channels are cut over more
// blocks while there are fewer.
// scratch (may be null): room for the step's decays, num_tokens * heads * dk floats (mode 0) or num_tokens * 2 heads
// (mode 1); with it, steps with long spans make their decays in a pass of their own over all SMs.
int ifx_decay_scan(const float* q, long long q_stride, const float* k, long long k_stride, const float* v, long long v_stride,
                   const float* raw, long long raw_stride, float* state, long long state_slot_stride, const int* req_slot,
                   const int* cu_seqlens, float* out, const float* step_bias, const float* log_rate, const float* skip,
                   int num_requests, int num_tokens, int max_span, int heads, int groups, int dk, int dv, int mode, float tau,
                   float q_scale, int blocks_wanted, float* scratch, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || dk <= 0 || dv <= 0 || (mode != 0 && mode != 1) || max_span <= 0)
    return IFX_E_BADARG;
  if (mode == 0 && !(tau > 0.0f)) return IFX_E_BADARG;
  if (mode == 1 && (step_bias == nullptr || log_rate == nullptr)) return IFX_E_BADARG;
  if (heads > 65535) return IFX_E_TOOBIG;
  int R = 0, KS = 0;
  const int rc = ifx_decay_scan_split(dk, &R, &KS);
  if (rc) return rc;
  // Columns a block holds: 256 threads' worth (with more, a token's instructions queue up on the SM's four schedulers; with
  // fewer, every block stages the same keys again for little work), fewer only for spans of one token, where staging is
  // nothing and more blocks bring the states in sooner.
  int cols = 256 / KS;
  if (cols > dv) cols = dv;
  const bool ready = scratch != nullptr && max_span >= 64;
  if (ready) {
    const int per_row = mode == 0 ? heads * dk : heads;
    const size_t total = (size_t)num_tokens * per_row;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
    decay_prepare_kernel<<<blocks, 256, 0, stream>>>(raw, raw_stride, scratch, num_tokens, per_row, heads, mode,
                                                    mode == 0 ? 1.0f / tau : 0.0f, step_bias, log_rate);
    raw = scratch;
    raw_stride = mode == 0 ? per_row : 2 * heads;
  }
  if (max_span == 1)
    while (cols > 8 && (long long)num_requests * heads * ((dv + cols - 1) / cols) < blocks_wanted) cols = (cols + 1) / 2;
  else if (ready)                                            // ready decays: blocks of four warps, while SMs are left
    while (cols * KS > 128 && (long long)num_requests * heads * ((dv + cols - 1) / cols) < 148) cols = (cols + 1) / 2;
  const int zsplits = (dv + cols - 1) / cols;
  if (zsplits > 65535) return IFX_E_TOOBIG;
  int threads = ((cols * KS + 31) / 32) * 32;
  const int DKP = R * KS;
  const int ROW = DKP + ((DKP >> 5) << 2);                   // four floats of padding behind every 32
  const size_t per_token = ((size_t)(mode == 0 ? 3 : 2) * ROW + cols) * sizeof(float);
  int chunk = (int)((48 * 1024 - 64) / (2 * (per_token + 8)));          // two buffers
  if (chunk > 16) chunk = 16;
  if (chunk > max_span) chunk = max_span;
  if (chunk < 1) chunk = 1;
  const size_t buf_floats = ((size_t)chunk * per_token / sizeof(float) + (mode == 1 ? (size_t)2 * chunk : 0) + 3) / 4 * 4;
  const size_t smem = 2 * buf_floats * sizeof(float);
  DecayScanArgs a;
  a.q = q; a.q_stride = q_stride; a.k = k; a.k_stride = k_stride; a.v = v; a.v_stride = v_stride;
  a.raw = raw; a.raw_stride = raw_stride; a.state = state; a.state_slot_stride = state_slot_stride;
  a.req_slot = req_slot; a.cu_seqlens = cu_seqlens; a.out = out; a.step_bias = step_bias; a.log_rate = log_rate;
  a.skip = skip; a.heads = heads; a.groups = groups; a.dk = dk; a.dv = dv; a.ks = KS; a.cols = cols; a.chunk = chunk;
  a.inv_tau = mode == 0 ? 1.0f / tau : 0.0f;
  a.q_scale = q_scale;
  a.ready = ready ? 1 : 0;
  auto by16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  a.vec = (dk % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && (mode == 1 || raw_stride % 4 == 0) && by16(q) && by16(k) &&
           (mode == 1 || by16(raw))) ? 1 : 0;
  dim3 grid((unsigned)num_requests, (unsigned)heads, (unsigned)zsplits);
  const int lrc = mode == 0 ? launch_decay_scan<DECAY_CHANNEL>(a, R, grid, threads, smem, stream)
                            : launch_decay_scan<DECAY_STEP>(a, R, grid, threads, smem, stream);
  if (lrc) return lrc;
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
