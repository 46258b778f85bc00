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
// lanes share it, lane s keeping key channels s, s + KS, s + 2 KS, ... (R of them) in registers.  Per token a lane
// does R multiply-adds for the update and R for the read-out, and the KS partial sums meet through shuffles.  A
// stretch of tokens' q, k, w and v is staged in shared memory by the whole block (the exponentials are taken there,
// once per token and channel).  Every sum's order depends on (dk, R, KS) only, never on how the tokens were cut
// into steps or which other requests are in the batch.
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
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

template <int R, int MODE>
__global__ void __launch_bounds__(512) decay_scan_kernel(const DecayScanArgs a) {
  extern __shared__ float smem[];
  const int r = blockIdx.x, h = blockIdx.y;
  const int KS = a.ks, CB = a.cols, CH = a.chunk;
  const int DKP = R * KS;                                    // key channels, padded
  float* sq = smem;                                          // [CH][DKP]
  float* sk = sq + (size_t)CH * DKP;                         // [CH][DKP]
  float* sw = sk + (size_t)CH * DKP;                         // DECAY_CHANNEL: [CH][DKP]; DECAY_STEP: [CH] w, then [CH] dt
  float* sv = sw + (MODE == DECAY_CHANNEL ? (size_t)CH * DKP : (size_t)2 * CH);   // [CH][CB]
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int s = tid % KS, jl = tid / KS;
  const int j = blockIdx.z * CB + jl;
  const bool live = jl < CB && j < a.dv;
  const int dk = a.dk, dv = a.dv;
  const int g = h / (a.heads / a.groups);
  const int first = a.cu_seqlens[r], n = a.cu_seqlens[r + 1] - first;
  float* st = a.state + (long long)a.req_slot[r] * a.state_slot_stride + ((size_t)h * dv + (live ? j : 0)) * dk;

  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int c = i * KS + s;
    S[i] = (live && c < dk) ? st[c] : 0.0f;
  }
  const float skip = a.skip ? a.skip[h] : 0.0f;
  const float rate = MODE == DECAY_STEP ? expf(a.log_rate[h]) : 0.0f;
  const float sbias = MODE == DECAY_STEP ? a.step_bias[h] : 0.0f;

  for (int t0 = 0; t0 < n; t0 += CH) {
    const int m = min(CH, n - t0);
    __syncthreads();                                         // the stretch before has been read
    if (MODE == DECAY_STEP) {
      for (int tt = tid; tt < m; tt += nthreads) {
        const float dt = softplus(a.raw[(size_t)(first + t0 + tt) * a.raw_stride + h] + sbias);
        sw[tt] = expf(-rate * dt);
        sw[CH + tt] = dt;
      }
      __syncthreads();
    }
    for (int e = tid; e < m * DKP; e += nthreads) {
      const int tt = e / DKP, c = e % DKP;
      const size_t t = (size_t)(first + t0 + tt);
      float qv = 0.0f, kv = 0.0f, wv = 1.0f;
      if (c < dk) {
        qv = a.q[t * a.q_stride + (size_t)g * dk + c] * a.q_scale;
        kv = a.k[t * a.k_stride + (size_t)g * dk + c];
        if (MODE == DECAY_CHANNEL) wv = expf(log_sigmoid(a.raw[t * a.raw_stride + (size_t)h * dk + c]) * a.inv_tau);
        else kv *= sw[CH + tt];
      }
      sq[e] = qv;
      sk[e] = kv;
      if (MODE == DECAY_CHANNEL) sw[e] = wv;
    }
    for (int e = tid; e < m * CB; e += nthreads) {
      const int tt = e / CB, c = e % CB;
      const int col = blockIdx.z * CB + c;
      sv[e] = col < dv ? a.v[(size_t)(first + t0 + tt) * a.v_stride + (size_t)h * dv + col] : 0.0f;
    }
    __syncthreads();
    {                                                        // every thread walks the stretch: whole warps meet in the shuffles
      for (int tt = 0; tt < m; ++tt) {
        const float vj = jl < CB ? sv[tt * CB + jl] : 0.0f;
        const float* qrow = sq + (size_t)tt * DKP + s;
        const float* krow = sk + (size_t)tt * DKP + s;
        const float* wrow = sw + (size_t)tt * DKP + s;
        const float w_all = MODE == DECAY_STEP ? sw[tt] : 0.0f;
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const float w = MODE == DECAY_STEP ? w_all : wrow[i * KS];
          S[i] = fmaf(w, S[i], krow[i * KS] * vj);
          acc = fmaf(S[i], qrow[i * KS], acc);
        }
        for (int o = KS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (s == 0 && live) a.out[(size_t)(first + t0 + tt) * ((size_t)a.heads * dv) + (size_t)h * dv + j] = fmaf(skip, vj, acc);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int c = i * KS + s;
      if (c < dk) st[c] = S[i];
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
    case 2: IFX_SCAN(2); break;
    case 4: IFX_SCAN(4); break;
    case 6: IFX_SCAN(6); break;
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

// How the kernel splits dk key channels: R per lane (2, 4, 6, 8 or 16) times KS lanes (a power of two up to 32),
// the pair with the least padding, the larger R on a tie from 8 down.  dk <= 512.
int ifx_decay_scan_split(int dk, int* R_out, int* KS_out) {
  if (dk <= 0 || dk > 512) return IFX_E_TOOBIG;
  const int Rs[5] = {8, 6, 4, 16, 2};
  int best_R = 0, best_KS = 0, best_pad = 1 << 30;
  for (int i = 0; i < 5; ++i) {
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
int ifx_decay_scan(const float* q, long long q_stride, const float* k, long long k_stride, const float* v, long long v_stride,
                   const float* raw, long long raw_stride, float* state, long long state_slot_stride, const int* req_slot,
                   const int* cu_seqlens, float* out, const float* step_bias, const float* log_rate, const float* skip,
                   int num_requests, int max_span, int heads, int groups, int dk, int dv, int mode, float tau, float q_scale,
                   int blocks_wanted, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || dk <= 0 || dv <= 0 || (mode != 0 && mode != 1) || max_span <= 0)
    return IFX_E_BADARG;
  if (mode == 0 && !(tau > 0.0f)) return IFX_E_BADARG;
  if (mode == 1 && (step_bias == nullptr || log_rate == nullptr)) return IFX_E_BADARG;
  if (heads > 65535) return IFX_E_TOOBIG;
  int R = 0, KS = 0;
  const int rc = ifx_decay_scan_split(dk, &R, &KS);
  if (rc) return rc;
  int cols = 512 / KS;                                      // columns a block of 512 threads holds
  if (cols > dv) cols = dv;
  while (cols > 8 && (long long)num_requests * heads * ((dv + cols - 1) / cols) < blocks_wanted) cols = (cols + 1) / 2;
  const int zsplits = (dv + cols - 1) / cols;
  if (zsplits > 65535) return IFX_E_TOOBIG;
  int threads = ((cols * KS + 31) / 32) * 32;
  const int DKP = R * KS;
  const size_t per_token = ((size_t)(mode == 0 ? 3 : 2) * DKP + cols) * sizeof(float);
  int chunk = (int)((40 * 1024) / per_token);
  if (chunk > 16) chunk = 16;
  if (chunk > max_span) chunk = max_span;
  if (chunk < 1) chunk = 1;
  const size_t smem = (size_t)chunk * per_token + (mode == 1 ? (size_t)2 * chunk * sizeof(float) : 0);
  DecayScanArgs a;
  a.q = q; a.q_stride = q_stride; a.k = k; a.k_stride = k_stride; a.v = v; a.v_stride = v_stride;
  a.raw = raw; a.raw_stride = raw_stride; a.state = state; a.state_slot_stride = state_slot_stride;
  a.req_slot = req_slot; a.cu_seqlens = cu_seqlens; a.out = out; a.step_bias = step_bias; a.log_rate = log_rate;
  a.skip = skip; a.heads = heads; a.groups = groups; a.dk = dk; a.dv = dv; a.ks = KS; a.cols = cols; a.chunk = chunk;
  a.inv_tau = mode == 0 ? 1.0f / tau : 0.0f;
  a.q_scale = q_scale;
  dim3 grid((unsigned)num_requests, (unsigned)heads, (unsigned)zsplits);
  const int lrc = mode == 0 ? launch_decay_scan<DECAY_CHANNEL>(a, R, grid, threads, smem, stream)
                            : launch_decay_scan<DECAY_STEP>(a, R, grid, threads, smem, stream);
  if (lrc) return lrc;
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
