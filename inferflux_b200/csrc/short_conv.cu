// Causal depthwise convolution over time with a few taps, added to its input:
//
//   out[t, c] = h[t, c] + sum_j w[c, j] * h[t - (taps - 1) + j, c]        j = 0 .. taps - 1
//
// (tap taps - 1 multiplies the present input).  Inputs before a request's first
// token are zeros.  The taps - 1 inputs before a step's first token come from the
// request's state, state[slot, i, c] = input at position start - (taps - 1) + i,
// which a new request finds zeroed.  After the step the state holds the last
// taps - 1 inputs again.
//
// Two kernels, because rows of one span read the state that the span's end
// replaces: short_conv_kernel computes every row; short_conv_state_kernel, launched
// after it, moves the state on.  A request that brings a single token has nobody
// else reading its state, so its row moves the state on itself (inline_single), and
// a step of single tokens only needs no second launch.
//
// Products and sums in float32; one thread owns a channel of a row.
//
// Options (ifx_short_conv_ex): the input's rows may be wider than the convolution (in_stride elements from row to row,
// the pointer already at the first convolved column); self_weight 1 adds the input (the form above), 0 gives the
// convolution alone; a bias per channel is added behind the sum; act 1 applies SiLU to the result.
#include "common.cuh"

namespace ifx {

constexpr int kMaxTaps = 16;

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                  long long state_slot_stride, const int* __restrict__ token_req,
                                  const int* __restrict__ req_slot, const int* __restrict__ cu_seqlens,
                                  T* __restrict__ out, int channels, int taps, int inline_single, long long in_stride,
                                  float self_weight, const float* __restrict__ bias, int act) {
  const int t = blockIdx.x;
  const int r = token_req[t];
  const int first = cu_seqlens[r], n = cu_seqlens[r + 1] - first;
  const int i = t - first;                               // index inside the span
  float* st = state ? state + (long long)req_slot[r] * state_slot_stride : nullptr;
  const bool move_on = inline_single && n == 1 && st != nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float* wc = w + (size_t)c * taps;
    const float now = to_f32(h[(size_t)t * in_stride + c]);
    float acc = fmaf(wc[taps - 1], now, now * self_weight);
    float older[kMaxTaps - 1];
#pragma unroll
    for (int k = 1; k < kMaxTaps; ++k) {                 // the input k steps back
      if (k < taps) {
        float v;
        if (k <= i) v = to_f32(h[(size_t)(t - k) * in_stride + c]);
        else v = st[(size_t)((taps - 1) - (k - i)) * channels + c];
        older[k - 1] = v;
        acc = fmaf(wc[taps - 1 - k], v, acc);
      }
    }
    if (bias != nullptr) acc += bias[c];
    if (act == 1) acc = acc / (1.0f + expf(-acc));
    out[(size_t)t * channels + c] = from_f32<T>(acc);
    if (move_on) {                                       // i == 0: older[k - 1] = state[taps - 1 - k]
#pragma unroll
      for (int k = 1; k < kMaxTaps; ++k)
        if (k < taps) st[(size_t)(taps - 1 - k) * channels + c] = (k == 1) ? now : older[k - 2];
    }
  }
}

// The same for up to 4 taps and channel counts that are multiples of 16 bytes' worth of elements: a thread owns
// VEC consecutive channels (one 16-byte load per input row) and, in steps of many tokens, walks up to kConvRows
// consecutive tokens, so that the chain of metadata loads (token -> request -> span and slot) is paid once per
// request a block meets and a token's earlier inputs stay in registers for the next token.
constexpr int kConvRows = 8;

template <typename T> struct ConvVec;
template <> struct ConvVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct ConvVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <typename T>
__global__ void __launch_bounds__(256) short_conv_vec_kernel(
    const T* __restrict__ h, const float* __restrict__ w, float* __restrict__ state, long long state_slot_stride,
    const int* __restrict__ token_req, const int* __restrict__ req_slot, const int* __restrict__ cu_seqlens,
    T* __restrict__ out, int num_tokens, int channels, int taps, int inline_single, int rows_per_block,
    long long in_stride, float self_weight, const float* __restrict__ bias, int act) {
  constexpr int V = ConvVec<T>::N;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c0 >= channels) return;
  float wr[V][4];                                        // wr[v][k]: the tap of the input k steps back
#pragma unroll
  for (int v = 0; v < V; ++v)
#pragma unroll
    for (int k = 0; k < 4; ++k) wr[v][k] = k < taps ? w[(size_t)(c0 + v) * taps + (taps - 1 - k)] : 0.0f;
  const int t_end = min(num_tokens, (int)(blockIdx.x + 1) * rows_per_block);
  int r_at = -1, first = 0, n = 0;
  float* st = nullptr;
  float in[4][V];                                        // in[k]: the input k steps back
  for (int t = blockIdx.x * rows_per_block; t < t_end; ++t) {
    const int r = token_req[t];
    const bool carry = r == r_at;                        // the token before is this request's too: its inputs are in registers
    if (!carry) {
      r_at = r;
      first = cu_seqlens[r];
      n = cu_seqlens[r + 1] - first;
      st = state ? state + (long long)req_slot[r] * state_slot_stride : nullptr;
    }
    const int i = t - first;
    if (carry) {
#pragma unroll
      for (int k = 3; k >= 1; --k)
#pragma unroll
        for (int v = 0; v < V; ++v) in[k][v] = in[k - 1][v];
    }
    ConvVec<T>::load(h + (size_t)t * in_stride + c0, in[0]);
#pragma unroll
    for (int k = 1; k < 4; ++k) {
      if (k < taps && !carry) {
        if (k <= i) {
          ConvVec<T>::load(h + (size_t)(t - k) * in_stride + c0, in[k]);
        } else {
          const float* cell = st + (size_t)((taps - 1) - (k - i)) * channels + c0;
#pragma unroll
          for (int v = 0; v < V; v += 4) {
            const float4 a = *reinterpret_cast<const float4*>(cell + v);
            in[k][v] = a.x; in[k][v + 1] = a.y; in[k][v + 2] = a.z; in[k][v + 3] = a.w;
          }
        }
      }
    }
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      acc[v] = fmaf(wr[v][0], in[0][v], in[0][v] * self_weight);
#pragma unroll
      for (int k = 1; k < 4; ++k)
        if (k < taps) acc[v] = fmaf(wr[v][k], in[k][v], acc[v]);
      if (bias != nullptr) acc[v] += bias[c0 + v];
      if (act == 1) acc[v] = acc[v] / (1.0f + expf(-acc[v]));
    }
    ConvVec<T>::store(out + (size_t)t * channels + c0, acc);
    if (inline_single && n == 1 && st != nullptr) {      // the request's only token: it moves the state on itself
#pragma unroll
      for (int k = 1; k < 4; ++k)
        if (k < taps) {
          float* cell = st + (size_t)(taps - 1 - k) * channels + c0;
#pragma unroll
          for (int v = 0; v < V; v += 4)
            *reinterpret_cast<float4*>(cell + v) = make_float4(in[k - 1][v], in[k - 1][v + 1], in[k - 1][v + 2], in[k - 1][v + 3]);
        }
    }
  }
}

// New state of request r: the last taps - 1 entries of (old state ++ the span's inputs).
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ h, float* __restrict__ state,
                                        long long state_slot_stride, const int* __restrict__ req_slot,
                                        const int* __restrict__ cu_seqlens, int channels, int taps,
                                        int skip_single, long long in_stride) {
  const int r = blockIdx.x;
  const int first = cu_seqlens[r], n = cu_seqlens[r + 1] - first;
  if (skip_single && n == 1) return;
  float* st = state + (long long)req_slot[r] * state_slot_stride;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float next[kMaxTaps - 1];
#pragma unroll
    for (int s = 0; s < kMaxTaps - 1; ++s) {
      if (s < keep) {
        const int m = n + s;                             // index into old state ++ span
        next[s] = m < keep ? st[(size_t)m * channels + c] : to_f32(h[(size_t)(first + m - keep) * in_stride + c]);
      }
    }
#pragma unroll
    for (int s = 0; s < kMaxTaps - 1; ++s)
      if (s < keep) st[(size_t)s * channels + c] = next[s];
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// state: float32 [slots, ..., taps - 1, channels], already offset to this convolution's part of a slot;
// state_slot_stride: floats from one slot to the next.  any_long: some request brings more than one token.
int ifx_short_conv_ex(const void* h, long long in_stride, const float* w, const float* bias, float* state,
                      long long state_slot_stride, const int* token_req, const int* req_slot, const int* cu_seqlens, void* out,
                      int T, int R, int channels, int taps, int any_long, float self_weight, int act, int dtype,
                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if (channels <= 0 || taps <= 0 || R <= 0 || in_stride < channels || act < 0 || act > 1) return IFX_E_BADARG;
  if (taps > kMaxTaps) return IFX_E_TOOBIG;
  if (taps > 1 && state == nullptr) return IFX_E_BADARG;
  const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
  const unsigned gy = (unsigned)((channels + threads - 1) / threads);
  if (gy > 65535u) return IFX_E_TOOBIG;
  dim3 grid((unsigned)T, gy), sgrid((unsigned)R, gy);
  const int vec = dtype == IFX_DT_F32 ? 4 : 8;
  const bool wide = taps <= 4 && channels % vec == 0 && in_stride % vec == 0 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                    (state == nullptr || ((uintptr_t)state % 16 == 0 && state_slot_stride % 4 == 0));
  const int vthreads = channels / vec >= 256 ? 256 : ((channels / vec + 31) / 32) * 32;
  const int rows_per_block = T >= 256 * kConvRows ? kConvRows : (T >= 256 ? T / 256 : 1);
  dim3 vgrid((unsigned)((T + rows_per_block - 1) / rows_per_block), wide ? (unsigned)((channels / vec + vthreads - 1) / vthreads) : 1u);
#define IFX_LAUNCH(TT)                                                                                              \
  do {                                                                                                              \
    if (wide)                                                                                                       \
      short_conv_vec_kernel<TT><<<vgrid, vthreads, 0, stream>>>((const TT*)h, w, state, state_slot_stride,          \
                                                                token_req, req_slot, cu_seqlens, (TT*)out, T,       \
                                                                channels, taps, 1, rows_per_block, in_stride,       \
                                                                self_weight, bias, act);                            \
    else                                                                                                            \
      short_conv_kernel<TT><<<grid, threads, 0, stream>>>((const TT*)h, w, state, state_slot_stride, token_req,     \
                                                           req_slot, cu_seqlens, (TT*)out, channels, taps, 1,       \
                                                           in_stride, self_weight, bias, act);                      \
    if (taps > 1 && any_long)                                                                                       \
      short_conv_state_kernel<TT><<<sgrid, threads, 0, stream>>>((const TT*)h, state, state_slot_stride, req_slot,  \
                                                                 cu_seqlens, channels, taps, 1, in_stride);         \
  } while (0)
  if (dtype == IFX_DT_F32) IFX_LAUNCH(float);
  else if (dtype == IFX_DT_BF16) IFX_LAUNCH(__nv_bfloat16);
  else return IFX_E_DTYPE;
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_short_conv(const void* h, const float* w, float* state, long long state_slot_stride, const int* token_req,
                   const int* req_slot, const int* cu_seqlens, void* out, int T, int R, int channels, int taps,
                   int any_long, int dtype, cudaStream_t stream) {
  return ifx_short_conv_ex(h, channels, w, nullptr, state, state_slot_stride, token_req, req_slot, cu_seqlens, out, T, R,
                           channels, taps, any_long, 1.0f, 0, dtype, stream);
}

}  // extern "C"
