// Kernels of layers whose two sublayers read one norm and add their outputs together, and of a norm over groups.
//
//   groupnorm_stream      x += y / rms(y) * w_post           (optional: y null leaves x alone; x float32, in place)
//                         h  = x / rms_g(x) * w_next         the root mean square taken per group: the row in
//                                                            `groups` equal consecutive parts
//                         h2 = h + conv(h)                   (optional; only in steps whose requests bring one token
//                                                            each: the convolution's earlier inputs are all state)
//                         y may arrive as the float32 partial sums [splits, rows, hidden] of a K-split product
//   residual_add_scaled   x += scale * (a + b), then optionally x in the run's dtype; a and b plain or partial sums
//   gelu_mul_table        out = gelu_tanh(z) * table[token, first_column + j]
//   embed_scaled          out[t] = table[token[t]] * scale in float32
//   scale_f32             v *= factor
//
// One block per row; every reduction is a block's (or, per group, a warp's) reduction of fixed order over a block whose
// size is fixed, so a row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace ifx {

struct TokenConv {
  const float* w;            // [hidden, taps], null: no convolution
  float* state;              // this convolution's [taps - 1, hidden] of slot 0
  long long slot_stride;     // floats from one slot to the next
  const int* token_req;
  const int* req_slot;
  int taps;
};

template <typename TY, typename TO>
__global__ void __launch_bounds__(256) groupnorm_stream_kernel(
    float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ w_post, float eps_post,
    const float* __restrict__ w_next, float eps_next, int groups, TO* __restrict__ out, TO* __restrict__ out2,
    int hidden, int splits, size_t split_stride, TokenConv conv) {
  extern __shared__ float row_s[];                       // the row, kept between the passes; then `groups` scales
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float* xr = x + row * hidden;
  float* scale_s = row_s + hidden;
  if (y != nullptr) {
    const TY* yr = y + row * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = to_f32(yr[i]);
      for (int s = 1; s < splits; ++s) v += to_f32(yr[(size_t)s * split_stride + i]);
      row_s[i] = v;
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r1 = rsqrtf(ss / (float)hidden + eps_post);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = xr[i] + row_s[i] * r1 * w_post[i];
      xr[i] = v;
      row_s[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_s[i] = xr[i];
  }
  if (out == nullptr) return;
  __syncthreads();
  const int gs = hidden / groups;
  if (groups == 1) {
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) ss = fmaf(row_s[i], row_s[i], ss);
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) scale_s[0] = rsqrtf(ss / (float)hidden + eps_next);
  } else {                                               // a warp per group: lane order, then the shuffle tree
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int g = warp; g < groups; g += nwarps) {
      float ss = 0.0f;
      for (int i = lane; i < gs; i += 32) {
        const float v = row_s[g * gs + i];
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) scale_s[g] = rsqrtf(ss / (float)gs + eps_next);
    }
  }
  __syncthreads();
  TO* o = out + row * hidden;
  if (conv.w == nullptr) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<TO>(row_s[i] * scale_s[i / gs] * w_next[i]);
    return;
  }
  // h + conv(h) for a single token: the inputs before it are the state; afterwards the state ends with h
  TO* o2 = out2 + row * hidden;
  const int taps = conv.taps;
  float* st = taps > 1 ? conv.state + (long long)conv.req_slot[conv.token_req[row]] * conv.slot_stride : nullptr;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const TO hr = from_f32<TO>(row_s[i] * scale_s[i / gs] * w_next[i]);
    o[i] = hr;
    const float h = to_f32(hr);                          // the convolution reads h in the run's dtype
    const float* wc = conv.w + (size_t)i * taps;
    float acc = fmaf(wc[taps - 1], h, h);
    float newer = h;
    for (int k = 0; k < taps - 1; ++k) {                 // k + 1 steps back
      float* cell = st + (size_t)(taps - 2 - k) * hidden + i;
      const float old = *cell;
      acc = fmaf(wc[taps - 2 - k], old, acc);
      *cell = newer;
      newer = old;
    }
    o2[i] = from_f32<TO>(acc);
  }
}

// a, b: TA / TB tensors [rows, hidden], or float32 partial sums [splits, rows, hidden] (splits > 1).
template <typename TA, typename TB, typename TO>
__global__ void residual_add_scaled_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_splits,
                                           const TB* __restrict__ b, int b_splits, float scale, TO* __restrict__ out,
                                           size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float d = to_f32(a[i]);
    for (int s = 1; s < a_splits; ++s) d += to_f32(a[(size_t)s * total + i]);
    if (b != nullptr) {
      float e = to_f32(b[i]);
      for (int s = 1; s < b_splits; ++s) e += to_f32(b[(size_t)s * total + i]);
      d += e;
    }
    const float v = fmaf(scale, d, x[i]);
    x[i] = v;
    if (out != nullptr) out[i] = from_f32<TO>(v);
  }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gelu_mul_table_kernel(const T* __restrict__ z, const T* __restrict__ table, const int* __restrict__ tokens,
                                      int ld_table, int first_column, int vocab, T* __restrict__ out, int rows, int dim) {
  const long long n = (long long)rows * dim;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / dim), j = (int)(i % dim);
    const int id = tokens[t];
    const float e = (id >= 0 && id < vocab) ? to_f32(table[(size_t)id * ld_table + first_column + j]) : 0.0f;
    out[i] = from_f32<T>(gelu_tanh_f(to_f32(z[i])) * e);
  }
}

template <typename T>
__global__ void embed_scaled_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ out,
                                    int hidden, int vocab, float scale) {
  const int t = blockIdx.x;
  const int id = tokens[t];
  float* o = out + (size_t)t * hidden;
  const bool ok = id >= 0 && id < vocab;                 // the host refuses other ids before launch
  const T* row = table + (size_t)(ok ? id : 0) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_f32(row[i]) * scale : 0.0f;
}

__global__ void scale_f32_kernel(float* __restrict__ v, long long n, float factor) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    v[i] *= factor;
}

inline unsigned elem_grid(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  return (unsigned)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// y null: x is left as it is.  out null: the sum alone.  conv_w non-null (with out and out2; only for steps in which every
// request brings one token): out2 = out + conv(out) over time, `conv_state` (this convolution's part of slot 0, slots
// conv_slot_stride floats apart) read and moved on.  splits > 1: y is float32 [splits, T, hidden].
int ifx_groupnorm_stream(float* x, const void* y, const float* w_post, float eps_post, const float* w_next, float eps_next,
                         int groups, void* out, void* out2, int T, int hidden, int y_dtype, int out_dtype, int splits,
                         const float* conv_w, int taps, float* conv_state, long long conv_slot_stride,
                         const int* token_req, const int* req_slot, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden <= 0 || groups <= 0 || hidden % groups || splits < 1 || (y != nullptr && splits > 1 && y_dtype != IFX_DT_F32))
    return IFX_E_BADARG;
  if (y != nullptr && w_post == nullptr) return IFX_E_BADARG;
  if (out != nullptr && w_next == nullptr) return IFX_E_BADARG;
  if (conv_w != nullptr && (out == nullptr || out2 == nullptr || taps < 1 || taps > 16 || (taps > 1 && conv_state == nullptr) ||
                            token_req == nullptr || req_slot == nullptr))
    return IFX_E_BADARG;
  TokenConv conv = {conv_w, conv_state, conv_slot_stride, token_req, req_slot, taps};
  const size_t smem = (size_t)(hidden + groups) * sizeof(float);
  if (smem > 200 * 1024) return IFX_E_TOOBIG;
  const size_t split_stride = (size_t)T * hidden;
#define IFX_LAUNCH(TY, TO)                                                                                          \
  do {                                                                                                              \
    auto kern = groupnorm_stream_kernel<TY, TO>;                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    kern<<<T, 256, smem, stream>>>(x, (const TY*)y, w_post, eps_post, w_next, eps_next, groups, (TO*)out, (TO*)out2, \
                                   hidden, splits, split_stride, conv);                                             \
  } while (0)
  const int yd = y == nullptr ? IFX_DT_F32 : y_dtype;
  const int od = out == nullptr ? IFX_DT_F32 : out_dtype;
  if (yd == IFX_DT_F32 && od == IFX_DT_F32) IFX_LAUNCH(float, float);
  else if (yd == IFX_DT_BF16 && od == IFX_DT_BF16) IFX_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (yd == IFX_DT_F32 && od == IFX_DT_BF16) IFX_LAUNCH(float, __nv_bfloat16);
  else if (yd == IFX_DT_BF16 && od == IFX_DT_F32) IFX_LAUNCH(__nv_bfloat16, float);
  else return IFX_E_DTYPE;
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  return 0;
}

// a_splits / b_splits > 1: that operand is float32 partial sums whatever its dtype code says.  b may be null.
int ifx_residual_add_scaled(float* x, const void* a, int a_dtype, int a_splits, const void* b, int b_dtype, int b_splits,
                            float scale, void* out, int out_dtype, int T, int hidden, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden <= 0 || a == nullptr || a_splits < 1 || b_splits < 1) return IFX_E_BADARG;
  if (a_splits > 1) a_dtype = IFX_DT_F32;
  if (b_splits > 1 || b == nullptr) b_dtype = b == nullptr ? a_dtype : IFX_DT_F32;
  const size_t total = (size_t)T * hidden;
  const unsigned grid = elem_grid((long long)total, 256);
  const int od = out == nullptr ? IFX_DT_F32 : out_dtype;
#define IFX_LAUNCH(TA, TB, TO)                                                                                     \
  residual_add_scaled_kernel<TA, TB, TO><<<grid, 256, 0, stream>>>(x, (const TA*)a, a_splits, (const TB*)b, b_splits, \
                                                                  scale, (TO*)out, total)
#define IFX_BY_OUT(TA, TB)                                         \
  do {                                                             \
    if (od == IFX_DT_F32) IFX_LAUNCH(TA, TB, float);               \
    else if (od == IFX_DT_BF16) IFX_LAUNCH(TA, TB, __nv_bfloat16); \
    else return IFX_E_DTYPE;                                       \
  } while (0)
  if (a_dtype == IFX_DT_F32 && b_dtype == IFX_DT_F32) IFX_BY_OUT(float, float);
  else if (a_dtype == IFX_DT_F32 && b_dtype == IFX_DT_BF16) IFX_BY_OUT(float, __nv_bfloat16);
  else if (a_dtype == IFX_DT_BF16 && b_dtype == IFX_DT_F32) IFX_BY_OUT(__nv_bfloat16, float);
  else if (a_dtype == IFX_DT_BF16 && b_dtype == IFX_DT_BF16) IFX_BY_OUT(__nv_bfloat16, __nv_bfloat16);
  else return IFX_E_DTYPE;
#undef IFX_BY_OUT
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_gelu_mul_table(const void* z, const void* table, const int* tokens, int ld_table, int first_column, int vocab,
                       void* out, int T, int dim, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dim <= 0 || first_column < 0 || first_column + dim > ld_table || vocab <= 0) return IFX_E_BADARG;
  const unsigned grid = elem_grid((long long)T * dim, 256);
  if (dtype == IFX_DT_F32)
    gelu_mul_table_kernel<float><<<grid, 256, 0, stream>>>((const float*)z, (const float*)table, tokens, ld_table,
                                                           first_column, vocab, (float*)out, T, dim);
  else if (dtype == IFX_DT_BF16)
    gelu_mul_table_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)z, (const __nv_bfloat16*)table,
                                                                   tokens, ld_table, first_column, vocab,
                                                                   (__nv_bfloat16*)out, T, dim);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_embed_scaled(const void* table, const int* tokens, float* out, int num_tokens, int hidden, int vocab, float scale,
                     int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return IFX_E_BADARG;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == IFX_DT_F32)
    embed_scaled_kernel<float><<<num_tokens, threads, 0, stream>>>((const float*)table, tokens, out, hidden, vocab, scale);
  else if (dtype == IFX_DT_BF16)
    embed_scaled_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, tokens, out, hidden,
                                                                           vocab, scale);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_scale_f32(float* v, long long n, float factor, cudaStream_t stream) {
  if (n <= 0) return 0;
  scale_f32_kernel<<<elem_grid(n, 256), 256, 0, stream>>>(v, n, factor);
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
