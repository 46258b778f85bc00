// Small kernels around a pair of mixers that read the same rows and a block that adds both sublayers at once.
//
//   bigram_add            x[t] += table[(token before * a + token * b) mod buckets], the table's last row at position 0;
//                         the token before a span's first one is the request's state, which takes the span's last token
//   rmsnorm_pair          two RMS norms of the same float32 rows (one sum of squares, two weights)
//   gate_mul              a * sigmoid(g) or a * silu(g)
//   gated_groupnorm       rows in equal parts, each over its own root mean square, times a weight and silu(gate), the
//                         gate in front of the norm or behind it
//   pair_combine          c_a a + c_b b, or c_a a / rms(a) * w_a + c_b b / rms(b) * w_b; the result is float32
//   residual_add_vectors  x += s_a * a + s_b * (b + b2), vectors along the row
//
// Norms, sums and gates are float32 whatever the dtype of what comes in or goes out.
#include "common.cuh"

namespace ifx {

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == IFX_DT_F32 ? static_cast<const float*>(p)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
  if (dtype == IFX_DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

template <typename T>
__global__ void bigram_add_kernel(float* __restrict__ x, const T* __restrict__ table, const int* __restrict__ tokens,
                                  const int* __restrict__ positions, const int* __restrict__ token_req,
                                  const int* __restrict__ req_slot, const int* __restrict__ cu_seqlens,
                                  int* __restrict__ state, long long state_slot_stride, int hidden, int vocab,
                                  long long mul_prev, long long mul_cur, int buckets) {
  __shared__ int row_s;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    const int r = token_req[t];
    const int first = cu_seqlens[r], last = cu_seqlens[r + 1] - 1;
    int* st = state + (long long)req_slot[r] * state_slot_stride;
    const int tok = tokens[t];
    const int before = t > first ? tokens[t - 1] : st[0];
    // only the block of a span's first token reads the state, and it reads before it writes
    if (t == first) st[0] = tokens[last];
    int row = -1;
    if (tok >= 0 && tok < vocab) {
      if (positions[t] == 0) row = buckets;
      else if (before >= 0 && before < vocab) row = (int)(((long long)before * mul_prev + (long long)tok * mul_cur) % buckets);
    }
    row_s = row;
  }
  __syncthreads();
  const int row = row_s;
  if (row < 0) return;                                     // an id outside the vocabulary adds nothing
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    x[(size_t)t * hidden + c] += to_f32(table[(size_t)row * hidden + c]);
}

// With `a`: the row first takes x += s_a * a + s_b * (b + b2) (the sum residual_add_vectors makes), in the same pass.
__global__ void rmsnorm_pair_kernel(float* __restrict__ x, const float* __restrict__ w_a, float eps_a,
                                    const float* __restrict__ w_b, float eps_b, void* __restrict__ out_a,
                                    void* __restrict__ out_b, int hidden, int out_dtype, const void* __restrict__ a,
                                    int a_dtype, const float* __restrict__ s_a, const void* __restrict__ b,
                                    const void* __restrict__ b2, int b_dtype, const float* __restrict__ s_b) {
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = x[base + c];
    if (a != nullptr) {
      float sum = load_as_f32(a, a_dtype, base + c) * (s_a ? s_a[c] : 1.0f);
      if (b != nullptr) {
        float f = load_as_f32(b, b_dtype, base + c);
        if (b2 != nullptr) f += load_as_f32(b2, b_dtype, base + c);
        sum = fmaf(f, s_b ? s_b[c] : 1.0f, sum);
      }
      v += sum;
      x[base + c] = v;                                     // read again below by the thread that wrote it
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float ra = rsqrtf(ss / (float)hidden + eps_a), rb = rsqrtf(ss / (float)hidden + eps_b);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = x[base + c];
    store_from_f32(out_a, out_dtype, base + c, v * ra * w_a[c]);
    store_from_f32(out_b, out_dtype, base + c, v * rb * w_b[c]);
  }
}

__global__ void gate_mul_kernel(const void* __restrict__ a, const void* __restrict__ g, void* __restrict__ out, size_t total,
                                int dtype, int silu) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float gv = load_as_f32(g, dtype, i);
    const float sg = 1.0f / (1.0f + expf(-gv));
    store_from_f32(out, dtype, i, load_as_f32(a, dtype, i) * (silu ? gv * sg : sg));
  }
}

// One block a row, a warp a part at a time.  y [T, C] float32 contiguous; gate float32 with a row stride.
__global__ void __launch_bounds__(256) gated_groupnorm_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                                                              long long gate_stride, const float* __restrict__ w, int w_size,
                                                              float eps, void* __restrict__ out, int C, int groups,
                                                              int gate_first, int out_dtype) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int part = C / groups;
  const float* yr = y + (size_t)t * C;
  const float* gr = gate + (size_t)t * gate_stride;
  for (int p = warp; p < groups; p += nwarps) {
    float ss = 0.0f;
    for (int e = lane; e < part; e += 32) {
      const int c = p * part + e;
      float v = yr[c];
      if (gate_first) {
        const float gv = gr[c];
        v *= gv / (1.0f + expf(-gv));
      }
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)part + eps);
    for (int e = lane; e < part; e += 32) {
      const int c = p * part + e;
      const float gv = gr[c];
      const float sg = gv / (1.0f + expf(-gv));
      float v = yr[c];
      if (gate_first) v *= sg;
      v = v * inv * w[w_size == C ? c : e];
      if (!gate_first) v *= sg;
      store_from_f32(out, out_dtype, (size_t)t * C + c, v);
    }
  }
}

// The same for few, long parts: the whole block works on one part after the other.
__global__ void __launch_bounds__(512) gated_groupnorm_wide_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                                                                   long long gate_stride, const float* __restrict__ w,
                                                                   int w_size, float eps, void* __restrict__ out, int C,
                                                                   int groups, int gate_first, int out_dtype) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int part = C / groups;
  const float* yr = y + (size_t)t * C;
  const float* gr = gate + (size_t)t * gate_stride;
  for (int p = 0; p < groups; ++p) {
    float ss = 0.0f;
    for (int e = threadIdx.x; e < part; e += blockDim.x) {
      const int c = p * part + e;
      float v = yr[c];
      if (gate_first) {
        const float gv = gr[c];
        v *= gv / (1.0f + expf(-gv));
      }
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)part + eps);
    for (int e = threadIdx.x; e < part; e += blockDim.x) {
      const int c = p * part + e;
      const float gv = gr[c];
      const float sg = gv / (1.0f + expf(-gv));
      float v = yr[c];
      if (gate_first) v *= sg;
      v = v * inv * w[w_size == C ? c : e];
      if (!gate_first) v *= sg;
      store_from_f32(out, out_dtype, (size_t)t * C + c, v);
    }
  }
}

__global__ void pair_combine_kernel(const void* __restrict__ a, int a_dtype, const void* __restrict__ b, int b_dtype,
                                    const float* __restrict__ w_a, const float* __restrict__ w_b, float c_a, float c_b,
                                    float eps, float* __restrict__ out, int C) {
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * C;
  float ra = 1.0f, rb = 1.0f;
  if (w_a != nullptr) {
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const float va = load_as_f32(a, a_dtype, base + c), vb = load_as_f32(b, b_dtype, base + c);
      sa = fmaf(va, va, sa);
      sb = fmaf(vb, vb, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    ra = rsqrtf(sa / (float)C + eps);
    rb = rsqrtf(sb / (float)C + eps);
  }
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float va = load_as_f32(a, a_dtype, base + c) * ra, vb = load_as_f32(b, b_dtype, base + c) * rb;
    if (w_a != nullptr) {
      va *= w_a[c];
      vb *= w_b[c];
    }
    out[base + c] = c_a * va + c_b * vb;
  }
}

__global__ void residual_add_vectors_kernel(float* __restrict__ x, const void* __restrict__ a, int a_dtype,
                                            const float* __restrict__ s_a, const void* __restrict__ b,
                                            const void* __restrict__ b2, int b_dtype, const float* __restrict__ s_b, int C,
                                            size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    float sum = load_as_f32(a, a_dtype, i) * (s_a ? s_a[c] : 1.0f);
    if (b != nullptr) {
      float f = load_as_f32(b, b_dtype, i);
      if (b2 != nullptr) f += load_as_f32(b2, b_dtype, i);
      sum = fmaf(f, s_b ? s_b[c] : 1.0f, sum);
    }
    x[i] += sum;
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" {

int ifx_bigram_add(float* x, const void* table, const int* tokens, const int* positions, const int* token_req,
                   const int* req_slot, const int* cu_seqlens, int* state, long long state_slot_stride, int T, int hidden,
                   int vocab, long long mul_prev, long long mul_cur, int buckets, int table_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden <= 0 || vocab <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0 || state == nullptr) return IFX_E_BADARG;
  const int threads = hidden >= 256 ? 256 : ((hidden + 31) / 32) * 32;
  if (table_dtype == IFX_DT_F32)
    bigram_add_kernel<float><<<T, threads, 0, stream>>>(x, (const float*)table, tokens, positions, token_req, req_slot,
                                                        cu_seqlens, state, state_slot_stride, hidden, vocab, mul_prev, mul_cur,
                                                        buckets);
  else if (table_dtype == IFX_DT_BF16)
    bigram_add_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(x, (const __nv_bfloat16*)table, tokens, positions, token_req,
                                                                req_slot, cu_seqlens, state, state_slot_stride, hidden, vocab,
                                                                mul_prev, mul_cur, buckets);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_rmsnorm_pair(float* x, const float* w_a, float eps_a, const float* w_b, float eps_b, void* out_a, void* out_b,
                     int T, int hidden, int out_dtype, const void* a, int a_dtype, const float* s_a, const void* b,
                     const void* b2, int b_dtype, const float* s_b, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden <= 0 || (a == nullptr && b != nullptr) || (b == nullptr && b2 != nullptr)) return IFX_E_BADARG;
  if (out_dtype != IFX_DT_F32 && out_dtype != IFX_DT_BF16) return IFX_E_DTYPE;
  for (int dt : {a_dtype, b_dtype})
    if (dt != IFX_DT_F32 && dt != IFX_DT_BF16) return IFX_E_DTYPE;
  const int threads = hidden >= 1024 ? 512 : (hidden >= 256 ? 256 : ((hidden + 31) / 32) * 32);
  rmsnorm_pair_kernel<<<T, threads, 0, stream>>>(x, w_a, eps_a, w_b, eps_b, out_a, out_b, hidden, out_dtype, a, a_dtype, s_a, b,
                                                 b2, b_dtype, s_b);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_gate_mul(const void* a, const void* g, void* out, long long total, int dtype, int silu, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (dtype != IFX_DT_F32 && dtype != IFX_DT_BF16) return IFX_E_DTYPE;
  const long long blocks = (total + 255) / 256;
  gate_mul_kernel<<<(unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, stream>>>(a, g, out, (size_t)total, dtype, silu);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_gated_groupnorm(const float* y, const float* gate, long long gate_stride, const float* w, int w_size, float eps,
                        void* out, int T, int C, int groups, int gate_first, int out_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || groups <= 0 || C % groups || (w_size != C && w_size != C / groups) || gate_stride < C) return IFX_E_BADARG;
  if (out_dtype != IFX_DT_F32 && out_dtype != IFX_DT_BF16) return IFX_E_DTYPE;
  const int part = C / groups;
  if (groups < 8 && part > 64) {                            // few long parts: a block per row takes them in turn
    const int threads = part >= 2048 ? 512 : (part >= 256 ? 256 : ((part + 31) / 32) * 32);
    gated_groupnorm_wide_kernel<<<T, threads, 0, stream>>>(y, gate, gate_stride, w, w_size, eps, out, C, groups, gate_first,
                                                           out_dtype);
  } else {
    const int warps = groups >= 8 ? 8 : groups;
    gated_groupnorm_kernel<<<T, warps * 32, 0, stream>>>(y, gate, gate_stride, w, w_size, eps, out, C, groups, gate_first,
                                                        out_dtype);
  }
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_pair_combine(const void* a, int a_dtype, const void* b, int b_dtype, const float* w_a, const float* w_b, float c_a,
                     float c_b, float eps, float* out, int T, int C, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || (w_a == nullptr) != (w_b == nullptr)) return IFX_E_BADARG;
  for (int dt : {a_dtype, b_dtype})
    if (dt != IFX_DT_F32 && dt != IFX_DT_BF16) return IFX_E_DTYPE;
  const int threads = C >= 1024 ? 512 : (C >= 256 ? 256 : ((C + 31) / 32) * 32);
  pair_combine_kernel<<<T, threads, 0, stream>>>(a, a_dtype, b, b_dtype, w_a, w_b, c_a, c_b, eps, out, C);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_residual_add_vectors(float* x, const void* a, int a_dtype, const float* s_a, const void* b, const void* b2,
                             int b_dtype, const float* s_b, int T, int C, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || a == nullptr || (b == nullptr && b2 != nullptr)) return IFX_E_BADARG;
  for (int dt : {a_dtype, b_dtype})
    if (dt != IFX_DT_F32 && dt != IFX_DT_BF16) return IFX_E_DTYPE;
  const size_t total = (size_t)T * C;
  const size_t blocks = (total + 255) / 256;
  residual_add_vectors_kernel<<<(unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, stream>>>(
      x, a, a_dtype, s_a, b, b2, b_dtype, s_b, C, total);
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
