// Attention whose keys and values of all heads are made from one normed latent
// vector per token; only the latent is cached (one plane of one "head" of size
// rank per page slot).
//
//   c_j          = rmsnorm(dkv_j) * w_norm                         (latent_norm_append)
//   k_j,h = Wuk_h c_j ,  v_j,h = Wuv_h c_j
//   s_ij,h       = scale * q_i,h . k_j,h = scale * (Wuk_h^T q_i,h) . c_j
//   p_ij,h       = exp(s_ij,h) / (sum_j' exp(s_ij',h) + exp(sink_h))      over the window
//   o_i,h        = sum_j p_ij,h v_j,h = Wuv_h (sum_j p_ij,h c_j)
//
// The kernels work on the latent side of both identities: a query head is first
// carried into latent space (rank numbers), scores and the weighted sum run over
// cached latents, and the head's value projection is applied once to the sum.  Scores,
// softmax weights, the running maximum, sum and accumulator are float32.  A sink is
// a learned score per head with no key and no value: it only enlarges the
// denominator, once.  Without sinks (null) the softmax is the usual one.
//
// latent_attention_generic: one warp per (token, head), keys in chunks of 32 from
// the window's start in increasing position, so the order of every addition depends
// only on the token's position: the float32 path, and the path of sizes the tiled
// kernel does not take.
#include "common.cuh"

namespace ifx {

// ------------------------------------------------------------- norm + append
// One warp per token: c = x / rms(x) * w over `rank` columns starting at column
// `col0` of a row of `ld` elements; c goes to the cache at the token's position
// (and, if `c_out` is given, to c_out[t, :] as well).
template <typename T>
__global__ void latent_norm_append_kernel(const T* __restrict__ rows, int ld, int col0, const float* __restrict__ w,
                                          float eps, const int* __restrict__ positions,
                                          const int* __restrict__ token_req, const int* __restrict__ req_slot,
                                          const int* __restrict__ block_table, int max_blocks, int page_size,
                                          int num_pages, T* __restrict__ pool, T* __restrict__ c_out, int num_tokens,
                                          int rank) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= num_tokens) return;
  const T* x = rows + (size_t)t * ld + col0;
  float ss = 0.0f;
  for (int e = lane; e < rank; e += 32) {
    const float v = to_f32(x[e]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)rank + eps);
  T* dst = nullptr;
  if (pool != nullptr) {
    const int pos = positions[t];
    const int slot = req_slot[token_req[t]];
    const int page = block_table[(size_t)slot * max_blocks + pos / page_size];
    if (page >= 0 && page < num_pages) dst = pool + ((size_t)page * page_size + pos % page_size) * rank;
  }
  for (int e = lane; e < rank; e += 32) {
    const T c = from_f32<T>(to_f32(x[e]) * r * w[e]);
    if (dst) dst[e] = c;
    if (c_out) c_out[(size_t)t * rank + e] = c;
  }
}

// ------------------------------------------------- norm + rotation + append
// One warp per token.  The cached row is [c; k_t]: c = x / rms(x) * w over `lat` columns starting at `col0` of `rows`,
// k_t the `rot` columns behind them turned by the token's position.  Every query head's last `rot` elements (heads of
// dim + rot in `q`, rows ldq apart) are turned the same way and written to q_out (rows ld_out apart, heads head_stride
// apart, at `out_offset` in a head): q itself, or the tail of a query in latent space.  The first `rot_used` of the
// `rot` elements turn (pair i is (2i, 2i + 1) when interleaved, else (i, i + rot_used / 2)); angle = position *
// inv_freq[i] in float32, cos and sin times `magnitude`.
template <typename T>
__device__ __forceinline__ void turn_store(const T* src, T* dst, int rot, int rot_used, int interleaved,
                                           const float* __restrict__ cs, float* __restrict__ held, int lane) {
  const int half = rot_used >> 1;                        // cs: cos[half], sin[half] of this token
  __syncwarp();
  for (int e = lane; e < rot; e += 32) held[e] = to_f32(src[e]);       // all of it first: dst may be src
  __syncwarp();
  for (int e = lane; e < rot; e += 32) {
    float v = held[e];
    if (e < rot_used) {
      const int i = interleaved ? (e >> 1) : (e < half ? e : e - half);
      const bool first = interleaved ? !(e & 1) : e < half;
      const float m = held[interleaved ? (e ^ 1) : (first ? e + half : e - half)];
      v = first ? v * cs[i] - m * cs[half + i] : v * cs[i] + m * cs[half + i];
    }
    dst[e] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void latent_rope_append_kernel(const T* __restrict__ rows, int ld, int col0, const float* __restrict__ w,
                                          float eps, const T* q, int ldq, T* q_out, int ld_out,
                                          int head_stride, int out_offset, const float* __restrict__ inv_freq,
                                          int rot_used, int interleaved, float magnitude,
                                          const int* __restrict__ positions, const int* __restrict__ token_req,
                                          const int* __restrict__ req_slot, const int* __restrict__ block_table,
                                          int max_blocks, int page_size, int num_pages, T* __restrict__ pool,
                                          int num_tokens, int lat, int rot, int heads, int dim) {
  extern __shared__ float cs_s[];                        // per warp: cos and sin of the token's angles, then `rot` staged numbers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= num_tokens) return;
  const int pos = positions[t];
  const int half = rot_used >> 1;
  float* cs = cs_s + (size_t)warp * (rot_used + rot);
  float* held = cs + rot_used;
  for (int i = lane; i < half; i += 32) {
    float sn, c;
    sincosf((float)pos * inv_freq[i], &sn, &c);
    cs[i] = c * magnitude;
    cs[half + i] = sn * magnitude;
  }
  __syncwarp();
  const T* x = rows + (size_t)t * ld + col0;
  float ss = 0.0f;
  for (int e = lane; e < lat; e += 32) {
    const float v = to_f32(x[e]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)lat + eps);
  if (pool != nullptr) {
    const int slot = req_slot[token_req[t]];
    const int page = block_table[(size_t)slot * max_blocks + pos / page_size];
    if (page >= 0 && page < num_pages) {
      T* dst = pool + ((size_t)page * page_size + pos % page_size) * (lat + rot);
      for (int e = lane; e < lat; e += 32) dst[e] = from_f32<T>(to_f32(x[e]) * r * w[e]);
      turn_store(x + lat, dst + lat, rot, rot_used, interleaved, cs, held, lane);
    }
  }
  for (int h = 0; h < heads; ++h)
    turn_store(q + (size_t)t * ldq + (size_t)h * (dim + rot) + dim, q_out + (size_t)t * ld_out + (size_t)h * head_stride + out_offset,
               rot, rot_used, interleaved, cs, held, lane);
}

// ------------------------------------------------------------------ attention
constexpr int kLatentWarps = 4;

// NR = ceil(rank / 32): latent elements a lane owns (e = lane + 32 i).
template <typename T, int NR>
__global__ void __launch_bounds__(kLatentWarps * 32) latent_attention_generic_kernel(
    const T* __restrict__ q, int ldq, const T* __restrict__ w_uk, const T* __restrict__ w_uv,
    const float* __restrict__ sinks, const T* __restrict__ pool, const int* __restrict__ block_table,
    const int* __restrict__ positions, const int* __restrict__ token_req, const int* __restrict__ req_slot,
    const int* __restrict__ rows, T* __restrict__ out, int num_tokens, int heads, int dim, int vdim, int lat,
    int page_size, int max_blocks, int num_pages, int window, float scale, int rot) {
  // `lat`: numbers of a latent; `rot`: numbers behind it in every cached row and behind the `dim` plain ones of every
  // query head, which meet each other directly.  `rank` is the cached row: the kernel's sums run over all of it.
  extern __shared__ float lat_s[];                       // per warp: `rank` floats (query in latent space, then the sum)
  const int rank = lat + rot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kLatentWarps + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = rows ? rows[item / heads] : (int)(item / heads), h = (int)(item % heads);
  float* ql = lat_s + (size_t)warp * rank;
  const int pos = positions[t];
  const int slot = req_slot[token_req[t]];
  const int* table = block_table + (size_t)slot * max_blocks;

  // the query head in latent space: ql[e] = sum_d Wuk[h dim + d, e] q[d]
  {
    const T* qh = q + (size_t)t * ldq + (size_t)h * (dim + rot);
    const T* wk = w_uk + (size_t)h * dim * lat;
    float a[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) a[i] = 0.0f;
    for (int d = 0; d < dim; ++d) {
      const float qd = to_f32(qh[d]);
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int e = lane + 32 * i;
        if (e < lat) a[i] = fmaf(to_f32(wk[(size_t)d * lat + e]), qd, a[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int e = lane + 32 * i;
      if (e < lat) ql[e] = a[i];
      else if (e < rank) ql[e] = to_f32(qh[dim + e - lat]);      // the turned part as it is
    }
    __syncwarp();
  }

  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int end = pos + 1;
  float m = -INFINITY, l = 0.0f;
  float acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) acc[i] = 0.0f;

  for (int base = first; base < end; base += 32) {
    const int j = base + lane;
    const bool valid = j < end;
    float s = -INFINITY;
    const T* crow = pool;
    if (valid) {
      int page = table[j / page_size];
      if (page < 0 || page >= num_pages) page = 0;       // a broken table must not read outside the pool
      crow = pool + ((size_t)page * page_size + j % page_size) * rank;
      float dot = 0.0f;
      for (int e = 0; e < rank; ++e) dot = fmaf(ql[e], to_f32(crow[e]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.0f;
    const float corr = expf(m - m_new);                  // m = -inf at the start: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] *= corr;
    const int count = min(32, end - base);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* cr = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, (unsigned long long)crow, jj));
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int e = lane + 32 * i;
        if (e < rank) acc[i] = fmaf(pj, to_f32(cr[e]), acc[i]);
      }
    }
  }
  if (sinks != nullptr) {                                // the sink joins the denominator only
    const float sk = sinks[h];
    const float m_new = fmaxf(m, sk);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] *= corr;
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  __syncwarp();
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int e = lane + 32 * i;
    if (e < rank) ql[e] = acc[i] * inv;
  }
  __syncwarp();
  // the head's values: o[v] = sum_e Wuv[h vdim + v, e] ql[e]
  T* orow = out + ((size_t)t * heads + h) * vdim;
  const T* wv = w_uv + (size_t)h * vdim * lat;
  for (int v0 = 0; v0 < vdim; v0 += 32) {
    const int v = v0 + lane;
    if (v < vdim) {
      const T* wr = wv + (size_t)v * lat;
      float o = 0.0f;
      for (int e = 0; e < lat; ++e) o = fmaf(to_f32(wr[e]), ql[e], o);
      orow[v] = from_f32<T>(o);
    }
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" {

int ifx_latent_norm_append(const void* rows, int ld, int col0, const float* w, float eps, const int* positions,
                           const int* token_req, const int* req_slot, const int* block_table, int max_blocks,
                           int page_size, int num_pages, void* pool, void* c_out, int T, int rank, int dtype,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rank <= 0 || ld < col0 + rank || col0 < 0) return IFX_E_BADARG;
  if (pool != nullptr && (page_size <= 0 || max_blocks <= 0 || block_table == nullptr)) return IFX_E_BADARG;
  const int warps = 4;
  const unsigned blocks = (unsigned)((T + warps - 1) / warps);
  if (dtype == IFX_DT_F32)
    latent_norm_append_kernel<float><<<blocks, warps * 32, 0, stream>>>(
        (const float*)rows, ld, col0, w, eps, positions, token_req, req_slot, block_table, max_blocks, page_size,
        num_pages, (float*)pool, (float*)c_out, T, rank);
  else if (dtype == IFX_DT_BF16)
    latent_norm_append_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
        (const __nv_bfloat16*)rows, ld, col0, w, eps, positions, token_req, req_slot, block_table, max_blocks,
        page_size, num_pages, (__nv_bfloat16*)pool, (__nv_bfloat16*)c_out, T, rank);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

// pool null: nothing is stored.  q_out may be q itself (ld_out = ldq, head_stride = dim + rot, out_offset = dim).
int ifx_latent_rope_append(const void* rows, int ld, int col0, const float* w, float eps, const void* q, int ldq, void* q_out,
                           int ld_out, int head_stride, int out_offset, const float* inv_freq, int rot_used, int interleaved,
                           float magnitude, const int* positions, const int* token_req, const int* req_slot,
                           const int* block_table, int max_blocks, int page_size, int num_pages, void* pool, int T, int lat,
                           int rot, int heads, int dim, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (lat <= 0 || rot < 0 || col0 < 0 || ld < col0 + lat + rot || heads <= 0 || dim < 0 || ldq < heads * (dim + rot) ||
      rot_used < 0 || rot_used > rot || (rot_used & 1) || (rot_used > 0 && inv_freq == nullptr))
    return IFX_E_BADARG;
  if (pool != nullptr && (page_size <= 0 || max_blocks <= 0 || block_table == nullptr)) return IFX_E_BADARG;
  const int warps = 4;
  const unsigned blocks = (unsigned)((T + warps - 1) / warps);
  const size_t smem = (size_t)warps * (rot_used + rot + 1) * sizeof(float);
  if (dtype == IFX_DT_F32)
    latent_rope_append_kernel<float><<<blocks, warps * 32, smem, stream>>>(
        (const float*)rows, ld, col0, w, eps, (const float*)q, ldq, (float*)q_out, ld_out, head_stride, out_offset, inv_freq,
        rot_used, interleaved, magnitude, positions, token_req, req_slot, block_table, max_blocks, page_size, num_pages,
        (float*)pool, T, lat, rot, heads, dim);
  else if (dtype == IFX_DT_BF16)
    latent_rope_append_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)rows, ld, col0, w, eps, (const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)q_out, ld_out,
        head_stride, out_offset, inv_freq, rot_used, interleaved, magnitude, positions, token_req, req_slot, block_table,
        max_blocks, page_size, num_pages, (__nv_bfloat16*)pool, T, lat, rot, heads, dim);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_latent_attention_max_rank() { return 1024; }

int ifx_latent_attention_generic_rot(const void* q, int ldq, const void* w_uk, const void* w_uv, const float* sinks,
                                     const void* pool, const int* block_table, const int* positions,
                                     const int* token_req, const int* req_slot, const int* rows, void* out,
                                     int num_tokens, int heads, int dim, int vdim, int lat, int page_size,
                                     int max_blocks, int num_pages, int window, float scale, int rot, int dtype,
                                     cudaStream_t stream);

int ifx_latent_attention_generic(const void* q, int ldq, const void* w_uk, const void* w_uv, const float* sinks,
                                 const void* pool, const int* block_table, const int* positions,
                                 const int* token_req, const int* req_slot, const int* rows, void* out,
                                 int num_tokens, int heads, int dim, int vdim, int rank, int page_size,
                                 int max_blocks, int num_pages, int window, float scale, int dtype,
                                 cudaStream_t stream) {
  return ifx_latent_attention_generic_rot(q, ldq, w_uk, w_uv, sinks, pool, block_table, positions, token_req, req_slot, rows,
                                          out, num_tokens, heads, dim, vdim, rank, page_size, max_blocks, num_pages, window,
                                          scale, 0, dtype, stream);
}

// The same with `rot` numbers behind the latent in every cached row (rows of lat + rot) and behind the `dim` plain
// elements of every query head (heads of dim + rot in q); w_uk [heads * dim, lat], w_uv [heads * vdim, lat].
int ifx_latent_attention_generic_rot(const void* q, int ldq, const void* w_uk, const void* w_uv, const float* sinks,
                                     const void* pool, const int* block_table, const int* positions,
                                     const int* token_req, const int* req_slot, const int* rows, void* out,
                                     int num_tokens, int heads, int dim, int vdim, int lat, int page_size,
                                     int max_blocks, int num_pages, int window, float scale, int rot, int dtype,
                                     cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || lat <= 0 || rot < 0 || page_size <= 0 || max_blocks <= 0 ||
      ldq < heads * (dim + rot))
    return IFX_E_BADARG;
  const int rank = lat + rot;
  if (rank > 1024) return IFX_E_TOOBIG;
  const long long items = (long long)num_tokens * heads;
  const unsigned blocks = (unsigned)((items + kLatentWarps - 1) / kLatentWarps);
  const size_t smem = (size_t)kLatentWarps * rank * sizeof(float);
#define IFX_LAUNCH(TT, NR)                                                                                         \
  latent_attention_generic_kernel<TT, NR><<<blocks, kLatentWarps * 32, smem, stream>>>(                            \
      (const TT*)q, ldq, (const TT*)w_uk, (const TT*)w_uv, sinks, (const TT*)pool, block_table, positions,         \
      token_req, req_slot, rows, (TT*)out, num_tokens, heads, dim, vdim, lat, page_size, max_blocks, num_pages,    \
      window, scale, rot)
#define IFX_BY_RANK(TT)                          \
  do {                                           \
    if (rank <= 64) IFX_LAUNCH(TT, 2);           \
    else if (rank <= 128) IFX_LAUNCH(TT, 4);     \
    else if (rank <= 256) IFX_LAUNCH(TT, 8);     \
    else if (rank <= 512) IFX_LAUNCH(TT, 16);    \
    else IFX_LAUNCH(TT, 32);                     \
  } while (0)
  if (dtype == IFX_DT_F32) IFX_BY_RANK(float);
  else if (dtype == IFX_DT_BF16) IFX_BY_RANK(__nv_bfloat16);
  else return IFX_E_DTYPE;
#undef IFX_BY_RANK
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
