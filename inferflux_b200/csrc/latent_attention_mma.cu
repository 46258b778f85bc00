// Attention over cached latents on the tensor cores (bfloat16), for prompt portions
// and decoded tokens alike.  The latent of a key serves all heads as key and as
// value, so a thread block takes a tile of one request's tokens with ALL their heads
// as its rows, (token, head) pairs, and every latent tile it stages in shared memory
// is used by all of them, for the scores and for the weighted sum:
//
//   S = Ql C^T     Ql [rows, rank] queries carried into latent space, C [keys, rank]
//   P = exp2(S * scale * log2(e) - m)          float32, running maximum m and sum l
//   O += P C                                   P rounded to bfloat16 as the product's operand
//
// mma.sync m16n8k16 with float32 accumulators; a warp owns 16 rows; the 32-key tile is
// double-buffered with cp.async through the block table.  A row (token at position p,
// any head) sees keys max(0, p - window + 1) .. p.  The sink of a head joins the
// denominator at the end, once.  With `splits` > 1 (decoded tokens, few rows, long
// windows) the key range of a block is cut over gridDim.z; each part leaves its
// unnormalised sum, maximum and denominator in a workspace, and latent_merge_kernel
// adds them (and the sink) in split order.
//
// With `rot` > 0 a cached row is [latent of `rank`; `rot` more numbers] and a query row
// likewise: the scores run over all rank + rot columns, the weighted sum over the first
// `rank` only (a key part that is no part of the value, a rotated one for instance).
//
// Sizes: rank a multiple of 16 up to 256, rot a multiple of 16 up to 64; any number of
// heads (up to 64 share a block); pages of any size.  Everything else goes to the
// generic kernel.
#include "common.cuh"

namespace ifx {

constexpr int kRowsPerBlock = 64;      // 4 warps x 16 rows
constexpr int kKeyTile = 32;
constexpr int kPad = 8;                // elements of padding per shared-memory row (16 bytes)

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// items[i] = (slot, first flat token, tokens, first position): up to 64 consecutive tokens of one request.
// Block (x, y, z): item x / subs, its tokens [sub * QT, (sub + 1) * QT) with sub = x % subs; heads y * HC ..; key part z.
template <int RMAX, int XMAX>
__global__ void __launch_bounds__(128, 3) latent_attention_mma_kernel(   // 32 .. 128 threads: a warp per 16 rows; three blocks a SM
    const __nv_bfloat16* __restrict__ ql, const __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_table,
    const int4* __restrict__ items, const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
    float* __restrict__ part_o, float2* __restrict__ part_ml, int total_rows, int heads, int rank, int page_size,
    int max_blocks, int num_pages, int window, float scale_log2, int QT, int HC, int subs, int splits, int rot) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kw = rank + rot;                                           // a cached row, a query row
  const int stride = kw + kPad;                                        // elements per shared row
  const int nthreads = blockDim.x, nwarps = nthreads >> 5, rows_blk = nwarps * 16;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [rows of the block][stride]
  __nv_bfloat16* c_s = q_s + rows_blk * stride;                        // [2][32][stride]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bx = gridDim.x - 1 - blockIdx.x;                            // later tokens see more keys: they start first
  const int4 item = items[bx / subs];
  const int sub = bx % subs;
  const int tok0 = sub * QT;
  if (tok0 >= item.z) return;
  const int ntok = min(QT, item.z - tok0);
  const int slot = item.x, t0 = item.y + tok0, p0 = item.w + tok0;
  const int h0 = blockIdx.y * HC, nh = min(HC, heads - h0);
  const int* table = block_table + (size_t)slot * max_blocks;

  // key range of the block, and this block's part of it
  const int lo_all = window > 0 ? max(0, p0 - window + 1) : 0;
  const int hi_all = p0 + ntok;                                        // exclusive
  int k_lo = lo_all, k_hi = hi_all;
  if (splits > 1) {
    int chunk = (hi_all - lo_all + splits - 1) / splits;
    chunk = (chunk + kKeyTile - 1) / kKeyTile * kKeyTile;
    k_lo = lo_all + blockIdx.z * chunk;
    k_hi = min(hi_all, k_lo + chunk);
  }
  const int chunks_per_row = kw >> 3;                                  // 16-byte pieces of a cached row

  // A tile's 32 rows: lane k of every warp finds where key k lies (one table entry), then the warps take
  // turns at stretches of 32 pieces, a lane per 16-byte piece, the address coming from the lane that looked it up.
  const int pieces = kKeyTile * chunks_per_row;
  auto load_tile = [&](int buf, int key0) {
    __nv_bfloat16* dst = c_s + (size_t)buf * kKeyTile * stride;
    const int key = key0 + lane;
    unsigned long long src = 0ull;                                     // 0: no such key, the row becomes zeros
    if (key < k_hi) {
      int page = table[key / page_size];
      if (page < 0 || page >= num_pages) page = 0;                     // a broken table must not read outside the pool
      src = (unsigned long long)(pool + ((size_t)page * page_size + key % page_size) * kw);
    }
    for (int first = warp * 32; first < pieces; first += nthreads) {   // the same trips for every lane of a warp
      const int i = first + lane;
      const int kk = min(i / chunks_per_row, kKeyTile - 1), my_piece = i % chunks_per_row;
      const unsigned long long from = __shfl_sync(0xffffffffu, src, kk);
      if (i < pieces) {
        __nv_bfloat16* d = dst + kk * stride + my_piece * 8;
        if (from) cp_async16(d, reinterpret_cast<const __nv_bfloat16*>(from) + my_piece * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);   // finite values: 0 * garbage must not be NaN
      }
    }
  };

  // queries of the block's rows (row = token * HC + head), zeros for rows that do not exist
  for (int i = tid; i < rows_blk * chunks_per_row; i += nthreads) {
    const int r = i / chunks_per_row, cc = i % chunks_per_row;
    const int qi = r / HC, hi = r % HC;
    __nv_bfloat16* d = q_s + r * stride + cc * 8;
    if (qi < ntok && hi < nh) cp_async16(d, ql + ((size_t)(t0 + qi) * heads + h0 + hi) * kw + cc * 8);
    else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
  }
  const int ntiles = k_hi > k_lo ? (k_hi - k_lo + kKeyTile - 1) / kKeyTile : 0;
  if (ntiles > 0) load_tile(0, k_lo);
  cp_async_commit();

  // the two rows of this thread: g and g + 8 of the warp's 16
  const int g = lane >> 2, quad = lane & 3;
  int row_pos[2], row_lo[2];
  bool row_ok[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = warp * 16 + g + e * 8;
    const int qi = r / HC, hi = r % HC;
    row_ok[e] = qi < ntok && hi < nh;
    row_pos[e] = p0 + qi;
    row_lo[e] = window > 0 ? max(0, row_pos[e] - window + 1) : 0;
  }
  // keys that every row of this warp sees (no mask needed for a tile inside): from the window's start of the
  // warp's last token to the position of its first
  const int warp_q0 = (warp * 16) / HC, warp_q1 = min(ntok - 1, (warp * 16 + 15) / HC);
  const int all_lo = window > 0 ? max(0, p0 + warp_q1 - window + 1) : 0, all_hi = min(p0 + warp_q0, k_hi - 1);
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  constexpr int NT = RMAX / 8;                                         // 8-column tiles of the accumulator
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  const int ksteps = kw >> 4, ntile_o = rank >> 3;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1, key0 = k_lo + tile * kKeyTile;
    if (tile + 1 < ntiles) load_tile(buf ^ 1, key0 + kKeyTile);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* ct = c_s + (size_t)buf * kKeyTile * stride;

    // S = Ql C^T for 16 rows x 32 keys
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < (RMAX + XMAX) / 16; ++ks) {
      if (ks < ksteps) {
        uint32_t a0, a1, a2, a3;
        const int mi = lane >> 3, rr = lane & 7;
        ldsm_x4(a0, a1, a2, a3, q_s + (warp * 16 + rr + (mi & 1) * 8) * stride + ks * 16 + (mi >> 1) * 8);
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {                               // two 8-key tiles per load
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, ct + (jp * 16 + rr + (mi >> 1) * 8) * stride + ks * 16 + (mi & 1) * 8);
          mma_bf16(s[jp * 2], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[jp * 2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    // mask, running maximum and sum
    float m_new[2] = {m_run[0], m_run[1]};
    if (key0 >= all_lo && key0 + kKeyTile - 1 <= all_hi) {             // every key of the tile counts for every row
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          s[j][c] *= scale_log2;
          m_new[c >> 1] = fmaxf(m_new[c >> 1], s[j][c]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int e = c >> 1;
          const int key = key0 + j * 8 + quad * 2 + (c & 1);
          const bool ok = row_ok[e] && key >= row_lo[e] && key <= row_pos[e] && key < k_hi;
          s[j][c] = ok ? s[j][c] * scale_log2 : -INFINITY;
          m_new[e] = fmaxf(m_new[e], s[j][c]);
        }
      }
    }
    float corr[2], m_use[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 1));
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 2));
      m_use[e] = m_new[e] == -INFINITY ? 0.0f : m_new[e];              // a row that has seen no key yet
      corr[e] = exp2f(m_run[e] - m_use[e]);                            // exp2(-inf) = 0 at the start
      m_run[e] = m_new[e];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(s[j][c] - m_use[c >> 1]);
        s[j][c] = p;
        sum[c >> 1] += p;
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      sum[e] += __shfl_xor_sync(0xffffffffu, sum[e], 1);
      sum[e] += __shfl_xor_sync(0xffffffffu, sum[e], 2);
      l_run[e] = l_run[e] * corr[e] + sum[e];
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {   // no row's maximum moved: nothing to rescale
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
    }
    // O += P C: the weights as the product's A operand, the same latent tile transposed as B
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {                                   // 16 keys per step
      const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {                            // two 8-column tiles per load
        if (np * 2 < ntile_o) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(b0, b1, b2, b3, ct + (kk * 16 + rr + (mi & 1) * 8) * stride + np * 16 + (mi >> 1) * 8);
          mma_bf16(o[np * 2], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[np * 2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();                                                   // the buffer is loaded again two tiles on
  }
  cp_async_wait<0>();

  // results
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    if (!row_ok[e]) continue;
    const int r = warp * 16 + g + e * 8;
    const int qi = r / HC, hi = r % HC;
    const size_t grow = (size_t)(t0 + qi) * heads + h0 + hi;           // (token, head)
    if (splits > 1) {
      float* po = part_o + ((size_t)blockIdx.z * total_rows + grow) * rank;
#pragma unroll
      for (int i = 0; i < NT; ++i)
        if (i < ntile_o) *reinterpret_cast<float2*>(po + i * 8 + quad * 2) = make_float2(o[i][e * 2], o[i][e * 2 + 1]);
      if (quad == 0) part_ml[(size_t)blockIdx.z * total_rows + grow] = make_float2(m_run[e], l_run[e]);
    } else {
      float m = m_run[e], l = l_run[e], c = 1.0f;
      if (sinks != nullptr) {
        const float sk = sinks[h0 + hi] * 1.4426950408889634f;
        const float mn = fmaxf(m, sk);
        c = exp2f(m - mn);
        l = l * c + exp2f(sk - mn);
      }
      const float inv = l > 0.0f ? c / l : 0.0f;
      __nv_bfloat16* orow = out + grow * rank;
#pragma unroll
      for (int i = 0; i < NT; ++i)
        if (i < ntile_o)
          *reinterpret_cast<uint32_t*>(orow + i * 8 + quad * 2) = pack_bf16(o[i][e * 2] * inv, o[i][e * 2 + 1] * inv);
    }
  }
}

// One block per (token, head), a thread per latent column: adds the parts in split order, counts the sink,
// normalises.  The parts' maxima and sums go through shared memory once; the columns' loads of different parts
// are independent, four in flight.
constexpr int kMaxSplits = 64;

__global__ void __launch_bounds__(256) latent_merge_kernel(const float* __restrict__ part_o,
                                                           const float2* __restrict__ part_ml,
                                                           const float* __restrict__ sinks,
                                                           __nv_bfloat16* __restrict__ out, int total_rows, int heads,
                                                           int rank, int splits) {
  __shared__ float w_s[kMaxSplits];
  __shared__ float inv_s;
  const int row = blockIdx.x, c = threadIdx.x;
  if (c < 32) {                                                        // one warp: weights of the parts and the denominator
    const float sk = sinks != nullptr ? sinks[row % heads] * 1.4426950408889634f : -INFINITY;
    float2 ml[kMaxSplits / 32];
    float m = sk;
#pragma unroll
    for (int i = 0; i < kMaxSplits / 32; ++i) {
      const int s = c + 32 * i;
      ml[i] = s < splits ? part_ml[(size_t)s * total_rows + row] : make_float2(-INFINITY, 0.0f);
      m = fmaxf(m, ml[i].x);
    }
    m = warp_max(m);
    float l = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxSplits / 32; ++i) {
      const int s = c + 32 * i;
      const float w = (ml[i].x == -INFINITY || m == -INFINITY) ? 0.0f : exp2f(ml[i].x - m);
      if (s < splits) w_s[s] = w;
      l = fmaf(ml[i].y, w, l);
    }
    l = warp_sum(l);
    if (sk != -INFINITY) l += exp2f(sk - m);
    if (c == 0) inv_s = l > 0.0f ? 1.0f / l : 0.0f;
  }
  __syncthreads();
  if (c >= rank) return;
  const float* po = part_o + (size_t)row * rank + c;
  const size_t step = (size_t)total_rows * rank;
  float acc = 0.0f;
  int s = 0;
  for (; s + 4 <= splits; s += 4) {
    const float a0 = po[(size_t)s * step], a1 = po[(size_t)(s + 1) * step], a2 = po[(size_t)(s + 2) * step],
                a3 = po[(size_t)(s + 3) * step];
    acc = fmaf(a0, w_s[s], acc);
    acc = fmaf(a1, w_s[s + 1], acc);
    acc = fmaf(a2, w_s[s + 2], acc);
    acc = fmaf(a3, w_s[s + 3], acc);
  }
  for (; s < splits; ++s) acc = fmaf(po[(size_t)s * step], w_s[s], acc);
  out[(size_t)row * rank + c] = __float2bfloat16_rn(acc * inv_s);
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// 1 if the tiled kernel takes a latent of this size (with `rot` more numbers in every row).
int ifx_latent_attention_mma_supports_rot(int rank, int rot) {
  return rank > 0 && rank % 16 == 0 && rank <= 256 && rot >= 0 && rot % 16 == 0 && rot <= 64;
}
int ifx_latent_attention_mma_supports(int rank) { return ifx_latent_attention_mma_supports_rot(rank, 0); }

// Bytes of float32 workspace the parts of a split launch need: sums [splits, rows, rank] and (max, sum) pairs.
long long ifx_latent_attention_mma_workspace(int total_rows, int rank, int splits) {
  return splits > 1 ? (long long)splits * total_rows * (rank + 2) * 4 : 0;
}

// ql: [T, heads, rank + rot], out: [T, heads, rank] bfloat16; cached rows of rank + rot.  items: [num_items, 4]
// (slot, first flat token, tokens <= 64, first position).  max_item_tokens: the largest token count among the items.
// workspace: as ifx_latent_attention_mma_workspace says.
int ifx_latent_attention_mma_rot(const void* ql, const void* pool, const int* block_table, const int* items, int num_items,
                                 int max_item_tokens, const float* sinks, void* out, void* workspace, int T, int heads,
                                 int rank, int rot, int page_size, int max_blocks, int num_pages, int window, float scale,
                                 int splits, cudaStream_t stream) {
  if (num_items <= 0 || T <= 0) return 0;
  if (!ifx_latent_attention_mma_supports_rot(rank, rot) || heads <= 0 || page_size <= 0 || max_blocks <= 0 || splits < 1 ||
      max_item_tokens < 1 || max_item_tokens > 64 || splits > kMaxSplits)
    return IFX_E_BADARG;
  if (splits > 1 && workspace == nullptr) return IFX_E_BADARG;
  const int HC = heads < kRowsPerBlock ? heads : kRowsPerBlock;
  int QT = kRowsPerBlock / HC;                                         // tokens per block
  if (QT > max_item_tokens) QT = max_item_tokens;
  const int nwarps = (QT * HC + 15) / 16;                              // a warp per 16 rows: one for a decoded token of up to 16 heads
  const int subs = (max_item_tokens + QT - 1) / QT;
  const int total_rows = T * heads;
  dim3 grid((unsigned)(num_items * subs), (unsigned)((heads + HC - 1) / HC), (unsigned)splits);
  if (grid.y > 65535u || grid.z > 65535u) return IFX_E_TOOBIG;
  const size_t smem = (size_t)(nwarps * 16 + 2 * kKeyTile) * (rank + rot + kPad) * sizeof(__nv_bfloat16);
  float* part_o = (float*)workspace;
  float2* part_ml = splits > 1 ? (float2*)(part_o + (size_t)splits * total_rows * rank) : nullptr;
  const float scale_log2 = scale * 1.4426950408889634f;
#define IFX_LAUNCH(RMAX, XMAX)                                                                                      \
  do {                                                                                                              \
    auto kern = latent_attention_mma_kernel<RMAX, XMAX>;                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 88 * 1024);       \
    kern<<<grid, nwarps * 32, smem, stream>>>((const __nv_bfloat16*)ql, (const __nv_bfloat16*)pool, block_table,            \
                                      (const int4*)items, sinks, (__nv_bfloat16*)out, part_o, part_ml, total_rows,  \
                                      heads, rank, page_size, max_blocks, num_pages, window, scale_log2, QT, HC,    \
                                      subs, splits, rot);                                                           \
  } while (0)
  if (rot == 0) {
    if (rank <= 64) IFX_LAUNCH(64, 0);
    else if (rank <= 128) IFX_LAUNCH(128, 0);
    else IFX_LAUNCH(256, 0);
  } else {
    if (rank <= 64) IFX_LAUNCH(64, 64);
    else if (rank <= 128) IFX_LAUNCH(128, 64);
    else IFX_LAUNCH(256, 64);
  }
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  if (splits > 1) {
    latent_merge_kernel<<<total_rows, 256, 0, stream>>>(
        part_o, part_ml, sinks, (__nv_bfloat16*)out, total_rows, heads, rank, splits);
    IFX_CHECK_LAUNCH();
  }
  return 0;
}

int ifx_latent_attention_mma(const void* ql, const void* pool, const int* block_table, const int* items, int num_items,
                             int max_item_tokens, const float* sinks, void* out, void* workspace, int T, int heads,
                             int rank, int page_size, int max_blocks, int num_pages, int window, float scale,
                             int splits, cudaStream_t stream) {
  return ifx_latent_attention_mma_rot(ql, pool, block_table, items, num_items, max_item_tokens, sinks, out, workspace, T,
                                      heads, rank, 0, page_size, max_blocks, num_pages, window, scale, splits, stream);
}

}  // extern "C"
