// A mixture of small feed-forward experts: the router's choice and the experts' work for every token.
//
//   moe_route     scores = softmax(z) over all router outputs (float32); the `top` largest of score + correction
//                 are chosen (the earlier index wins a tie); their weights are the scores themselves
//                 (of_chosen: the `top` largest of z + correction are chosen and the weights are the softmax over
//                 the chosen z alone; sigmoid: scores = sigmoid(z), the `top` largest of score + correction are chosen,
//                 and the weights are the chosen scores divided by (their sum + floor))
//   moe_up        act[p] = relu(W_up[e] h[t])^2 for every (token, choice) pair p = t * top + c whose expert e
//                 has weights (experts numbered from `experts` on hand their input on unchanged); or, gated (an
//                 expert's gate rows above its up rows, [experts, 2 ff, width]), with g = min(gate, limit) and
//                 u = clamp(up, -limit, limit): act[p] = g sigmoid(slope g) (u + offset)
//   moe_down      out[t] = sum over the token's choices, in their order, of weight * (W_down[e] act[p]), or
//                 weight * h[t] for an expert without weights
//
// Steps with many tokens in bfloat16 sort their (token, choice) pairs by expert instead and multiply whole tiles on the
// tensor cores (the grouped modes of gemm_tcgen05.cu):
//
//   moe_sort      every expert's pairs get a stretch of rows that starts on a multiple of 128; per row the pair it
//                 holds (or -1) and the pair's weight (or 0); per 128-row tile its expert (or -1); per pair its row
//   moe_gather    rows[r] = h[token of the pair in row r], zeros for a row without a pair
//   moe_combine   out[t] = sum over the token's choices, in their order, of y[row of the pair] (already weighted), or
//                 weight * h[t] for an expert without weights
//
// The kernels below the sort are those of the float32 run and of steps with few tokens: a warp makes one output number as a dot
// product (lanes stride the inner size, then a shuffle tree), so every sum has an order that depends on the sizes
// alone.  Expert weights are stacked: up [experts, ff, width], down [experts, width, ff].
#include "common.cuh"

namespace ifx {

constexpr int kMaxRouterOutputs = 1024;

__global__ void moe_route_kernel(const float* __restrict__ z, const float* __restrict__ correction,
                                 int* __restrict__ ids, float* __restrict__ weights, int T, int n, int top, int of_chosen,
                                 float floor) {
  const bool sigmoid = of_chosen == 2;
  __shared__ float score_s[4][kMaxRouterOutputs];
  __shared__ float choice_s[4][kMaxRouterOutputs];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  const float* zr = z + (size_t)t * n;
  if (of_chosen == 1) {
    for (int i = lane; i < n; i += 32) {
      score_s[warp][i] = zr[i];
      choice_s[warp][i] = zr[i] + (correction ? correction[i] : 0.0f);
    }
    __syncwarp();
    float m = -INFINITY;                                // the largest chosen logit, known to lane 0
    for (int c = 0; c < top; ++c) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int i = lane; i < n; i += 32) {
        const float v = choice_s[warp][i];
        if (v > best) { best = v; at = i; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at >= n) at = 0;
      if (lane == 0) {
        ids[(size_t)t * top + c] = at;
        m = fmaxf(m, score_s[warp][at]);
        choice_s[warp][at] = -INFINITY;
      }
      __syncwarp();
    }
    if (lane == 0) {                                     // softmax over the chosen alone, in the order of the choice
      float sum = 0.0f;
      for (int c = 0; c < top; ++c) {
        const float e = expf(score_s[warp][ids[(size_t)t * top + c]] - m);
        weights[(size_t)t * top + c] = e;
        sum += e;
      }
      for (int c = 0; c < top; ++c) weights[(size_t)t * top + c] /= sum;
    }
    return;
  }
  float m = -INFINITY;
  for (int i = lane; i < n; i += 32) m = fmaxf(m, zr[i]);
  m = warp_max(m);
  float sum = 0.0f;
  for (int i = lane; i < n; i += 32) {
    const float e = sigmoid ? 1.0f / (1.0f + expf(-zr[i])) : expf(zr[i] - m);
    score_s[warp][i] = e;
    sum += e;
  }
  sum = sigmoid ? 1.0f : warp_sum(sum);
  for (int i = lane; i < n; i += 32) {
    const float sc = score_s[warp][i] / sum;
    score_s[warp][i] = sc;
    choice_s[warp][i] = sc + (correction ? correction[i] : 0.0f);
  }
  __syncwarp();
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
      const float v = choice_s[warp][i];
      if (v > best) { best = v; at = i; }              // i ascends: the earlier index stays on a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= n) at = 0;                               // only if every score is NaN
    if (lane == 0) {
      ids[(size_t)t * top + c] = at;
      weights[(size_t)t * top + c] = score_s[warp][at];
      choice_s[warp][at] = -INFINITY;
    }
    __syncwarp();
  }
  if (sigmoid && lane == 0) {                            // the chosen scores over their sum, added in the order of the choice
    float total = 0.0f;
    for (int c = 0; c < top; ++c) total += weights[(size_t)t * top + c];
    total += floor;
    for (int c = 0; c < top; ++c) weights[(size_t)t * top + c] /= total;
  }
}

template <typename T>
__device__ __forceinline__ float dot_lanes(const T* __restrict__ w, const float* __restrict__ a, int n, int lane) {
  float s = 0.0f;
  for (int i = lane; i < n; i += 32) s = fmaf(to_f32(w[i]), a[i], s);
  return warp_sum(s);
}

// bfloat16 weights in 16-byte pieces, four of them in flight per lane, when the row allows it.
template <>
__device__ __forceinline__ float dot_lanes<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ a,
                                                          int n, int lane) {
  float s = 0.0f;
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    const uint4* w8 = reinterpret_cast<const uint4*>(w);
    const int chunks = n >> 3;
    auto use = [&](uint4 raw, int chunk) {
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float4 a0 = *reinterpret_cast<const float4*>(a + 8 * chunk), a1 = *reinterpret_cast<const float4*>(a + 8 * chunk + 4);
      const float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
      const float2 f2 = __bfloat1622float2(p2[2]), f3 = __bfloat1622float2(p2[3]);
      s = fmaf(f0.x, a0.x, s); s = fmaf(f0.y, a0.y, s); s = fmaf(f1.x, a0.z, s); s = fmaf(f1.y, a0.w, s);
      s = fmaf(f2.x, a1.x, s); s = fmaf(f2.y, a1.y, s); s = fmaf(f3.x, a1.z, s); s = fmaf(f3.y, a1.w, s);
    };
    int i = lane;
    for (; i + 96 < chunks; i += 128) {
      const uint4 r0 = __ldg(w8 + i), r1 = __ldg(w8 + i + 32), r2 = __ldg(w8 + i + 64), r3 = __ldg(w8 + i + 96);
      use(r0, i); use(r1, i + 32); use(r2, i + 64); use(r3, i + 96);
    }
    for (; i < chunks; i += 32) use(__ldg(w8 + i), i);
  } else {
    for (int i = lane; i < n; i += 32) s = fmaf(__bfloat162float(w[i]), a[i], s);
  }
  return warp_sum(s);
}

// NR rows of bfloat16 weights against the same staged vector, their 16-byte loads in flight together (a row alone
// leaves a lane with too few bytes under way to keep the memory busy).  Each row's sum is added in the order dot_lanes uses.
template <int NR>
__device__ __forceinline__ void dot_lanes_rows(const __nv_bfloat16* const (&w)[NR], const float* __restrict__ a, int n,
                                               int lane, float (&out)[NR]) {
  float s[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) s[r] = 0.0f;
  bool wide = (n & 7) == 0;
#pragma unroll
  for (int r = 0; r < NR; ++r) wide = wide && (reinterpret_cast<uintptr_t>(w[r]) & 15) == 0;
  if (wide) {
    const int chunks = n >> 3;
    auto use = [&](uint4 raw, int chunk, float& acc) {
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float4 a0 = *reinterpret_cast<const float4*>(a + 8 * chunk), a1 = *reinterpret_cast<const float4*>(a + 8 * chunk + 4);
      const float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
      const float2 f2 = __bfloat1622float2(p2[2]), f3 = __bfloat1622float2(p2[3]);
      acc = fmaf(f0.x, a0.x, acc); acc = fmaf(f0.y, a0.y, acc); acc = fmaf(f1.x, a0.z, acc); acc = fmaf(f1.y, a0.w, acc);
      acc = fmaf(f2.x, a1.x, acc); acc = fmaf(f2.y, a1.y, acc); acc = fmaf(f3.x, a1.z, acc); acc = fmaf(f3.y, a1.w, acc);
    };
    int i = lane;
    for (; i + 32 < chunks; i += 64) {
      uint4 lo[NR], hi[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        lo[r] = __ldg(reinterpret_cast<const uint4*>(w[r]) + i);
        hi[r] = __ldg(reinterpret_cast<const uint4*>(w[r]) + i + 32);
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        use(lo[r], i, s[r]);
        use(hi[r], i + 32, s[r]);
      }
    }
    for (; i < chunks; i += 32) {
      uint4 lo[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) lo[r] = __ldg(reinterpret_cast<const uint4*>(w[r]) + i);
#pragma unroll
      for (int r = 0; r < NR; ++r) use(lo[r], i, s[r]);
    }
  } else {
    for (int i = lane; i < n; i += 32) {
#pragma unroll
      for (int r = 0; r < NR; ++r) s[r] = fmaf(__bfloat162float(w[r][i]), a[i], s[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) out[r] = warp_sum(s[r]);
}

template <int NR>
__device__ __forceinline__ void dot_lanes_rows(const float* const (&w)[NR], const float* __restrict__ a, int n, int lane,
                                               float (&out)[NR]) {
#pragma unroll
  for (int r = 0; r < NR; ++r) out[r] = dot_lanes<float>(w[r], a, n, lane);
}

constexpr int kMoeWarps = 8;

template <typename T, bool GLU>
__global__ void moe_up_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ ids,
                              T* __restrict__ act, int top, int experts, int width, int ff, int rows_per_block,
                              float limit, float slope, float offset) {
  extern __shared__ __align__(16) float h_s[];
  const int p = blockIdx.x;
  const int e = ids[p];
  if (e >= experts || e < 0) return;
  const int t = p / top;
  for (int i = threadIdx.x; i < width; i += blockDim.x) h_s[i] = to_f32(h[(size_t)t * width + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.y * rows_per_block;
  const T* w = w_up + (size_t)e * (GLU ? 2 : 1) * ff * width;
  const int last = min(ff, f0 + rows_per_block) - 1;
  for (int f = f0 + warp; f <= last; f += 4 * kMoeWarps) {           // four rows of a warp at a time
    const T* rows[4];
    float z[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) rows[r] = w + (size_t)min(f + r * kMoeWarps, last) * width;
    dot_lanes_rows<4>(rows, h_s, width, lane, z);
    if (GLU) {
      float up[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) rows[r] += (size_t)ff * width;     // the up rows lie ff rows below the gate rows
      dot_lanes_rows<4>(rows, h_s, width, lane, up);
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float g = fminf(z[r], limit), u = fminf(fmaxf(up[r], -limit), limit);
          if (f + r * kMoeWarps <= last)
            act[(size_t)p * ff + f + r * kMoeWarps] = from_f32<T>(g / (1.0f + expf(-slope * g)) * (u + offset));
        }
      }
      continue;
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float zf = fmaxf(z[r], 0.0f);
        if (f + r * kMoeWarps <= last) act[(size_t)p * ff + f + r * kMoeWarps] = from_f32<T>(zf * zf);
      }
    }
  }
}

template <typename T, typename TO>
__global__ void moe_down_kernel(const T* __restrict__ h, const T* __restrict__ act, const T* __restrict__ w_down,
                                const int* __restrict__ ids, const float* __restrict__ weights, TO* __restrict__ out,
                                int top, int experts, int width, int ff, int rows_per_block) {
  extern __shared__ __align__(16) float a_s[];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.y * rows_per_block, c1 = min(width, c0 + rows_per_block);
  float acc[8];                                         // rows c0 + warp + 8 r of this warp
#pragma unroll
  for (int r = 0; r < 8; ++r) acc[r] = 0.0f;
  for (int c = 0; c < top; ++c) {
    const int p = t * top + c;
    const int e = ids[p];
    const float g = weights[p];
    if (e >= experts || e < 0) {                        // the input itself
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int row = c0 + warp + kMoeWarps * r;
          if (row < c1) acc[r] = fmaf(g, to_f32(h[(size_t)t * width + row]), acc[r]);
        }
      }
      continue;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ff; i += blockDim.x) a_s[i] = to_f32(act[(size_t)p * ff + i]);
    __syncthreads();
    const T* w = w_down + (size_t)e * width * ff;
#pragma unroll
    for (int r0 = 0; r0 < 8; r0 += 4) {
      if (c0 + warp + kMoeWarps * r0 >= c1) break;
      const T* rows[4];
      float d[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) rows[r] = w + (size_t)min(c0 + warp + kMoeWarps * (r0 + r), c1 - 1) * ff;
      dot_lanes_rows<4>(rows, a_s, ff, lane, d);
#pragma unroll
      for (int r = 0; r < 4; ++r)
        if (c0 + warp + kMoeWarps * (r0 + r) < c1) acc[r0 + r] = fmaf(g, d[r], acc[r0 + r]);
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int row = c0 + warp + kMoeWarps * r;
      if (row < c1) out[(size_t)t * width + row] = from_f32<TO>(acc[r]);
    }
  }
}

// One block.  counts/offset/cursor live in shared memory: experts <= kMaxRouterOutputs.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, const float* __restrict__ weights,
                                                        int pairs, int experts, int* __restrict__ row_pair,
                                                        float* __restrict__ row_scale, int* __restrict__ tile_group,
                                                        int* __restrict__ pair_row, int rows_cap) {
  __shared__ int count_s[kMaxRouterOutputs], offset_s[kMaxRouterOutputs], cursor_s[kMaxRouterOutputs];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count_s[e] = cursor_s[e] = 0;
  for (int r = threadIdx.x; r < rows_cap; r += blockDim.x) {
    row_pair[r] = -1;
    row_scale[r] = 0.0f;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&count_s[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0;
    for (int e = 0; e < experts; ++e) {
      offset_s[e] = row;
      const int tiles = (count_s[e] + 127) / 128;
      for (int i = 0; i < tiles; ++i) tile_group[row / 128 + i] = e;
      row += tiles * 128;
    }
    for (int tile = row / 128; tile < rows_cap / 128; ++tile) tile_group[tile] = -1;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    int row = -1;
    if (e >= 0 && e < experts) {
      row = offset_s[e] + atomicAdd(&cursor_s[e], 1);      // which row inside the stretch does not change a row's result
      row_pair[row] = p;
      row_scale[row] = weights[p];
    }
    pair_row[p] = row;
  }
}

__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ h, const int* __restrict__ row_pair,
                                  __nv_bfloat16* __restrict__ rows, int top, int width8) {
  const int r = blockIdx.x;
  const int p = row_pair[r];
  const uint4* src = p >= 0 ? reinterpret_cast<const uint4*>(h) + (size_t)(p / top) * width8 : nullptr;
  uint4* dst = reinterpret_cast<uint4*>(rows) + (size_t)r * width8;
  for (int i = threadIdx.x; i < width8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

template <typename TO>
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ y,
                                   const int* __restrict__ ids, const float* __restrict__ weights,
                                   const int* __restrict__ pair_row, TO* __restrict__ out, int top, int experts,
                                   int width) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int p = t * top + k;
      const int row = pair_row[p];
      if (row >= 0) acc += y[(size_t)row * width + c];
      else acc = fmaf(weights[p], to_f32(h[(size_t)t * width + c]), acc);
    }
    out[(size_t)t * width + c] = from_f32<TO>(acc);
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// kind: 0 softmax over all, 1 softmax over the chosen, 2 sigmoid scores over the chosen scores' sum + floor.
int ifx_moe_route_kind(const float* z, const float* correction, int* ids, float* weights, int T, int n, int top,
                       int kind, float floor, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n <= 0 || top <= 0 || top > n || kind < 0 || kind > 2) return IFX_E_BADARG;
  if (n > kMaxRouterOutputs) return IFX_E_TOOBIG;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, stream>>>(z, correction, ids, weights, T, n, top, kind, floor);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_moe_route_ex(const float* z, const float* correction, int* ids, float* weights, int T, int n, int top,
                     int of_chosen, cudaStream_t stream) {
  return ifx_moe_route_kind(z, correction, ids, weights, T, n, top, of_chosen ? 1 : 0, 0.0f, stream);
}

int ifx_moe_route(const float* z, const float* correction, int* ids, float* weights, int T, int n, int top,
                  cudaStream_t stream) {
  return ifx_moe_route_ex(z, correction, ids, weights, T, n, top, 0, stream);
}

// h [T, width], act [T * top, ff] in `dtype`; out [T, width] in out_dtype.
int ifx_moe_experts_ex(const void* h, const void* w_up, const void* w_down, const int* ids, const float* weights,
                       void* act, void* out, int T, int top, int experts, int width, int ff, int dtype, int out_dtype,
                       int glu, float limit, float slope, cudaStream_t stream);
int ifx_moe_experts_glu(const void* h, const void* w_up, const void* w_down, const int* ids, const float* weights,
                        void* act, void* out, int T, int top, int experts, int width, int ff, int dtype, int out_dtype,
                        int glu, float limit, float slope, float offset, cudaStream_t stream);

int ifx_moe_experts(const void* h, const void* w_up, const void* w_down, const int* ids, const float* weights,
                    void* act, void* out, int T, int top, int experts, int width, int ff, int dtype, int out_dtype,
                    cudaStream_t stream) {
  return ifx_moe_experts_ex(h, w_up, w_down, ids, weights, act, out, T, top, experts, width, ff, dtype, out_dtype, 0, 0.0f,
                            0.0f, stream);
}

int ifx_moe_experts_ex(const void* h, const void* w_up, const void* w_down, const int* ids, const float* weights,
                       void* act, void* out, int T, int top, int experts, int width, int ff, int dtype, int out_dtype,
                       int glu, float limit, float slope, cudaStream_t stream) {
  return ifx_moe_experts_glu(h, w_up, w_down, ids, weights, act, out, T, top, experts, width, ff, dtype, out_dtype, glu, limit,
                             slope, 1.0f, stream);
}

// glu: w_up is [experts, 2 ff, width], an expert's gate rows above its up rows, and the activation is the gated one,
// g sigmoid(slope g) (u + offset) with g cut at limit from above and u on both sides (limit +inf: nothing is cut).
int ifx_moe_experts_glu(const void* h, const void* w_up, const void* w_down, const int* ids, const float* weights,
                        void* act, void* out, int T, int top, int experts, int width, int ff, int dtype, int out_dtype,
                        int glu, float limit, float slope, float offset, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || experts < 0 || width <= 0 || ff <= 0) return IFX_E_BADARG;
  if ((size_t)width * 4 > 160 * 1024 || (size_t)ff * 4 > 160 * 1024) return IFX_E_TOOBIG;
  const int up_rows = 32, down_rows = T <= 64 ? 32 : 64;  // few tokens: more blocks, so that more bytes are in flight
  dim3 grid_up(T * top, (ff + up_rows - 1) / up_rows), grid_down(T, (width + down_rows - 1) / down_rows);
  const size_t smem_up = (size_t)width * 4, smem_down = (size_t)ff * 4;
#define IFX_MOE(TT, TO)                                                                                           \
  do {                                                                                                            \
    if (experts > 0) {                                                                                            \
      auto up = glu ? moe_up_kernel<TT, true> : moe_up_kernel<TT, false>;                                         \
      if (smem_up > 48 * 1024) cudaFuncSetAttribute(up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up); \
      up<<<grid_up, kMoeWarps * 32, smem_up, stream>>>((const TT*)h, (const TT*)w_up, ids, (TT*)act, top, experts, \
                                                       width, ff, up_rows, limit, slope, offset);                         \
    }                                                                                                             \
    auto down = moe_down_kernel<TT, TO>;                                                                          \
    if (smem_down > 48 * 1024)                                                                                    \
      cudaFuncSetAttribute(down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);                    \
    down<<<grid_down, kMoeWarps * 32, smem_down, stream>>>((const TT*)h, (const TT*)act, (const TT*)w_down, ids,  \
                                                           weights, (TO*)out, top, experts, width, ff, down_rows); \
  } while (0)
  if (dtype == IFX_DT_F32 && out_dtype == IFX_DT_F32) IFX_MOE(float, float);
  else if (dtype == IFX_DT_BF16 && out_dtype == IFX_DT_BF16) IFX_MOE(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == IFX_DT_BF16 && out_dtype == IFX_DT_F32) IFX_MOE(__nv_bfloat16, float);
  else return IFX_E_DTYPE;
#undef IFX_MOE
  IFX_CHECK_LAUNCH();
  return 0;
}

// Rows that the sorted form needs at most: every expert's stretch is rounded up to whole tiles of 128.
int ifx_moe_sorted_rows(int pairs, int experts) {
  return (pairs + experts * 127 + 127) / 128 * 128;
}

int ifx_moe_sort(const int* ids, const float* weights, int pairs, int experts, int* row_pair, float* row_scale,
                 int* tile_group, int* pair_row, int rows_cap, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (experts <= 0 || experts > kMaxRouterOutputs || rows_cap % 128 || rows_cap < ifx_moe_sorted_rows(pairs, experts))
    return IFX_E_BADARG;
  moe_sort_kernel<<<1, 1024, 0, stream>>>(ids, weights, pairs, experts, row_pair, row_scale, tile_group, pair_row, rows_cap);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_moe_gather(const void* h, const int* row_pair, void* rows, int rows_cap, int top, int width, cudaStream_t stream) {
  if (rows_cap <= 0) return 0;
  if (width % 8 || (uintptr_t)h % 16 || (uintptr_t)rows % 16) return IFX_E_ALIGN;
  moe_gather_kernel<<<rows_cap, 128, 0, stream>>>((const __nv_bfloat16*)h, row_pair, (__nv_bfloat16*)rows, top, width / 8);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_moe_combine(const void* h, const float* y, const int* ids, const float* weights, const int* pair_row, void* out,
                    int T, int top, int experts, int width, int out_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (out_dtype == IFX_DT_BF16)
    moe_combine_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>((const __nv_bfloat16*)h, y, ids, weights, pair_row,
                                                             (__nv_bfloat16*)out, top, experts, width);
  else if (out_dtype == IFX_DT_F32)
    moe_combine_kernel<float><<<T, 256, 0, stream>>>((const __nv_bfloat16*)h, y, ids, weights, pair_row, (float*)out, top,
                                                     experts, width);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
