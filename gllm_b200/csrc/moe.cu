// Routed experts: every token is served by `top` of `experts` small feed-forwards.
//   moe_route    per token (one warp): scores s = sigmoid(z) of the fp32 router logits, or softmax(z) over all
//                experts (`softmax_scores`); the choice is made on
//                s + correction, optionally only among the experts of the `keep` best of `groups` equal groups of
//                neighbours (a group's score: the sum of its two largest choice scores, or its largest alone with
//                `group_max`; experts of other groups
//                count as minus infinity); the weights are the chosen experts' s (divided by their sum + renorm_eps with
//                `renorm`), times `weight_scale`.  Ties go to the lower index.
//   moe_align    (one block) sorts the (token, slot) pairs by expert: every expert's pairs form whole tiles of
//                `tile_m` rows (the last one filled up with -1), so that a tile of the products below reads ONE
//                expert's weights; writes the pair of every row, the expert of every tile and the tile count.
//   moe_gemm     out[pair] = A[row of pair] @ W[expert]^T over the tiles; `gated`: W holds gate and up rows and
//                the result is silu(gate) * up, rounded to T; `act` 1 (experts without a gate): the square of
//                max(result, 0), rounded to T; otherwise the fp32 result itself.
//   moe_combine  out[token] = sum over its slots, in slot order, of weight * result[pair] (+ a shared expert's
//                result, times sigmoid(shared_gate[token]) when the shared expert has a gate), rounded to T.
// A pair's result does not depend on which other pairs share its tile or on the tile's place: every row is a dot
// product over K in one fixed order.  Scores, choice, weights, accumulators and the combination are fp32.
#include "common.cuh"
#include <math_constants.h>

namespace {

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

__global__ void __launch_bounds__(32)
moe_route_kernel(const float* __restrict__ logits, int64_t stride, const float* __restrict__ correction,
                 int* __restrict__ ids, float* __restrict__ weights, int experts, int top, int groups, int keep,
                 int renorm, int softmax_scores, int group_max, float renorm_eps, float weight_scale) {
  extern __shared__ float sm[];
  float* s = sm;                 // [experts] scores
  float* c = s + experts;        // [experts] choice scores
  float* gs = c + experts;       // [groups] group scores, then 1 = kept
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x, lane = threadIdx.x;
  float z_max = -CUDART_INF_F, z_sum = 0.f;
  if (softmax_scores) {
    for (int e = lane; e < experts; e += 32) z_max = fmaxf(z_max, logits[(int64_t)i * stride + e]);
    z_max = warp_max(z_max);
    for (int e = lane; e < experts; e += 32) {
      const float v = expf(logits[(int64_t)i * stride + e] - z_max);
      s[e] = v;
      z_sum += v;
    }
    z_sum = warp_sum(z_sum);
  }
  for (int e = lane; e < experts; e += 32) {
    const float z = logits[(int64_t)i * stride + e];
    const float v = softmax_scores ? s[e] / z_sum : 1.0f / (1.0f + expf(-z));
    s[e] = v;
    c[e] = v + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = c[e];
        if (v > m1) {
          m2 = m1;
          m1 = v;
        } else if (v > m2) {
          m2 = v;
        }
      }
      gs[g] = (per > 1 && !group_max) ? m1 + m2 : m1;
    }
    __syncwarp();
    // the `keep` best groups, one after the other; a kept group is marked by +inf ... then turned into a flag
    for (int r = 0; r < keep; ++r) {
      float best = -CUDART_INF_F;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != CUDART_INF_F && (v > best || bi == 0x7fffffff)) {
          best = v;
          bi = g;
        }
      }
      warp_argmax(best, bi);
      __syncwarp();
      if (lane == 0 && bi < groups) gs[bi] = CUDART_INF_F;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / per] != CUDART_INF_F) c[e] = -CUDART_INF_F;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = c[e];
      if (v > best) {
        best = v;
        bi = e;
      }
    }
    warp_argmax(best, bi);
    __syncwarp();
    if (bi >= experts) bi = 0;              // nothing left to choose (NaN logits): keep the indices in range
    if (lane == 0) {
      ids[(int64_t)i * top + r] = bi;
      weights[(int64_t)i * top + r] = s[bi];
      c[bi] = -CUDART_INF_F;
    }
    total += s[bi];
    __syncwarp();
  }
  if (renorm || weight_scale != 1.0f) {
    __syncwarp();
    for (int r = lane; r < top; r += 32) {
      float wv = weights[(int64_t)i * top + r];
      if (renorm) wv /= total + renorm_eps;
      weights[(int64_t)i * top + r] = wv * weight_scale;
    }
  }
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int* __restrict__ sorted, int* __restrict__ tile_expert,
                 int* __restrict__ num_tiles, int* __restrict__ row_of_pair, int n_pairs, int experts, int tile_m,
                 int max_tiles) {
  extern __shared__ int smi[];
  int* counts = smi;                  // [experts]
  int* first = counts + experts;      // [experts + 1] first row of every expert
  int* cursor = first + experts + 1;  // [experts]
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = at;
      at += (counts[e] + tile_m - 1) / tile_m * tile_m;
    }
    first[experts] = at;
    num_tiles[0] = min(at / tile_m, max_tiles);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    for (int t = first[e] / tile_m; t < first[e + 1] / tile_m && t < max_tiles; ++t) tile_expert[t] = e;
  for (int r = threadIdx.x; r < max_tiles * tile_m; r += blockDim.x) sorted[r] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e < 0 || e >= experts) continue;
    const int row = first[e] + atomicAdd(&cursor[e], 1);
    if (row < max_tiles * tile_m) sorted[row] = p;
    if (row_of_pair) row_of_pair[p] = min(row, max_tiles * tile_m - 1);
  }
}

// out[row_of_pair[p]] = x[p / top]: the tokens' rows in the order of the sorted pairs, for products that read
// their rows in place (16 bytes a thread; width * sizeof(T) is a multiple of 16).
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ x, int64_t x_stride, const int* __restrict__ row_of_pair, T* __restrict__ out,
                  int top, int width) {
  pdl_trigger();
  pdl_wait();
  const int p = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(p / top) * x_stride);
  uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)row_of_pair[p] * width);
  const int n16 = width * (int)sizeof(T) / 16;
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
}

constexpr int MG_M = 16, MG_N = 64, MG_K = 32, MG_THREADS = 128;

// grid (max_tiles, ceil(n_cols / MG_N)).  A row of pair p: a + (p / a_div) * a_stride.  W of expert e: w + e *
// w_expert_stride, rows of k columns; gated: up rows lie `up_offset` elements behind the gate rows.
template <typename T>
__global__ void __launch_bounds__(MG_THREADS)
moe_gemm_kernel(const T* __restrict__ a, int64_t a_stride, int a_div, const T* __restrict__ w, int64_t w_expert_stride,
                int64_t up_offset, const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                const int* __restrict__ num_tiles, T* __restrict__ out_t, float* __restrict__ out_f, int n_cols, int k,
                int act) {
  __shared__ float As[MG_M][MG_K + 1];
  __shared__ float Bs[MG_N][MG_K + 1];
  __shared__ float Us[MG_N][MG_K + 1];
  __shared__ int pairs[MG_M];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x;
  if (tile >= num_tiles[0]) return;
  const bool gated = up_offset != 0;
  const int tid = threadIdx.x;
  if (tid < MG_M) pairs[tid] = sorted[tile * MG_M + tid];
  __syncthreads();
  const T* we = w + (int64_t)tile_expert[tile] * w_expert_stride;
  const int col0 = blockIdx.y * MG_N;
  const int ty = tid / 16, tx = tid % 16;          // rows 2 ty, 2 ty + 1; columns tx, tx + 16, tx + 32, tx + 48
  float acc[2][4] = {}, acu[2][4] = {};
  for (int k0 = 0; k0 < k; k0 += MG_K) {
    for (int idx = tid; idx < MG_M * MG_K; idx += MG_THREADS) {
      const int r = idx / MG_K, kk = idx % MG_K;
      const int p = pairs[r];
      As[r][kk] = (p >= 0 && k0 + kk < k) ? to_float(a[(int64_t)(p / a_div) * a_stride + k0 + kk]) : 0.f;
    }
    for (int idx = tid; idx < MG_N * MG_K; idx += MG_THREADS) {
      const int c = idx / MG_K, kk = idx % MG_K;
      const bool ok = col0 + c < n_cols && k0 + kk < k;
      const int64_t at = (int64_t)(col0 + c) * k + k0 + kk;
      Bs[c][kk] = ok ? to_float(we[at]) : 0.f;
      if (gated) Us[c][kk] = ok ? to_float(we[up_offset + at]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < MG_K; ++kk) {
      const float a0 = As[2 * ty][kk], a1 = As[2 * ty + 1][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Bs[tx + 16 * j][kk];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
        if (gated) {
          const float u = Us[tx + 16 * j][kk];
          acu[0][j] = fmaf(a0, u, acu[0][j]);
          acu[1][j] = fmaf(a1, u, acu[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int p = pairs[2 * ty + i];
    if (p < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx + 16 * j;
      if (c >= n_cols) continue;
      if (gated) {
        const float g = acc[i][j];
        out_t[(int64_t)p * n_cols + c] = from_float<T>(g / (1.0f + expf(-g)) * acu[i][j]);
      } else if (act == 1) {
        const float r = fmaxf(acc[i][j], 0.f);
        out_t[(int64_t)p * n_cols + c] = from_float<T>(r * r);
      } else {
        out_f[(int64_t)p * n_cols + c] = acc[i][j];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, const T* __restrict__ shared,
                   T* __restrict__ out, const int* __restrict__ row_of_pair, int top, int width,
                   const float* __restrict__ shared_gate, int64_t shared_gate_stride) {
  pdl_trigger();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const float sg = (shared && shared_gate) ? 1.0f / (1.0f + expf(-shared_gate[t * shared_gate_stride])) : 1.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < top; ++s) {
      const int64_t row = row_of_pair ? (int64_t)row_of_pair[t * top + s] : t * top + s;
      acc = fmaf(weights[t * top + s], y[row * width + c], acc);
    }
    if (shared) acc = fmaf(sg, to_float(shared[t * width + c]), acc);
    out[t * width + c] = from_float<T>(acc);
  }
}

// out = max(in, 0)^2 rounded to T: the activation of experts without a gate, between the two tensor-core products.
template <typename T>
__global__ void __launch_bounds__(256)
moe_relu_sq_kernel(const float* __restrict__ in, T* __restrict__ out, int64_t n) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float r = fmaxf(in[i], 0.f);
    out[i] = from_float<T>(r * r);
  }
}

template <typename T>
int moe_gemm_launch(const T* a, int64_t a_stride, int a_div, const T* w, int64_t w_expert_stride, int64_t up_offset,
                    const int* sorted, const int* tile_expert, const int* num_tiles, void* out, int max_tiles,
                    int n_cols, int k, int tile_m, int act, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (tile_m != MG_M || n_cols < 1 || k < 1 || a_div < 1 || act < 0 || act > 1) return (int)cudaErrorInvalidValue;
  const bool gated = up_offset != 0 || act == 1;
  return gllm_launch(moe_gemm_kernel<T>, dim3(max_tiles, (n_cols + MG_N - 1) / MG_N), dim3(MG_THREADS), 0, stream, a,
                     a_stride, a_div, w, w_expert_stride, up_offset, sorted, tile_expert, num_tiles,
                     gated ? (T*)out : (T*)nullptr, gated ? (float*)nullptr : (float*)out, n_cols, k, act);
}
}  // namespace

GLLM_API int gllm_moe_route(const float* logits, int64_t stride, const float* correction, int* ids, float* weights,
                            int n_tokens, int experts, int top, int groups, int keep, int renorm, int softmax_scores,
                            int group_max, float renorm_eps, float weight_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (experts < 1 || top < 1 || top > experts || groups < 1 || experts % groups || keep < 1 || keep > groups ||
      top > keep * (experts / groups))
    return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (size_t)(2 * experts + groups);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  return gllm_launch(moe_route_kernel, dim3(n_tokens), dim3(32), smem, stream, logits, stride, correction, ids, weights,
                     experts, top, groups, keep, renorm, softmax_scores, group_max, renorm_eps, weight_scale);
}

GLLM_API int gllm_moe_align(const int* ids, int* sorted, int* tile_expert, int* num_tiles, int* row_of_pair,
                            int n_pairs, int experts, int tile_m, int max_tiles, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  const size_t smem = sizeof(int) * (size_t)(3 * experts + 1);
  if (smem > 48 * 1024 || tile_m < 1 || max_tiles < 1) return (int)cudaErrorInvalidValue;
  return gllm_launch(moe_align_kernel, dim3(1), dim3(1024), smem, stream, ids, sorted, tile_expert, num_tiles, row_of_pair,
                     n_pairs, experts, tile_m, max_tiles);
}

GLLM_API int gllm_moe_gemm_f32(const float* a, int64_t a_stride, int a_div, const float* w, int64_t w_expert_stride,
                               int64_t up_offset, const int* sorted, const int* tile_expert, const int* num_tiles,
                               void* out, int max_tiles, int n_cols, int k, int tile_m, int act, cudaStream_t stream) {
  return moe_gemm_launch<float>(a, a_stride, a_div, w, w_expert_stride, up_offset, sorted, tile_expert, num_tiles, out,
                                max_tiles, n_cols, k, tile_m, act, stream);
}
GLLM_API int gllm_moe_gemm_bf16(const __nv_bfloat16* a, int64_t a_stride, int a_div, const __nv_bfloat16* w,
                                int64_t w_expert_stride, int64_t up_offset, const int* sorted, const int* tile_expert,
                                const int* num_tiles, void* out, int max_tiles, int n_cols, int k, int tile_m,
                                int act, cudaStream_t stream) {
  return moe_gemm_launch<__nv_bfloat16>(a, a_stride, a_div, w, w_expert_stride, up_offset, sorted, tile_expert,
                                        num_tiles, out, max_tiles, n_cols, k, tile_m, act, stream);
}

GLLM_API int gllm_moe_combine_f32(const float* y, const float* weights, const float* shared, float* out,
                                  const int* row_of_pair, int n_tokens, int top, int width, const float* shared_gate,
                                  int64_t shared_gate_stride, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  return gllm_launch(moe_combine_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, y, weights, shared, out,
                     row_of_pair, top, width, shared_gate, shared_gate_stride);
}
GLLM_API int gllm_moe_combine_bf16(const float* y, const float* weights, const __nv_bfloat16* shared,
                                   __nv_bfloat16* out, const int* row_of_pair, int n_tokens, int top, int width,
                                   const float* shared_gate, int64_t shared_gate_stride, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  return gllm_launch(moe_combine_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, y, weights, shared, out,
                     row_of_pair, top, width, shared_gate, shared_gate_stride);
}
GLLM_API int gllm_moe_gather_bf16(const __nv_bfloat16* x, int64_t x_stride, const int* row_of_pair, __nv_bfloat16* out,
                                  int n_pairs, int top, int width, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (width % 8 || x_stride % 8 || top < 1 || (reinterpret_cast<uintptr_t>(x) & 15)) return (int)cudaErrorInvalidValue;
  return gllm_launch(moe_gather_kernel<__nv_bfloat16>, dim3(n_pairs), dim3(256), 0, stream, x, x_stride, row_of_pair, out,
                     top, width);
}

GLLM_API int gllm_moe_relu_sq_bf16(const float* in, __nv_bfloat16* out, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  int64_t blocks = (n + 255) / 256;
  if (blocks > (int64_t)gllm_sm_count() * 8) blocks = (int64_t)gllm_sm_count() * 8;
  return gllm_launch(moe_relu_sq_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, in, out, n);
}
