// Differential attention over the paged cache: every query head carries TWO query maps and every key head two key
// maps; each pair (query map m, key map m) is a causal softmax attention of its own over the SAME values, with the
// scores capped softly, s <- cap * tanh(s * scale / cap); the head's result is
//     o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale,   o <- o * sigmoid(gate)
// (lambda one number per layer).  Beside it, the kernel that prepares its operands: rotation of the first
// `rotary_dim` columns of every query and key map (neighbouring columns paired, or the two halves) and the store of
// the rotated keys and the values into their pages.
//
// Row of the projection: [q: hq * 2 * dk | k: hkv * 2 * dk | v: hkv * dv | ...] (k and v absent in a layer that reads
// another layer's pages).  Page layout: [kv_heads, block_size, 2 * dk] keys, then [kv_heads, block_size, dv] values.
// Scores, the caps, maxima, sums, both accumulators, the difference, the norm and the gate are fp32; keys are taken
// in blocks of 32 aligned to absolute positions, so a result depends neither on how the request was cut into steps
// nor on the rest of the batch.  One warp per (token, query head).
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_DK = 256;     // width of one map
constexpr int MAX_DV = 256;

// One warp per (token, unit): a query map, a key map or a value head.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
diff_rope_store_kernel(T* __restrict__ proj, int64_t stride, const int* __restrict__ positions,
                       const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping, T* __restrict__ cache,
                       int n_tokens, int hq, int hkv, int dk, int dv, int rotary_dim, int interleaved, int own_kv,
                       int block_size, int num_pages, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_units = 2 * hq, k_units = own_kv ? 2 * hkv : 0, v_units = own_kv ? hkv : 0;
  const int per_token = q_units + k_units + v_units;
  const int64_t item = (int64_t)blockIdx.x * WARPS + warp;
  if (item >= (int64_t)n_tokens * per_token) return;
  const int n = (int)(item / per_token), u = (int)(item - (int64_t)n * per_token);
  T* row = proj + (int64_t)n * stride;
  const size_t page_elems = (size_t)hkv * block_size * (2 * dk + dv);
  int64_t dst = -1;
  if (u >= q_units) {
    if (slot_mapping == nullptr) return;
    const int slot = slot_mapping[n];
    if (slot < 0) return;
    const int page = slot / block_size, off = slot % block_size;
    if (page >= num_pages) {
      if (lane == 0) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      return;
    }
    if (u < q_units + k_units) {
      const int ku = u - q_units;                  // key head ku / 2, map ku % 2
      dst = (int64_t)((size_t)page * page_elems + ((size_t)(ku >> 1) * block_size + off) * 2 * dk + (size_t)(ku & 1) * dk);
    } else {
      dst = (int64_t)((size_t)page * page_elems + (size_t)hkv * block_size * 2 * dk +
                      ((size_t)(u - q_units - k_units) * block_size + off) * dv);
    }
  }
  if (u >= q_units + k_units) {                    // a value head: stored as it is
    const T* src = row + (int64_t)(q_units + k_units) * dk + (int64_t)(u - q_units - k_units) * dv;
    for (int c = lane; c < dv; c += 32) cache[dst + c] = src[c];
    return;
  }
  T* x = row + (int64_t)u * dk;                    // query maps, then key maps, lie one after the other
  const float pos = (float)positions[n];
  const int half = rotary_dim / 2;
  for (int i = lane; i < half; i += 32) {
    const float ang = pos * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    const float x0 = to_float(x[i0]), x1 = to_float(x[i1]);
    const T r0 = from_float<T>(x0 * c - x1 * s), r1 = from_float<T>(x1 * c + x0 * s);
    if (dst < 0) {
      x[i0] = r0;
      x[i1] = r1;
    } else {
      cache[dst + i0] = r0;
      cache[dst + i1] = r1;
    }
  }
  if (dst >= 0)
    for (int c = rotary_dim + lane; c < dk; c += 32) cache[dst + c] = x[c];
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_diff_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ gate, int64_t gate_stride,
                      T* __restrict__ out, int64_t out_stride, const T* __restrict__ cache,
                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ positions,
                      const int* __restrict__ token_row, int n_tokens, int hq, int hkv, int dk, int dv, int block_size,
                      int num_pages, float scale, float softcap, float lambda, float eps, float out_scale,
                      int* __restrict__ status) {
  __shared__ float q_s[WARPS][2 * MAX_DK];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * WARPS + warp;
  if (item >= (int64_t)n_tokens * hq) return;
  const int n = (int)(item / hq), h = (int)(item - (int64_t)n * hq);
  const int kvh = h / (hq / hkv);
  const int qpos = positions[n];
  const int* bt = block_table + (int64_t)token_row[n] * bt_stride;
  const T* qv = q + (int64_t)n * q_stride + (int64_t)h * 2 * dk;
  for (int i = lane; i < 2 * dk; i += 32) q_s[warp][i] = to_float(qv[i]);
  __syncwarp();
  const size_t page_elems = (size_t)hkv * block_size * (2 * dk + dv);
  const size_t v_base = (size_t)hkv * block_size * 2 * dk;
  const float inv_cap = 1.0f / softcap;
  float acc1[MAX_DV / 32], acc2[MAX_DV / 32];
#pragma unroll
  for (int i = 0; i < MAX_DV / 32; ++i) acc1[i] = acc2[i] = 0.f;
  float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, l1 = 0.f, l2 = 0.f;
  for (int j0 = 0; j0 <= qpos; j0 += 32) {
    const int j = j0 + lane;
    float s1 = -CUDART_INF_F, s2 = -CUDART_INF_F;
    int64_t vbase = -1;
    if (j <= qpos) {
      const int page = bt[j / block_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      } else {
        const int off = j % block_size;
        const T* kp = cache + (size_t)page * page_elems + ((size_t)kvh * block_size + off) * 2 * dk;
        float d1 = 0.f, d2 = 0.f;
        for (int i = 0; i < dk; ++i) {
          d1 = fmaf(q_s[warp][i], to_float(kp[i]), d1);
          d2 = fmaf(q_s[warp][dk + i], to_float(kp[dk + i]), d2);
        }
        s1 = softcap * tanhf(d1 * scale * inv_cap);
        s2 = softcap * tanhf(d2 * scale * inv_cap);
        vbase = (int64_t)((size_t)page * page_elems + v_base + ((size_t)kvh * block_size + off) * dv);
      }
    }
    // the block's maxima join the running ones; what has been summed so far is brought to the new reference
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float r1 = n1 == -CUDART_INF_F ? 1.f : expf(m1 - n1), r2 = n2 == -CUDART_INF_F ? 1.f : expf(m2 - n2);
    const float p1 = vbase < 0 ? 0.f : expf(s1 - n1), p2 = vbase < 0 ? 0.f : expf(s2 - n2);
    l1 = l1 * r1 + warp_sum(p1);
    l2 = l2 * r2 + warp_sum(p2);
    m1 = n1;
    m2 = n2;
#pragma unroll
    for (int i = 0; i < MAX_DV / 32; ++i) {
      acc1[i] *= r1;
      acc2[i] *= r2;
    }
    const int count = min(32, qpos - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj1 = __shfl_sync(0xffffffffu, p1, jj), pj2 = __shfl_sync(0xffffffffu, p2, jj);
      const int64_t vb = __shfl_sync(0xffffffffu, vbase, jj);
      if (vb < 0) continue;
      const T* vp = cache + vb;
#pragma unroll
      for (int i = 0; i < MAX_DV / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) {
          const float v = to_float(vp[c]);
          acc1[i] = fmaf(pj1, v, acc1[i]);
          acc2[i] = fmaf(pj2, v, acc2[i]);
        }
      }
    }
  }
  const float i1 = l1 > 0.f ? 1.0f / l1 : 0.f, i2 = l2 > 0.f ? lambda / l2 : 0.f;
  float o[MAX_DV / 32], ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_DV / 32; ++i) {
    o[i] = lane + 32 * i < dv ? acc1[i] * i1 - acc2[i] * i2 : 0.f;
    ss = fmaf(o[i], o[i], ss);
  }
  ss = warp_sum(ss);
  const float mult = out_scale / sqrtf(ss / (float)dv + eps);
  T* orow = out + (int64_t)n * out_stride + (int64_t)h * dv;
  const T* grow = gate ? gate + (int64_t)n * gate_stride + (int64_t)h * dv : nullptr;
#pragma unroll
  for (int i = 0; i < MAX_DV / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) {
      float v = o[i] * mult;
      if (grow) v *= 1.0f / (1.0f + expf(-to_float(grow[c])));
      orow[c] = from_float<T>(v);
    }
  }
}

template <typename T>
int diff_rope_store_launch(T* proj, int64_t stride, const int* positions, const float* inv_freq,
                           const int* slot_mapping, T* cache, int n_tokens, int hq, int hkv, int dk, int dv,
                           int rotary_dim, int interleaved, int own_kv, int block_size, int num_pages, int* status,
                           cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || dk <= 0 || dv <= 0 || rotary_dim < 0 || rotary_dim > dk || (rotary_dim & 1) ||
      (rotary_dim > 0 && inv_freq == nullptr) || (slot_mapping != nullptr && block_size <= 0))
    return (int)cudaErrorInvalidValue;
  const int per_token = 2 * hq + (own_kv ? 3 * hkv : 0);
  const int64_t blocks = ((int64_t)n_tokens * per_token + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(diff_rope_store_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, proj, stride,
                     positions, inv_freq, slot_mapping, cache, n_tokens, hq, hkv, dk, dv, rotary_dim, interleaved, own_kv,
                     block_size, num_pages, status);
}

template <typename T>
int attention_diff_launch(const T* q, int64_t q_stride, const T* gate, int64_t gate_stride, T* out, int64_t out_stride,
                          const T* cache, const int* block_table, int bt_stride, const int* positions,
                          const int* token_row, int n_tokens, int hq, int hkv, int dk, int dv, int block_size,
                          int num_pages, float scale, float softcap, float lambda, float eps, float out_scale,
                          int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dk > MAX_DK || dv <= 0 || dv > MAX_DV || hq <= 0 || hkv <= 0 || hq % hkv || !(softcap > 0.f))
    return (int)cudaErrorInvalidValue;
  const int64_t blocks = ((int64_t)n_tokens * hq + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(attention_diff_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, q, q_stride, gate,
                     gate_stride, out, out_stride, cache, block_table, bt_stride, positions, token_row, n_tokens, hq, hkv,
                     dk, dv, block_size, num_pages, scale, softcap, lambda, eps, out_scale, status);
}
}  // namespace

#define GLLM_DIFF_EXPORTS(T, S)                                                                                        \
  GLLM_API int gllm_diff_rope_store_##S(T* proj, int64_t stride, const int* positions, const float* inv_freq,          \
                                        const int* slot_mapping, T* cache, int n_tokens, int hq, int hkv, int dk,      \
                                        int dv, int rotary_dim, int interleaved, int own_kv, int block_size,           \
                                        int num_pages, int* status, cudaStream_t stream) {                             \
    return diff_rope_store_launch<T>(proj, stride, positions, inv_freq, slot_mapping, cache, n_tokens, hq, hkv, dk, dv, \
                                     rotary_dim, interleaved, own_kv, block_size, num_pages, status, stream);          \
  }                                                                                                                    \
  GLLM_API int gllm_attention_diff_##S(const T* q, int64_t q_stride, const T* gate, int64_t gate_stride, T* out,       \
                                       int64_t out_stride, const T* cache, const int* block_table, int bt_stride,      \
                                       const int* positions, const int* token_row, int n_tokens, int hq, int hkv,      \
                                       int dk, int dv, int block_size, int num_pages, float scale, float softcap,      \
                                       float lambda, float eps, float out_scale, int* status, cudaStream_t stream) {   \
    return attention_diff_launch<T>(q, q_stride, gate, gate_stride, out, out_stride, cache, block_table, bt_stride,    \
                                    positions, token_row, n_tokens, hq, hkv, dk, dv, block_size, num_pages, scale,     \
                                    softcap, lambda, eps, out_scale, status, stream);                                  \
  }

GLLM_DIFF_EXPORTS(float, f32)
GLLM_DIFF_EXPORTS(__nv_bfloat16, bf16)
