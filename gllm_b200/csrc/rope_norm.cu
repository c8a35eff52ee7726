// Rotation, norm and cache store of one attention layer's projections in one kernel, for layers whose
// queries and keys are normed AFTER the rotation and whose sine and cosine carry a multiplier.
// qkv is [n, (hq + 2*hkv) * d]: q heads, k heads, v heads.  One warp per (token, head):
//   q, k: the first rotary_dim columns turn in pairs (neighbours (2i, 2i+1) when `interleaved`, else the two
//         halves (i, i + rotary_dim/2)) by position * inv_freq[i], sine and cosine times `magnitude`; then,
//         with norm_dim > 0, the head is divided by sqrt(sum(x^2) / norm_dim + eps) (an RMS norm without a
//         weight; norm_dim may be less than d when the head is stored with zero columns behind it);
//   k, v: stored into the token's cache slot, layout [page][k|v][kv_head][block_size][d].
// Angles, sine, cosine, the rotation and the norm are fp32; the result is rounded to T once.
// qkv may arrive as unsummed fp32 splits of the projection (summed in ascending order, rounded to T first).
#include "common.cuh"

namespace {
constexpr int RN_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(128)
rope_norm_store_kernel(T* __restrict__ qkv, const float* __restrict__ parts, int n_parts, int64_t part_stride,
                       const int* __restrict__ positions, const float* __restrict__ inv_freq, float magnitude,
                       const int* __restrict__ slot_mapping, T* __restrict__ cache, int n_tokens, int hq, int hkv,
                       int d, int rotary_dim, int interleaved, int norm_dim, float eps, int block_size, int num_pages,
                       int* __restrict__ status) {
  __shared__ float sm[4][RN_MAX_D];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = hq + 2 * hkv;
  const int64_t item = (int64_t)blockIdx.x * 4 + warp;
  if (item >= (int64_t)n_tokens * heads) return;
  const int n = (int)(item / heads), h = (int)(item - (int64_t)n * heads);
  const int64_t width = (int64_t)heads * d;
  T* row = qkv + n * width + (int64_t)h * d;
  float* x = sm[warp];
  for (int c = lane; c < d; c += 32)
    x[c] = parts ? to_float(from_float<T>(sum_parts16(parts + n * width + (int64_t)h * d + c, n_parts, part_stride)))
                 : to_float(row[c]);
  __syncwarp();
  float inv = 1.0f;
  if (h < hq + hkv) {
    if (inv_freq && rotary_dim > 0) {
      const float pos = (float)positions[n];
      const int half = rotary_dim / 2;
      for (int i = lane; i < half; i += 32) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        s *= magnitude;
        c *= magnitude;
        const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
        const float x0 = x[i0], x1 = x[i1];
        x[i0] = x0 * c - x1 * s;
        x[i1] = x1 * c + x0 * s;
      }
      __syncwarp();
    }
    if (norm_dim > 0) {
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) ss = fmaf(x[c], x[c], ss);
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)norm_dim + eps);
    }
  }
  T* dst = nullptr;
  if (h >= hq && slot_mapping) {
    const int slot = slot_mapping[n];
    if (slot >= 0) {
      const int page = slot / block_size, off = slot - page * block_size;
      if (page >= num_pages) {
        if (lane == 0) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      } else {
        const int kv = h - hq;                       // 0 .. hkv-1: keys, hkv .. 2 hkv-1: values
        dst = cache + (((int64_t)page * 2 * hkv + kv) * block_size + off) * d;
      }
    }
  }
  for (int c = lane; c < d; c += 32) {
    const T y = from_float<T>(x[c] * inv);
    row[c] = y;
    if (dst) dst[c] = y;
  }
}

template <typename T>
int rope_norm_store_launch(T* qkv, const float* parts, int n_parts, int64_t part_stride, const int* positions,
                           const float* inv_freq, float magnitude, const int* slot_mapping, T* cache, int n_tokens,
                           int hq, int hkv, int d, int rotary_dim, int interleaved, int norm_dim, float eps,
                           int block_size, int num_pages, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d < 1 || d > RN_MAX_D || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || n_parts > 16)
    return (int)cudaErrorInvalidValue;
  const int64_t blocks = ((int64_t)n_tokens * (hq + 2 * hkv) + 3) / 4;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(rope_norm_store_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, stream, qkv, parts, n_parts,
                     part_stride, positions, inv_freq, magnitude, slot_mapping, cache, n_tokens, hq, hkv, d, rotary_dim,
                     interleaved, norm_dim, eps, block_size, num_pages, status);
}
}  // namespace

GLLM_API int gllm_rope_norm_store_f32(float* qkv, const float* parts, int n_parts, int64_t part_stride,
                                      const int* positions, const float* inv_freq, float magnitude,
                                      const int* slot_mapping, float* cache, int n_tokens, int hq, int hkv, int d,
                                      int rotary_dim, int interleaved, int norm_dim, float eps, int block_size,
                                      int num_pages, int* status, cudaStream_t stream) {
  return rope_norm_store_launch<float>(qkv, parts, n_parts, part_stride, positions, inv_freq, magnitude, slot_mapping,
                                       cache, n_tokens, hq, hkv, d, rotary_dim, interleaved, norm_dim, eps, block_size,
                                       num_pages, status, stream);
}
GLLM_API int gllm_rope_norm_store_bf16(__nv_bfloat16* qkv, const float* parts, int n_parts, int64_t part_stride,
                                       const int* positions, const float* inv_freq, float magnitude,
                                       const int* slot_mapping, __nv_bfloat16* cache, int n_tokens, int hq, int hkv,
                                       int d, int rotary_dim, int interleaved, int norm_dim, float eps, int block_size,
                                       int num_pages, int* status, cudaStream_t stream) {
  return rope_norm_store_launch<__nv_bfloat16>(qkv, parts, n_parts, part_stride, positions, inv_freq, magnitude,
                                               slot_mapping, cache, n_tokens, hq, hkv, d, rotary_dim, interleaved,
                                               norm_dim, eps, block_size, num_pages, status, stream);
}
