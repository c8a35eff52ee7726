// The norm kernel of layers that norm a sublayer's result before it joins the residual ("sandwich" norms):
//   resid[r] += value[r] / sqrt(mean(value[r]^2) + post_eps) * post_w  (+ extra[r]);   out[r] = rms(resid[r]) * w
// (without post_w the value is added as it is; value and extra may each be absent) in one pass over the row: the add that the pre-norm layers defer to the next norm's kernel is deferred here
// as well, together with the norm of what is added.  `value` may arrive as unsummed fp32 splits of a product
// (summed in ascending order and rounded to T, as the product would have); `extra` is a second fp32 stream
// that is added as it is (the embedding output that a repeated stretch of layers takes in again).  With
// `rows` only those rows are normed and resid stays untouched (the final norm at the wanted rows).
// Statistics, the normed value and the sums are fp32 whatever T is.
#include "common.cuh"

namespace {

// VEC consecutive columns of a row, to and from fp32 (VEC = 4 wants the address aligned to 4 elements).
template <int VEC> __device__ __forceinline__ void load_cols(const float* p, float (&v)[VEC]) {
  if (VEC == 4) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x, v[VEC > 1 ? 1 : 0] = x.y, v[VEC > 2 ? 2 : 0] = x.z, v[VEC > 3 ? 3 : 0] = x.w;
  } else {
    v[0] = p[0];
  }
}
template <int VEC> __device__ __forceinline__ void load_cols(const __nv_bfloat16* p, float (&v)[VEC]) {
  if (VEC == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = lo.x, v[VEC > 1 ? 1 : 0] = lo.y, v[VEC > 2 ? 2 : 0] = hi.x, v[VEC > 3 ? 3 : 0] = hi.y;
  } else {
    v[0] = __bfloat162float(p[0]);
  }
}
template <int VEC> __device__ __forceinline__ void store_cols(float* p, const float (&v)[VEC]) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[VEC > 1 ? 1 : 0], v[VEC > 2 ? 2 : 0], v[VEC > 3 ? 3 : 0]);
  else p[0] = v[0];
}
template <int VEC> __device__ __forceinline__ void store_cols(__nv_bfloat16* p, const float (&v)[VEC]) {
  if (VEC == 4) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[VEC > 1 ? 1 : 0]);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[VEC > 2 ? 2 : 0], v[VEC > 3 ? 3 : 0]);
    *reinterpret_cast<uint2*>(p) = raw;
  } else {
    p[0] = __float2bfloat16(v[0]);
  }
}

// A thread takes VEC consecutive columns at a time (VEC = 4 when the rows hold a multiple of 4 columns).
template <typename T, int VEC>
__global__ void __launch_bounds__(1024)
postnorm_add_rmsnorm_kernel(const T* __restrict__ value, const float* __restrict__ parts, int n_parts,
                            int64_t part_stride, const float* __restrict__ post_w, float post_eps,
                            const float* __restrict__ extra, float* __restrict__ resid, const float* __restrict__ w,
                            float eps, T* __restrict__ out, const int* __restrict__ rows, int n_rows, int hidden) {
  extern __shared__ __align__(16) float xs[];
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int64_t r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* x = resid + r * hidden;
  const bool has_value = value != nullptr || parts != nullptr;
  const int first = threadIdx.x * VEC, stride = blockDim.x * VEC;
  float inv1 = 1.f;
  if (has_value) {
    float ss = 0.f;
    for (int c = first; c < hidden; c += stride) {
      float v[VEC];
      if (parts) {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          v[e] = to_float(from_float<T>(sum_parts16(parts + r * hidden + c + e, n_parts, part_stride)));
      } else {
        load_cols<VEC>(value + r * hidden + c, v);
      }
      store_cols<VEC>(xs + c, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(v[e], v[e], ss);
    }
    if (post_w) {
      ss = block_sum(ss, scratch);
      inv1 = 1.0f / sqrtf(ss / (float)hidden + post_eps);
    }
  }
  float ss2 = 0.f;
  for (int c = first; c < hidden; c += stride) {
    float v[VEC];
    load_cols<VEC>((const float*)x + c, v);
    if (has_value) {
      float a[VEC];
      load_cols<VEC>((const float*)xs + c, a);
      if (post_w) {
        float pw[VEC];
        load_cols<VEC>(post_w + c, pw);
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] += a[e] * inv1 * pw[e];
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] += a[e];
      }
    }
    if (extra) {
      float a[VEC];
      load_cols<VEC>(extra + r * hidden + c, a);
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] += a[e];
    }
    store_cols<VEC>(xs + c, v);
    if (!rows) store_cols<VEC>(x + c, v);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ss2 = fmaf(v[e], v[e], ss2);
  }
  if (!w) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)hidden + eps);
  T* o = out + (int64_t)blockIdx.x * hidden;
  for (int c = first; c < hidden; c += stride) {
    float v[VEC], ww[VEC];
    load_cols<VEC>((const float*)xs + c, v);
    load_cols<VEC>(w + c, ww);
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = v[e] * inv2 * ww[e];
    store_cols<VEC>(o + c, v);
  }
}

template <typename T>
int postnorm_launch(const T* value, const float* parts, int n_parts, int64_t part_stride, const float* post_w,
                    float post_eps, const float* extra, float* resid, const float* w, float eps, T* out,
                    const int* rows, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = sizeof(float) * (size_t)hidden;
  if (smem > 200 * 1024 || n_parts > 16) return (int)cudaErrorInvalidValue;
  auto misaligned = [](const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  const bool vec = hidden % 4 == 0 && !misaligned(value) && !misaligned(post_w) && !misaligned(extra) &&
                   !misaligned(resid) && !misaligned(w) && !misaligned(out) &&
                   (value == nullptr || (reinterpret_cast<uintptr_t>(value) & 7) == 0);
  auto kernel = vec ? postnorm_add_rmsnorm_kernel<T, 4> : postnorm_add_rmsnorm_kernel<T, 1>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  // few rows: a row's three passes are chains of loads, so more threads make each chain shorter
  int threads = n_rows <= 64 && hidden > 1024 ? 1024 : 256;
  if (vec) threads = std::max(64, std::min(threads, (hidden / 4 + 31) / 32 * 32));
  return gllm_launch(kernel, dim3(n_rows), dim3(threads), smem, stream, value, parts, n_parts, part_stride, post_w,
                     post_eps, extra, resid, w, eps, out, rows, n_rows, hidden);
}
}  // namespace

GLLM_API int gllm_postnorm_add_rmsnorm_f32(const float* value, const float* parts, int n_parts, int64_t part_stride,
                                           const float* post_w, float post_eps, const float* extra, float* resid,
                                           const float* w, float eps, float* out, const int* rows, int n_rows,
                                           int hidden, cudaStream_t stream) {
  return postnorm_launch<float>(value, parts, n_parts, part_stride, post_w, post_eps, extra, resid, w, eps, out, rows,
                                n_rows, hidden, stream);
}
GLLM_API int gllm_postnorm_add_rmsnorm_bf16(const __nv_bfloat16* value, const float* parts, int n_parts,
                                            int64_t part_stride, const float* post_w, float post_eps,
                                            const float* extra, float* resid, const float* w, float eps,
                                            __nv_bfloat16* out, const int* rows, int n_rows, int hidden,
                                            cudaStream_t stream) {
  return postnorm_launch<__nv_bfloat16>(value, parts, n_parts, part_stride, post_w, post_eps, extra, resid, w, eps, out,
                                        rows, n_rows, hidden, stream);
}
