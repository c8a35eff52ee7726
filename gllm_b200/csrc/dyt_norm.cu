// A norm that takes no statistic of its row ("dynamic tanh"), fused with the residual add:
//     resid += branch            (fp32, in place)
//     out = tanh(alpha * resid) * weight + bias
// alpha is one learned number (read from device memory), weight and bias one value per column.  With `rows` only
// those rows are computed and the residual stays as it is (the final norm at the rows whose logits are wanted).
// The branch may come as `n_parts` fp32 partial sums of a product cut along K ([part][row][hidden]): they are added
// in ascending order and rounded to T first, as the product itself would have rounded its result.
// Nothing couples the columns of a row, so the kernel is a flat sweep: one thread per four neighbouring columns when
// the row length allows 16-byte accesses, one per column otherwise.
#include "common.cuh"

namespace {

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
    v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<const uint32_t*>(&a);
    x.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
};

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
add_dyt_kernel(const T* __restrict__ branch, const float* __restrict__ parts, int n_parts, int64_t part_stride,
               float* __restrict__ resid, const float* __restrict__ alpha_p, const float* __restrict__ weight,
               const float* __restrict__ bias, T* __restrict__ out, const int* __restrict__ rows, int n_rows,
               int hidden) {
  pdl_trigger();
  const int per_row = hidden / VEC;
  const int64_t total = (int64_t)n_rows * per_row;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = (int)(idx / per_row), c = (int)(idx - (int64_t)i * per_row) * VEC;
  // alpha, weight and bias never depend on the kernel before this one: they are fetched before the wait
  const float alpha = alpha_p[0];
  float w[VEC], b[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    w[e] = weight[c + e];
    b[e] = bias ? bias[c + e] : 0.f;
  }
  pdl_wait();
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;
  float* res = resid + r * hidden + c;
  float x[VEC], y[VEC];
  if constexpr (VEC == 4) {
    Vec4<float>::load(res, x);
  } else {
    x[0] = res[0];
  }
  if (parts) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      x[e] += to_float(from_float<T>(sum_parts16(parts + r * hidden + c + e, n_parts, part_stride)));
  } else if (branch) {
    if constexpr (VEC == 4) {
      float v[4];
      Vec4<T>::load(branch + r * hidden + c, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] += v[e];
    } else {
      x[0] += to_float(branch[r * hidden + c]);
    }
  }
  if ((parts || branch) && !rows) {
    if constexpr (VEC == 4) Vec4<float>::store(res, x);
    else res[0] = x[0];
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) y[e] = fmaf(tanhf(alpha * x[e]), w[e], b[e]);
  T* o = out + (size_t)i * hidden + c;
  if constexpr (VEC == 4) Vec4<T>::store(o, y);
  else o[0] = from_float<T>(y[0]);
}

template <typename T>
int add_dyt_launch(const T* branch, const float* parts, int n_parts, int64_t part_stride, float* resid,
                   const float* alpha, const float* weight, const float* bias, T* out, const int* rows, int n_rows,
                   int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || n_parts > 16 || alpha == nullptr) return (int)cudaErrorInvalidValue;
  const bool vec = hidden % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(branch) | reinterpret_cast<uintptr_t>(resid) |
                     reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const int64_t total = (int64_t)n_rows * (vec ? hidden / 4 : hidden);
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (vec)
    return gllm_launch(add_dyt_kernel<T, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, branch, parts, n_parts,
                       part_stride, resid, alpha, weight, bias, out, rows, n_rows, hidden);
  return gllm_launch(add_dyt_kernel<T, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, branch, parts, n_parts,
                     part_stride, resid, alpha, weight, bias, out, rows, n_rows, hidden);
}
}  // namespace

GLLM_API int gllm_add_dyt_f32(const float* branch, const float* parts, int n_parts, int64_t part_stride, float* resid,
                              const float* alpha, const float* weight, const float* bias, float* out, const int* rows,
                              int n_rows, int hidden, cudaStream_t stream) {
  return add_dyt_launch<float>(branch, parts, n_parts, part_stride, resid, alpha, weight, bias, out, rows, n_rows,
                               hidden, stream);
}
GLLM_API int gllm_add_dyt_bf16(const __nv_bfloat16* branch, const float* parts, int n_parts, int64_t part_stride,
                               float* resid, const float* alpha, const float* weight, const float* bias,
                               __nv_bfloat16* out, const int* rows, int n_rows, int hidden, cudaStream_t stream) {
  return add_dyt_launch<__nv_bfloat16>(branch, parts, n_parts, part_stride, resid, alpha, weight, bias, out, rows,
                                       n_rows, hidden, stream);
}
