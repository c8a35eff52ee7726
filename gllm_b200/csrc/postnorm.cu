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

template <typename T>
__global__ void __launch_bounds__(1024)
postnorm_add_rmsnorm_kernel(const T* __restrict__ value, const float* __restrict__ parts, int n_parts,
                            int64_t part_stride, const float* __restrict__ post_w, float post_eps,
                            const float* __restrict__ extra, float* __restrict__ resid, const float* __restrict__ w,
                            float eps, T* __restrict__ out, const int* __restrict__ rows, int n_rows, int hidden) {
  extern __shared__ float xs[];
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int64_t r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* x = resid + r * hidden;
  const bool has_value = value != nullptr || parts != nullptr;
  float inv1 = 1.f;
  if (has_value) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = parts ? to_float(from_float<T>(sum_parts16(parts + r * hidden + c, n_parts, part_stride)))
                            : to_float(value[r * hidden + c]);
      xs[c] = v;
      ss = fmaf(v, v, ss);
    }
    if (post_w) {
      ss = block_sum(ss, scratch);
      inv1 = 1.0f / sqrtf(ss / (float)hidden + post_eps);
    }
  }
  float ss2 = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = x[c];
    if (has_value) v += post_w ? xs[c] * inv1 * post_w[c] : xs[c];
    if (extra) v += extra[r * hidden + c];
    xs[c] = v;
    if (!rows) x[c] = v;
    ss2 = fmaf(v, v, ss2);
  }
  if (!w) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)hidden + eps);
  T* o = out + (int64_t)blockIdx.x * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_float<T>(xs[c] * inv2 * w[c]);
}

template <typename T>
int postnorm_launch(const T* value, const float* parts, int n_parts, int64_t part_stride, const float* post_w,
                    float post_eps, const float* extra, float* resid, const float* w, float eps, T* out,
                    const int* rows, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = sizeof(float) * (size_t)hidden;
  if (smem > 200 * 1024 || n_parts > 16) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(postnorm_add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  // few rows: a row's three passes are chains of loads, so more threads make each chain shorter
  const int threads = n_rows <= 64 && hidden > 1024 ? 1024 : 256;
  return gllm_launch(postnorm_add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, stream, value, parts, n_parts,
                     part_stride, post_w, post_eps, extra, resid, w, eps, out, rows, n_rows, hidden);
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
