// The gated delta rule: a matrix state per head that forgets per key channel and is corrected, not just added to,
//   S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q,
// with everything but the projections in fp32.  Three kernels:
//   delta_prep         per token: the short causal convolution + SiLU of the q, k and v projections (over the
//                      request's own earlier tokens and its convolution state), q and k made unit vectors per head
//                      (q also times q_scale), the decays g = exp(-exp(A_log[h]) softplus(a + dt_bias)) and
//                      beta = sigmoid(b);
//   conv_state_update  per request: the last taps-1 inputs of the convolution become its new state;
//   delta_rule         per (request, head, block of value columns): the recurrence, token after token.
// Every value column of S obeys the same recurrence by itself (column c: s <- g s; u_c = beta (v_c - s.k);
// s <- s + k u_c; o_c = s.q), so a column is shared by `lanes` threads that each keep DPT of its key channels
// and add their parts of the two dot products by shuffles.  o_c is formed as (g s).q + u_c (k.q), which needs
// one round of shuffles per token instead of two.  The state is stored column by column, [slots, heads, dv, dk],
// as the other matrix recurrences store theirs.
// The flat batch holds prompt portions beside single tokens: request r owns rows cu_q[r] .. cu_q[r+1]-1 and row
// state_slots[r] of the state tensors, so a prompt may be cut anywhere.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

constexpr int DELTA_MAX_TAPS = 16;

// x [n, >= channels] at x_stride: the projections' output, q | k | v channels first (qk_cols = 2 * kv_heads * dk,
// then heads * dv).  Outputs fp32: qk [n, qk_cols], v [n, heads * dv], g [n, heads * dk], beta [n, heads].
// The work of a token is cut into units, one warp each: a q or k head (convolution, SiLU, unit norm: dk channels),
// or a v head (dv channels) together with that head's decays and beta.  grid.y blocks share a token's units, so a
// step of few tokens still fills the SMs.  `single` says that every request brings exactly one token: the thread
// that read a channel's state then also shifts it and appends the token's input (no other token reads that state in
// this step), and conv_state_update is not launched.
template <typename T>
__global__ void __launch_bounds__(256)
delta_prep_kernel(const T* __restrict__ x, int64_t x_stride, const float* __restrict__ conv_w,
                  float* conv_state, const int* __restrict__ positions,
                  const int* __restrict__ token_row, const float* __restrict__ a_raw, int64_t a_stride,
                  const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                  const float* __restrict__ b_raw, int64_t b_stride, float* __restrict__ qk, float* __restrict__ v,
                  float* __restrict__ g, float* __restrict__ beta, int heads, int kv_heads, int dk, int dv, int taps,
                  float unit_eps, float q_scale, int single) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int qk_cols = 2 * kv_heads * dk, channels = qk_cols + heads * dv, units = 2 * kv_heads + heads;
  const int row = token_row[i], pos = positions[i];
  // how many of the request's earlier tokens this batch holds right before row i (at most taps-1 matter)
  int here = 0;
  if (!single)
    while (here < taps - 1 && i - here - 1 >= 0 && token_row[i - here - 1] == row && positions[i - here - 1] == pos - here - 1)
      ++here;
  float* mine = sm + warp * dk;
  float* cs_row = conv_state + (int64_t)row * (taps - 1) * channels;
  for (int u = blockIdx.y * nwarps + warp; u < units; u += gridDim.y * nwarps) {
    const bool is_qk = u < 2 * kv_heads;
    const int h = u - 2 * kv_heads;
    const int c0 = is_qk ? u * dk : qk_cols + h * dv, width = is_qk ? dk : dv;
    float ss = 0.f;
    for (int c = lane; c < width; c += 32) {
      const int ch = c0 + c;
      const float* w = conv_w + (int64_t)ch * taps;
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) {          // j tokens back
        float val;
        if (j <= here) {
          val = to_float(x[(int64_t)(i - j) * x_stride + ch]);
        } else {
          const int idx = taps - 1 - (j - here);   // the state holds the inputs before the batch's first, oldest first
          val = cs_row[(int64_t)idx * channels + ch];
        }
        acc = fmaf(w[taps - 1 - j], val, acc);
      }
      if (single && taps > 1) {
        for (int j = 0; j + 2 < taps; ++j) cs_row[(int64_t)j * channels + ch] = cs_row[(int64_t)(j + 1) * channels + ch];
        cs_row[(int64_t)(taps - 2) * channels + ch] = to_float(x[(int64_t)i * x_stride + ch]);
      }
      const float val = acc / (1.0f + expf(-acc));
      if (is_qk) {
        mine[c] = val;                          // read back below by the lane that wrote it
        ss = fmaf(val, val, ss);
      } else {
        v[(int64_t)i * heads * dv + h * dv + c] = val;
      }
    }
    if (is_qk) {
      ss = warp_sum(ss);
      const float inv = (u < kv_heads ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
      for (int c = lane; c < dk; c += 32) qk[(int64_t)i * qk_cols + c0 + c] = mine[c] * inv;
    } else {
      const float rate = -expf(A_log[h]);
      for (int c = lane; c < dk; c += 32) {
        const int hc = h * dk + c;
        g[(int64_t)i * heads * dk + hc] = expf(rate * softplusf_(a_raw[(int64_t)i * a_stride + hc] + dt_bias[hc]));
      }
      if (lane == 0) beta[(int64_t)i * heads + h] = sigmoidf_(b_raw[(int64_t)i * b_stride + h]);
    }
  }
}

// conv_state [slots, taps-1, channels] <- the last taps-1 of (old state ++ this step's inputs), per request.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* __restrict__ x, int64_t x_stride, float* __restrict__ conv_state,
                         const int* __restrict__ cu_q, const int* __restrict__ state_slots, int channels, int taps) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t0 = cu_q[r], len = cu_q[r + 1] - t0;
  const int keep = taps - 1;
  float* cs = conv_state + (int64_t)state_slots[r] * keep * channels + c;
  for (int j = 0; j < keep; ++j) {           // ascending: what is read lies at or behind what is written
    const int ci = j + len;                  // index into (old state ++ inputs)
    cs[(int64_t)j * channels] = ci < keep ? cs[(int64_t)ci * channels]
                                          : to_float(x[(int64_t)(t0 + ci - keep) * x_stride + c]);
  }
}

constexpr int DELTA_THREADS = 128;
constexpr int DELTA_MAX_CHUNK = 16;

// Asynchronous copies global -> shared: a chunk's operands are on their way while the chunk before it is computed.
__device__ __forceinline__ void copy_async(float* dst, const float* src, int floats) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  if (floats == 4) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Tokens are taken in chunks of `tc`, in two buffers: q [tc][dkp], k [tc][dkp], g [tc][dkp], v [tc][cols], beta [tc]
// (dkp = lanes * DPT >= dk; what lies beyond dk or dv is zeroed once and never copied over).  VEC = 4 copies and
// reads four floats at a time, which needs dk and dv to be multiples of 4 (all row starts are then 16-byte aligned).
// Per token the chain from state to state is: dot products with the decayed key and query (the decay is folded
// into them, off the chain), their sums over the column's lanes, u, one fused multiply-add per state element.
template <int DPT, int LANES, int VEC>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_rule_kernel(const float* __restrict__ qk, const float* __restrict__ v, const float* __restrict__ g,
                  const float* __restrict__ beta, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, float* __restrict__ out, int heads, int kv_heads, int dk,
                  int dv, int tc) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  constexpr int lanes = LANES, cols = DELTA_THREADS / LANES, dkp = LANES * DPT;
  const int r = blockIdx.z, h = blockIdx.y, hg = h / (heads / kv_heads);
  const int cix = threadIdx.x / lanes, sub = threadIdx.x % lanes;
  const int col0 = blockIdx.x * cols, col = col0 + cix;
  const bool live = col < dv;
  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  if (t1 <= t0) return;
  const int buf_floats = (tc * (3 * dkp + cols + 1) + 3) & ~3;
  for (int i = threadIdx.x; i < 2 * buf_floats; i += DELTA_THREADS) sm[i] = 0.f;
  float S[DPT];
  float* sp = state + (((int64_t)state_slots[r] * heads + h) * dv + (live ? col : 0)) * dk + sub * DPT;
  if (VEC == 4) {
#pragma unroll
    for (int e = 0; e < DPT; e += 4) {
      const float4 x = live && sub * DPT + e < dk ? *reinterpret_cast<const float4*>(sp + e) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[e] = x.x, S[e + 1] = x.y, S[e + 2] = x.z, S[e + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < DPT; ++e) S[e] = live && sub * DPT + e < dk ? sp[e] : 0.f;
  }
  const int qk_cols = 2 * kv_heads * dk;
  const int dkv = dk / VEC, colv = cols / VEC;            // cols is a power of two >= 4
  const float* q_src = qk + hg * dk;
  const float* k_src = qk + (kv_heads + hg) * dk;
  const float* g_src = g + (int64_t)h * dk;
  const float* v_src = v + (int64_t)h * dv + col0;
  auto issue = [&](int c0, int nt, float* buf) {
    float* qs = buf;
    float* ks = qs + tc * dkp;
    float* gs = ks + tc * dkp;
    float* vs = gs + tc * dkp;
    float* bs = vs + tc * cols;
    for (int idx = threadIdx.x; idx < nt * dkv; idx += DELTA_THREADS) {
      const int t = idx / dkv, d = (idx - t * dkv) * VEC;
      const int64_t tok = c0 + t;
      copy_async(qs + t * dkp + d, q_src + tok * qk_cols + d, VEC);
      copy_async(ks + t * dkp + d, k_src + tok * qk_cols + d, VEC);
      copy_async(gs + t * dkp + d, g_src + tok * heads * dk + d, VEC);
    }
    for (int idx = threadIdx.x; idx < nt * colv; idx += DELTA_THREADS) {
      const int t = idx / colv, c = (idx - t * colv) * VEC;
      if (col0 + c < dv) copy_async(vs + t * cols + c, v_src + (int64_t)(c0 + t) * heads * dv + c, VEC);
    }
    for (int t = threadIdx.x; t < nt; t += DELTA_THREADS) copy_async(bs + t, beta + (int64_t)(c0 + t) * heads + h, 1);
    copy_async_commit();
  };
  __syncthreads();                                         // the zeros are there before the first copy lands
  issue(t0, min(tc, t1 - t0), sm);
  int which = 0;
  for (int c0 = t0; c0 < t1; c0 += tc, which ^= 1) {
    const int nt = min(tc, t1 - c0);
    if (c0 + tc < t1) {
      issue(c0 + tc, min(tc, t1 - c0 - tc), sm + (which ^ 1) * buf_floats);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const float* buf = sm + which * buf_floats;
    const float* qs = buf + sub * DPT;
    const float* ks = qs + tc * dkp;
    const float* gs = ks + tc * dkp;
    const float* vs = buf + 3 * tc * dkp + cix;
    const float* bs = buf + 3 * tc * dkp + tc * cols;
    float* op = out + ((int64_t)c0 * heads + h) * dv + col;
    // What a token brings (k, g, q, k.q summed over the lanes, v, beta) does not depend on the state and is fetched
    // one token ahead, so that the chain from state to state is the decay, two dot products (in ACC partial sums
    // each), their sums over the lanes, u and one fused multiply-add per element.
    constexpr int ACC = DPT >= 16 ? 4 : (DPT >= 8 ? 2 : 1);
    auto fetch = [&](int t, float (&k_)[DPT], float (&g_)[DPT], float (&q_)[DPT], float& kq_, float& v_, float& b_) {
      if (VEC == 4) {
#pragma unroll
        for (int e = 0; e < DPT; e += 4) {
          const float4 a = *reinterpret_cast<const float4*>(ks + t * dkp + e);
          const float4 b = *reinterpret_cast<const float4*>(gs + t * dkp + e);
          const float4 c = *reinterpret_cast<const float4*>(qs + t * dkp + e);
          k_[e] = a.x, k_[e + 1] = a.y, k_[e + 2] = a.z, k_[e + 3] = a.w;
          g_[e] = b.x, g_[e + 1] = b.y, g_[e + 2] = b.z, g_[e + 3] = b.w;
          q_[e] = c.x, q_[e + 1] = c.y, q_[e + 2] = c.z, q_[e + 3] = c.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < DPT; ++e) k_[e] = ks[t * dkp + e], g_[e] = gs[t * dkp + e], q_[e] = qs[t * dkp + e];
      }
      v_ = vs[t * cols];
      b_ = bs[t];
      float part[ACC] = {};
#pragma unroll
      for (int e = 0; e < DPT; ++e) part[e % ACC] = fmaf(k_[e], q_[e], part[e % ACC]);
#pragma unroll
      for (int w = ACC >> 1; w > 0; w >>= 1)
#pragma unroll
        for (int x = 0; x < w; ++x) part[x] += part[x + w];
      kq_ = part[0];
#pragma unroll
      for (int o = LANES >> 1; o > 0; o >>= 1) kq_ += __shfl_xor_sync(0xffffffffu, kq_, o);
    };
    float kk[DPT], gg[DPT], qq[DPT], kq, vv, bb;
    fetch(0, kk, gg, qq, kq, vv, bb);
#pragma unroll 2
    for (int t = 0; t < nt; ++t) {
      float nk[DPT], ng[DPT], nq[DPT], nkq, nv, nb;
      fetch(min(t + 1, nt - 1), nk, ng, nq, nkq, nv, nb);
      float pk[ACC] = {}, pq[ACC] = {};
#pragma unroll
      for (int e = 0; e < DPT; ++e) {
        S[e] *= gg[e];
        pk[e % ACC] = fmaf(S[e], kk[e], pk[e % ACC]);
        pq[e % ACC] = fmaf(S[e], qq[e], pq[e % ACC]);
      }
#pragma unroll
      for (int w = ACC >> 1; w > 0; w >>= 1)
#pragma unroll
        for (int x = 0; x < w; ++x) pk[x] += pk[x + w], pq[x] += pq[x + w];
      float sk = pk[0], sq = pq[0];
#pragma unroll
      for (int o = LANES >> 1; o > 0; o >>= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
      }
      const float u = bb * (vv - sk);
#pragma unroll
      for (int e = 0; e < DPT; ++e) S[e] = fmaf(kk[e], u, S[e]);
      if (sub == 0 && live) op[(int64_t)t * heads * dv] = fmaf(u, kq, sq);
#pragma unroll
      for (int e = 0; e < DPT; ++e) kk[e] = nk[e], gg[e] = ng[e], qq[e] = nq[e];
      kq = nkq, vv = nv, bb = nb;
    }
    __syncthreads();                                       // the next copies go into the buffer just read
  }
  if (live) {
    if (VEC == 4) {
#pragma unroll
      for (int e = 0; e < DPT; e += 4)
        if (sub * DPT + e < dk) *reinterpret_cast<float4*>(sp + e) = make_float4(S[e], S[e + 1], S[e + 2], S[e + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < DPT; ++e)
        if (sub * DPT + e < dk) sp[e] = S[e];
    }
  }
}

inline int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

template <typename T>
int delta_prep_launch(const T* x, int64_t x_stride, const float* conv_w, float* conv_state, const int* positions,
                      const int* token_row, const int* cu_q, const int* state_slots, int num_requests,
                      const float* a_raw, int64_t a_stride, const float* dt_bias, const float* A_log, const float* b_raw,
                      int64_t b_stride, float* qk, float* v, float* g, float* beta, int n_tokens, int heads, int kv_heads,
                      int dk, int dv, int taps, float unit_eps, float q_scale, int max_q_len, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int channels = 2 * kv_heads * dk + heads * dv, units = 2 * kv_heads + heads, nwarps = 8;
  const size_t smem = sizeof(float) * (size_t)nwarps * dk;
  if (taps < 1 || taps > DELTA_MAX_TAPS || heads % kv_heads || smem > 48 * 1024 || num_requests > 65535)
    return (int)cudaErrorInvalidValue;
  // a token's units spread over as many blocks as it takes to give every SM a few, at most one unit a warp
  int parts = (4 * 148 + n_tokens - 1) / n_tokens;
  parts = std::max(1, std::min(parts, (units + nwarps - 1) / nwarps));
  const int single = max_q_len == 1 && n_tokens == num_requests;
  int rc = gllm_launch(delta_prep_kernel<T>, dim3(n_tokens, parts), dim3(32 * nwarps), smem, stream, x, x_stride, conv_w,
                       conv_state, positions, token_row, a_raw, a_stride, dt_bias, A_log, b_raw, b_stride,
                       qk, v, g, beta, heads, kv_heads, dk, dv, taps, unit_eps, q_scale, single);
  if (rc != 0 || taps == 1 || num_requests <= 0 || single) return rc;
  return gllm_launch(conv_state_update_kernel<T>, dim3((channels + 255) / 256, num_requests), dim3(256), 0, stream, x,
                     x_stride, conv_state, cu_q, state_slots, channels, taps);
}

int delta_rule_launch(const float* qk, const float* v, const float* g, const float* beta, float* state,
                      const int* cu_q, const int* state_slots, float* out, int num_requests, int heads, int kv_heads,
                      int dk, int dv, int max_q_len, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (heads > 65535 || num_requests > 65535 || dk < 1 || dv < 1 || dk > 512 || heads % kv_heads)
    return (int)cudaErrorInvalidValue;
  // Key channels a thread keeps (DPT).  More of them mean fewer threads a column, so fewer rounds of shuffles and more
  // independent work per warp, but fewer warps in all.  Measured: four for heads of up to 64 key channels and eight
  // beyond when one prompt runs alone (every warp the step can have is wanted); eight when every request brings one
  // token (the step is then bound by reading and writing the states); thirty-two for several prompts at once, as soon
  // as that still gives every SM its blocks.
  // copies and loads of four floats at a time want every row start on a 16-byte boundary
  const bool vec = dk % 4 == 0 && dv % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(qk) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(g) |
                     reinterpret_cast<uintptr_t>(state)) & 15) == 0;
  int dpt = dk <= 128 ? 4 : (dk <= 256 ? 8 : 16);
  if (vec) {
    dpt = dk <= 64 ? 4 : (dk <= 256 ? 8 : 16);
    if (dk <= 64 && max_q_len == 1) dpt = std::min(8, std::max(4, dk));
    if (dk > 32 && dk <= 64 && max_q_len != 1 && (int64_t)((dv + 63) / 64) * heads * num_requests >= 240) dpt = 32;
  }
  if (const char* e = getenv("GLLM_B200_DELTA_DPT")) {
    const int want = atoi(e);
    if ((want == 4 || want == 8 || want == 16 || want == 32) && want * 32 >= dk && vec) dpt = want;
  }
  const int lanes = pow2_at_least((dk + dpt - 1) / dpt);
  const int cols = DELTA_THREADS / lanes, dkp = lanes * dpt;
  int tc = DELTA_MAX_CHUNK;
  while (tc > 2 && 2 * tc * (3 * dkp + cols + 1) * sizeof(float) > 96 * 1024) tc >>= 1;
  const size_t smem = sizeof(float) * 2 * (size_t)((tc * (3 * dkp + cols + 1) + 3) & ~3);
  using Kernel = void (*)(const float*, const float*, const float*, const float*, float*, const int*, const int*, float*,
                          int, int, int, int, int);
  Kernel kernel = nullptr;
#define GLLM_DELTA_PICK(D, L) \
  if (dpt == D && lanes == L) kernel = vec ? delta_rule_kernel<D, L, 4> : delta_rule_kernel<D, L, 1>;
#define GLLM_DELTA_PICK4(D, L) \
  if (dpt == D && lanes == L && vec) kernel = delta_rule_kernel<D, L, 4>;
  GLLM_DELTA_PICK(4, 1) GLLM_DELTA_PICK(4, 2) GLLM_DELTA_PICK(4, 4) GLLM_DELTA_PICK(4, 8) GLLM_DELTA_PICK(4, 16)
  GLLM_DELTA_PICK(4, 32) GLLM_DELTA_PICK(8, 32) GLLM_DELTA_PICK(16, 32)
  GLLM_DELTA_PICK4(8, 1) GLLM_DELTA_PICK4(8, 2) GLLM_DELTA_PICK4(8, 4) GLLM_DELTA_PICK4(8, 8) GLLM_DELTA_PICK4(8, 16)
  GLLM_DELTA_PICK4(16, 1) GLLM_DELTA_PICK4(16, 2) GLLM_DELTA_PICK4(16, 4) GLLM_DELTA_PICK4(16, 8) GLLM_DELTA_PICK4(16, 16)
  GLLM_DELTA_PICK4(32, 1) GLLM_DELTA_PICK4(32, 2) GLLM_DELTA_PICK4(32, 4) GLLM_DELTA_PICK4(32, 8) GLLM_DELTA_PICK4(32, 16)
#undef GLLM_DELTA_PICK4
#undef GLLM_DELTA_PICK
  if (kernel == nullptr) return (int)cudaErrorInvalidValue;
  // The kernel is bound by the latency of each warp's chain, so its blocks should lie evenly over the SMs.  A block
  // that starts while the kernel before it drains lands wherever a place frees first; asking for a share of an SM's
  // shared memory that lets no SM take more than its even share of the blocks keeps them spread.
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
      sm_count = 148;
  }
  const int64_t blocks = (int64_t)((dv + cols - 1) / cols) * heads * num_requests;
  const int64_t per_sm = (blocks + sm_count - 1) / sm_count;
  const size_t share = (size_t)(228 * 1024 / per_sm) - 1024;     // 1 KB of every block's share is the system's
  const size_t smem_ask = std::max(smem, std::min(share, (size_t)227 * 1024));
  if (smem_ask > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
  }
  return gllm_launch(kernel, dim3((dv + cols - 1) / cols, heads, num_requests), dim3(DELTA_THREADS), smem_ask, stream, qk, v,
                     g, beta, state, cu_q, state_slots, out, heads, kv_heads, dk, dv, tc);
}
}  // namespace

#define GLLM_DELTA_EXPORTS(T, S)                                                                                       \
  GLLM_API int gllm_delta_prep_##S(const T* x, int64_t x_stride, const float* conv_w, float* conv_state,               \
                                   const int* positions, const int* token_row, const int* cu_q,                        \
                                   const int* state_slots, int num_requests, const float* a_raw, int64_t a_stride,     \
                                   const float* dt_bias, const float* A_log, const float* b_raw, int64_t b_stride,     \
                                   float* qk, float* v, float* g, float* beta, int n_tokens, int heads, int kv_heads,  \
                                   int dk, int dv, int taps, float unit_eps, float q_scale, int max_q_len,             \
                                   cudaStream_t stream) {                                                              \
    return delta_prep_launch<T>(x, x_stride, conv_w, conv_state, positions, token_row, cu_q, state_slots,              \
                                num_requests, a_raw, a_stride, dt_bias, A_log, b_raw, b_stride, qk, v, g, beta,        \
                                n_tokens, heads, kv_heads, dk, dv, taps, unit_eps, q_scale, max_q_len, stream);        \
  }
GLLM_DELTA_EXPORTS(float, f32)
GLLM_DELTA_EXPORTS(__nv_bfloat16, bf16)

GLLM_API int gllm_delta_rule(const float* qk, const float* v, const float* g, const float* beta, float* state,
                             const int* cu_q, const int* state_slots, float* out, int num_requests, int heads,
                             int kv_heads, int dk, int dv, int max_q_len, cudaStream_t stream) {
  return delta_rule_launch(qk, v, g, beta, state, cu_q, state_slots, out, num_requests, heads, kv_heads, dk, dv, max_q_len,
                           stream);
}
