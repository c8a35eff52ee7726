// Kernels of the mixers that carry a state of fixed size from token to token instead of (or beside)
// cached keys and values: a short causal convolution per channel, the selective state-space scan
// (S <- exp(dt A) S + dt x B, y = S C + D x), and a matrix recurrence per head
// (S <- diag(a) S + b v^T, o = S^T q) that serves both gated linear attention (a = f, b = 1 - f) and a
// matrix memory with exponential gates held stable by a running maximum (a = scalar keep, b = take * k).
//
// The flat batch holds prompt portions of any length beside single tokens.  Request r owns the rows
// cu_q[r] .. cu_q[r+1]-1; its state lives in row state_slots[r] of each state tensor, is read at the
// start of the step and written back at its end, so a prompt may be cut anywhere.  States, decays,
// gates, step sizes and every sum over a state are fp32 whatever the activations' type; the order of
// the sums depends on nothing but the sizes of the model.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// Loads that stay where they are written: the look-ahead of the chunked kernels below asks for the next chunk's
// inputs before it computes the current one, and the compiler would otherwise move the loads down to their first
// use, behind the computation they are meant to overlap.
// They return the loaded bits untouched (a bfloat16 zero-extended by the load itself): any instruction on the value,
// even the shift that makes a float of a bfloat16, would wait for the load right there.  as_value() is for later.
__device__ __forceinline__ uint32_t load_ahead(const float* p) {
  uint32_t v;
  asm volatile("ld.global.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t load_ahead(const __nv_bfloat16* p) {
  uint32_t v;
  asm volatile("ld.global.u16 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
template <typename T> __device__ __forceinline__ float as_value(uint32_t bits);
template <> __device__ __forceinline__ float as_value<float>(uint32_t bits) { return __uint_as_float(bits); }
template <> __device__ __forceinline__ float as_value<__nv_bfloat16>(uint32_t bits) { return __uint_as_float(bits << 16); }

// --------------------------------------------------------------- causal convolution + SiLU
// out[i, c] = silu(bias[c] + sum_j w[c, taps-1-j] * x[i-j, c]) over the request's own earlier tokens;
// what lies before this step's first token comes from conv_state[slot, taps-1, channels] (the last
// taps-1 inputs of the request, oldest first; zero for a new request).  The state itself is brought
// up to date by the scan kernel that follows.
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* __restrict__ x, int64_t x_stride, const float* __restrict__ w, const float* __restrict__ bias,
                 const float* __restrict__ conv_state, const int* __restrict__ positions,
                 const int* __restrict__ token_row, T* __restrict__ out, int n_tokens, int channels, int taps) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int i = blockIdx.x;
  if (c >= channels) return;
  const int row = token_row[i], pos = positions[i];
  float acc = bias ? bias[c] : 0.f;
  int j0 = -1;   // first distance at which the batch no longer holds the request's token
  for (int j = 0; j < taps; ++j) {
    float v = 0.f;
    if (j0 < 0) {
      const int k = i - j;
      const bool here = k >= 0 && token_row[k] == row && positions[k] == pos - j;
      if (here) {
        v = to_float(x[(int64_t)k * x_stride + c]);
      } else {
        j0 = j;
      }
    }
    if (j0 >= 0) {
      const int idx = taps - 2 - (j - j0);
      v = conv_state[((int64_t)row * (taps - 1) + idx) * channels + c];
    }
    acc = fmaf(w[(int64_t)c * taps + (taps - 1 - j)], v, acc);
  }
  out[(int64_t)i * channels + c] = from_float<T>(siluf_(acc));
}

// --------------------------------------------------------------- selective scan
// One group of `lanes` threads per (request, channel); each thread keeps NPT of the channel's states (2 for up
// to 64 states, so that a token costs a warp few instructions: the scan is a chain from token to token and what
// bounds it is the length of that chain, not the amount of work; 8 beyond).
// The tokens of a request are taken in chunks of `tc`: while one chunk is computed from shared memory,
// the inputs of the next (step size, input and gate of every channel of the block, B and C rows) are
// already on their way from global memory into registers, and go into the other buffer afterwards.
// Blocks are large (512 threads) when there are channels enough: the warps of a block hide one another's
// latencies, and a block's B and C rows are staged once for all its channels.
constexpr int SCAN_MAX_CHUNK = 16;
constexpr int SCAN_PF_BC = 8;      // B/C values a thread fetches ahead per chunk: tc * 2 * n_state <= threads * 8
constexpr int SCAN_PF_CH = 8;      // (token, channel) cells a thread fetches ahead: tc * channels per block <= threads * 8

template <typename T, int NPT, int THREADS>
__global__ void __launch_bounds__(THREADS)
selective_scan_kernel(const T* __restrict__ xc,            // [n, channels]  convolved, activated input
                      const float* __restrict__ dt_raw,    // [n, channels]  step-size projection, before bias
                      const float* __restrict__ dt_bias,   // [channels]
                      const float* __restrict__ A,         // [channels, n_state]  (negative)
                      const T* __restrict__ bc, int64_t bc_stride, int b_off, int c_off,   // B, C rows
                      const float* __restrict__ D,         // [channels]
                      const T* __restrict__ xz, int64_t xz_stride, int z_off,              // raw input and gate
                      float* __restrict__ ssm_state,       // [slots, channels, n_state]
                      float* __restrict__ conv_state,      // [slots, taps-1, channels]
                      const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                      T* __restrict__ out,                 // [n, channels]  y * silu(z)
                      int channels, int n_state, int taps, int lanes, int tc) {
  extern __shared__ float scan_smem[];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int per_block = THREADS / lanes;
  const int c0 = blockIdx.x * per_block;
  const int cl = threadIdx.x / lanes;            // channel within the block
  const int c = c0 + cl;
  const int sub = threadIdx.x % lanes;
  const int start = cu_q[r], end = cu_q[r + 1];
  const int slot = state_slots[r];
  const bool live = c < channels;
  const int cc = live ? c : 0;
  // one buffer: B|C [tc][2 * n_state], then dt, x, silu(z) [tc][per_block] each
  const int buf_floats = tc * (2 * n_state + 3 * per_block);
  float S[NPT], a[NPT];
  float* sp = ssm_state + ((int64_t)slot * channels + cc) * n_state;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int n = sub * NPT + k;
    const bool ok = live && n < n_state;
    S[k] = ok ? sp[n] : 0.f;
    a[k] = ok ? A[(int64_t)cc * n_state + n] * 1.4426950408889634f : 0.f;    // exp(dt A) = 2^(dt A log2 e)
  }
  const float dskip = D[cc];

  uint32_t pf_bc[SCAN_PF_BC], pf_dt[SCAN_PF_CH], pf_x[SCAN_PF_CH], pf_z[SCAN_PF_CH];
  const int ch_mine = c0 + (threadIdx.x & (per_block - 1)), tt_c0 = threadIdx.x / per_block;   // per_block * lanes = THREADS
  const float bias_mine = ch_mine < channels ? dt_bias[ch_mine] : 0.f;
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int j = 0; j < SCAN_PF_BC; ++j) {
      const int idx = threadIdx.x + j * THREADS;
      if (idx >= nt * 2 * n_state) break;
      const int tt = idx / (2 * n_state), n = idx - tt * 2 * n_state;
      const T* row = bc + (int64_t)(t0 + tt) * bc_stride;
      pf_bc[j] = load_ahead(n < n_state ? row + b_off + n : row + c_off + n - n_state);
    }
    // a thread keeps one channel of the block and walks the chunk's tokens in steps of `lanes`
#pragma unroll
    for (int j = 0; j < SCAN_PF_CH; ++j) {
      const int tt = tt_c0 + j * lanes;
      if (tt >= nt) break;
      pf_dt[j] = pf_x[j] = pf_z[j] = 0u;
      if (ch_mine < channels) {
        const int64_t t = t0 + tt;
        pf_dt[j] = load_ahead(dt_raw + t * channels + ch_mine);
        pf_x[j] = load_ahead(xc + t * channels + ch_mine);
        pf_z[j] = load_ahead(xz + t * xz_stride + z_off + ch_mine);
      }
    }
  };
  auto stash = [&](int nt, float* buf) {
    float* bc_s = buf;
    float* dt_s = buf + tc * 2 * n_state;
    float* x_s = dt_s + tc * per_block;
    float* z_s = x_s + tc * per_block;
#pragma unroll
    for (int j = 0; j < SCAN_PF_BC; ++j) {
      const int idx = threadIdx.x + j * THREADS;
      if (idx >= nt * 2 * n_state) break;
      bc_s[idx] = as_value<T>(pf_bc[j]);
    }
#pragma unroll
    for (int j = 0; j < SCAN_PF_CH; ++j) {
      const int tt = tt_c0 + j * lanes;
      if (tt >= nt) break;
      const int idx = tt * per_block + (threadIdx.x & (per_block - 1));
      dt_s[idx] = softplusf_(as_value<float>(pf_dt[j]) + bias_mine);
      x_s[idx] = as_value<T>(pf_x[j]);
      z_s[idx] = siluf_(as_value<T>(pf_z[j]));
    }
  };

  if (start < end) {
    fetch(start, min(tc, end - start));
    stash(min(tc, end - start), scan_smem);
  }
  __syncthreads();
  int which = 0;
  for (int t0 = start; t0 < end; t0 += tc, which ^= 1) {
    const int nt = min(tc, end - t0);
    const int next = t0 + tc;
    const int nt_next = min(tc, end - next);
    if (next < end) fetch(next, nt_next);
    const float* buf = scan_smem + which * buf_floats;
    const float* bc_s = buf;
    const float* dt_s = buf + tc * 2 * n_state;
    const float* x_s = dt_s + tc * per_block;
    const float* z_s = x_s + tc * per_block;
    T* out_p = out + (int64_t)t0 * channels + cc;
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = dt_s[tt * per_block + cl];
      const float x = x_s[tt * per_block + cl];
      const float dx = dt * x;
      const float* brow = bc_s + tt * 2 * n_state;
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < NPT; ++k) {
        const int n = sub * NPT + k;
        if (n < n_state) {
          S[k] = exp2f(dt * a[k]) * S[k] + dx * brow[n];
          y = fmaf(S[k], brow[n_state + n], y);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        if (o < lanes) y += __shfl_xor_sync(0xffffffffu, y, o);          // (lanes is the same for the whole grid)
      if (sub == 0 && live) *out_p = from_float<T>((y + dskip * x) * z_s[tt * per_block + cl]);
      out_p += channels;
    }
    if (next < end) stash(nt_next, scan_smem + (which ^ 1) * buf_floats);
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
      const int n = sub * NPT + k;
      if (n < n_state) sp[n] = S[k];
    }
  }
  // the convolution's memory: the request's last taps-1 raw inputs, oldest first
  if (live && sub == 0 && taps > 1) {
    const int keep = taps - 1, q_len = end - start;
    float* cs = conv_state + (int64_t)slot * keep * channels + cc;
    float fresh[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {
      if (k < keep) {
        const int from_batch = q_len - keep + k;     // index among this step's tokens
        fresh[k] = from_batch >= 0 ? to_float(xz[(int64_t)(start + from_batch) * xz_stride + cc])
                                   : cs[(int64_t)(k + q_len) * channels];
      }
    }
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
      if (k < keep) cs[(int64_t)k * channels] = fresh[k];
  }
}

// --------------------------------------------------------------- the scalar gates of the exponential-gate memory
// Per (request, head): i = cap * tanh((i_raw + i_bias) / cap), f = logsigmoid(cap * tanh((f_raw + f_bias) / cap)) for
// every token of the step (in parallel), then the running maximum m' = max(f + m, i) token after token (one thread
// per head: two operations a token).  work [n, 4 * heads] = i | f | m before the token | m after it; the
// request's maximum in mstate is brought up to date here and nowhere else, so the blocks of the recurrence
// kernel, which may run at different times, all see the same values.
__global__ void __launch_bounds__(128)
exp_gate_scan_kernel(const float* __restrict__ gates, int64_t gates_stride, const float* __restrict__ gate_bias, float cap,
                     float* __restrict__ mstate, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                     float* __restrict__ work, int heads) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int start = cu_q[r], end = cu_q[r + 1];
  const int slot = state_slots[r];
  const int64_t total = (int64_t)(end - start) * heads;
  for (int64_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int64_t t = start + idx / heads;
    const int h = (int)(idx % heads);
    const float* g = gates + t * gates_stride;
    work[t * 4 * heads + h] = cap * tanhf((g[h] + gate_bias[h]) / cap);
    work[t * 4 * heads + heads + h] = logsigmoidf_(cap * tanhf((g[heads + h] + gate_bias[heads + h]) / cap));
  }
  __syncthreads();
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    float m = mstate[(int64_t)slot * heads + h];
    for (int64_t t0 = start; t0 < end; t0 += 8) {      // eight tokens' gates are asked for at once, then chained
      float ig[8], fg[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool ok = t0 + u < end;
        const float* w = work + (t0 + (ok ? u : 0)) * 4 * heads;
        ig[u] = __ldcg(w + h);
        fg[u] = __ldcg(w + heads + h);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (t0 + u < end) {
          float* w = work + (t0 + u) * 4 * heads;
          w[2 * heads + h] = m;
          m = fmaxf(fg[u] + m, ig[u]);
          w[3 * heads + h] = m;
        }
      }
    }
    mstate[(int64_t)slot * heads + h] = m;
  }
}

// --------------------------------------------------------------- matrix recurrence per head
// S [dvx, dk] per (request, head), stored column by column: S[c, d] is what key channel d holds of value
// column c.  mode 0 (gated linear attention): a[d] = f[d], b[d] = 1 - f[d] with
// f = lower + (1 - lower) * sigmoid(f_raw + f_bias) and q = silu(q_raw).  mode 1 (matrix memory with
// exponential gates): i = cap * tanh((i_raw + i_bias) / cap), f = logsigmoid(cap * tanh((f_raw + f_bias) / cap)),
// m' = max(f + m, i), a = exp(f + m - m'), b[d] = exp(i - m') * k[d], q = q_raw * q_scale; the state
// has one column more than there are value columns, fed with ones, which carries the normaliser n, and
// the output gets two columns more: n . q and exp(-m').  mode 2 (state-space duality): one step size per (token, head),
// dt = softplus(dt_raw + dt_bias[h]); a = exp(A[h] * dt) for the whole head (A = -exp(A_log) arrives in `lower`;
// the update is written S += b v - (1 - a) S with 1 - a from expm1),
// b[d] = dt * k[d] (k: the input projection B), q: the read-out projection C; heads share B and C in groups of
// `kv_div` neighbouring heads.
// A block owns `cols` columns of one (request, head); `lanes` threads share a column, each keeping DPT of its
// key channels (4 for up to 128 key channels, 16 beyond; 8 for 65..128 measured the same: the recurrence is a chain from token to token, bounded
// by the instructions a warp spends per token, so the state is spread over many threads).  Tokens are taken in chunks of `tc`: while a chunk is computed from shared memory, the raw
// inputs of the next one are on their way into registers; they are turned into the effective q, gate (or
// key) and v and put into the other buffer afterwards.
#ifndef REC_TOKEN_UNROLL
#define REC_TOKEN_UNROLL 2            // tokens of a chunk whose instructions the compiler may interleave
#endif
constexpr int REC_UNROLL_TOKENS = REC_TOKEN_UNROLL;
constexpr int REC_THREADS = 256;
constexpr int REC_MAX_CHUNK = 16;
constexpr int REC_LOOKAHEAD = 2048; // values of one operand that a block fetches ahead per chunk (8 per thread)
// (Blocks of 1,024 threads, which would activate a chunk's q and gate once for 64 columns instead of once per 16,
// measured the same or slower: 8 warps per scheduler then wait for issue slots instead of for one another.)

template <typename T, int DPT, int THREADS, int MODE>
__global__ void __launch_bounds__(THREADS)
matrix_recurrence_kernel(int,
                         const T* __restrict__ q, int64_t q_stride,       // [n, heads * dk] at its offset
                         const T* __restrict__ k, int64_t k_stride,       // mode 1
                         const T* __restrict__ v, int64_t v_stride,       // [n, heads * dv]
                         const float* __restrict__ gates, int64_t gates_stride,
                         // mode 0: f_raw [n, heads * dk]; mode 1: the gate scan's work [n, 4 * heads]
                         const float* __restrict__ gate_bias,             // mode 0: [heads * dk]
                         const float* __restrict__ lower,                 // mode 0: [heads * dk]
                         float q_scale,
                         float* __restrict__ state,                       // [slots, heads, dvx, dk]
                         const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                         float* __restrict__ out, int64_t out_stride,     // [n, heads * out_cols]
                         int heads, int dk, int dv, int lanes, int tc, int kv_div) {
  constexpr int PF = REC_LOOKAHEAD / THREADS;
  constexpr int mode = MODE;
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int cols = THREADS / lanes;
  const int dkp = lanes * DPT;                 // padded row of the staged operands
  const int dvx = dv + (mode == 1 ? 1 : 0);
  const int out_cols = dv + (mode == 1 ? 2 : 0);
  const int r = blockIdx.z, h = blockIdx.y;
  const int cix = threadIdx.x / lanes;
  const int col = blockIdx.x * cols + cix;
  const int sub = threadIdx.x % lanes;
  const int start = cu_q[r], end = cu_q[r + 1];
  const int slot = state_slots[r];
  const bool live = col < dvx;
  // one buffer: q [tc][dkp], gate or key [tc][dkp], v [tc][cols], keep | take | exp(-m') [3][tc] (padded to 4)
  const int buf_floats = tc * (2 * dkp + cols + 4);
  float* const bufs = smem;

  float S[DPT];
  float* sp = state + (((int64_t)slot * heads + h) * dvx + (live ? col : 0)) * dk;
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = ((i >> 2) * lanes + sub) * 4 + (i & 3);
    S[i] = (live && d < dk) ? sp[d] : 0.f;
  }

  uint32_t pq[PF], pg[PF], pv[PF], pi = 0u, pf = 0u, pmp = 0u, pmn = 0u;
  // Which cells of a chunk a thread fetches does not change from chunk to chunk.  With dkp <= THREADS (both powers
  // of two) a thread keeps one key channel and walks the tokens in steps of THREADS / dkp: no division per cell,
  // and a thread stops at the chunk's end instead of running through its dead look-ahead slots.
  const bool fast = dkp <= THREADS;
  const int d_mine = threadIdx.x & (dkp - 1), tt_q0 = threadIdx.x / dkp, tt_qstep = fast ? THREADS / dkp : 0;
  const int c_mine = threadIdx.x & (cols - 1), tt_v0 = threadIdx.x / cols, tt_vstep = lanes;   // THREADS / cols
  const int hd_mine = h * dk + min(d_mine, dk - 1);
  const int kd_mine = (h / kv_div) * dk + min(d_mine, dk - 1);      // q and k: shared by kv_div heads
  const int cg_mine = blockIdx.x * cols + c_mine;
  const float lo_mine = (mode == 0 && fast && d_mine < dk) ? lower[hd_mine] : 0.f;
  const float gb_mine = (mode == 0 && fast && d_mine < dk) ? gate_bias[hd_mine] : 0.f;
  auto fetch = [&](int t0, int nt) {
    if (fast) {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int tt = tt_q0 + j * tt_qstep;
        if (tt >= nt) break;
        pq[j] = pg[j] = 0u;
        if (d_mine < dk) {
          const int64_t t = t0 + tt;
          pq[j] = load_ahead(q + t * q_stride + kd_mine);
          pg[j] = mode >= 1 ? load_ahead(k + t * k_stride + kd_mine) : load_ahead(gates + t * gates_stride + hd_mine);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int idx = threadIdx.x + j * THREADS;
        if (idx >= nt * dkp) break;
        const int tt = idx / dkp, d = idx - tt * dkp;
        pq[j] = pg[j] = 0u;
        if (d < dk) {
          const int64_t t = t0 + tt;
          const int hd = h * dk + d, kd = (h / kv_div) * dk + d;
          pq[j] = load_ahead(q + t * q_stride + kd);
          pg[j] = mode >= 1 ? load_ahead(k + t * k_stride + kd) : load_ahead(gates + t * gates_stride + hd);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      const int tt = tt_v0 + j * tt_vstep;
      if (tt >= nt) break;
      pv[j] = cg_mine < dv ? load_ahead(v + (int64_t)(t0 + tt) * v_stride + (int64_t)h * dv + cg_mine) : 0u;
    }
    if (mode == 1 && (int)threadIdx.x < nt) {
      const float* g = gates + (int64_t)(t0 + threadIdx.x) * gates_stride;
      pi = load_ahead(g + h);
      pf = load_ahead(g + heads + h);
      pmp = load_ahead(g + 2 * heads + h);
      pmn = load_ahead(g + 3 * heads + h);
    }
    if (mode == 2 && (int)threadIdx.x < nt) pi = load_ahead(gates + (int64_t)(t0 + threadIdx.x) * gates_stride + h);
  };
  auto stash = [&](int nt, float* buf) {
    float* q_s = buf;
    float* g_s = buf + tc * dkp;
    float* v_s = g_s + tc * dkp;
    float* sc_s = v_s + tc * cols;
    if (fast) {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int tt = tt_q0 + j * tt_qstep;
        if (tt >= nt) break;
        const int idx = tt * dkp + d_mine;
        if (mode >= 1) {
          q_s[idx] = as_value<T>(pq[j]) * q_scale;
          g_s[idx] = as_value<T>(pg[j]);
        } else {
          q_s[idx] = d_mine < dk ? siluf_(as_value<T>(pq[j])) : 0.f;
          g_s[idx] = d_mine < dk ? lo_mine + (1.0f - lo_mine) * sigmoidf_(as_value<float>(pg[j]) + gb_mine) : 0.f;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int idx = threadIdx.x + j * THREADS;
        if (idx >= nt * dkp) break;
        const int d = idx % dkp;
        if (mode >= 1) {
          q_s[idx] = as_value<T>(pq[j]) * q_scale;
          g_s[idx] = as_value<T>(pg[j]);
        } else {
          const float lo = d < dk ? lower[h * dk + d] : 0.f;
          const float bias = d < dk ? gate_bias[h * dk + d] : 0.f;
          q_s[idx] = d < dk ? siluf_(as_value<T>(pq[j])) : 0.f;
          g_s[idx] = d < dk ? lo + (1.0f - lo) * sigmoidf_(as_value<float>(pg[j]) + bias) : 0.f;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      const int tt = tt_v0 + j * tt_vstep;
      if (tt >= nt) break;
      v_s[tt * cols + c_mine] = cg_mine < dv ? as_value<T>(pv[j]) : 1.0f;
    }
    if (mode == 1 && (int)threadIdx.x < nt) {
      const float m_new = as_value<float>(pmn);
      sc_s[threadIdx.x] = expf(as_value<float>(pf) + as_value<float>(pmp) - m_new);          // keep
      sc_s[tc + threadIdx.x] = expf(as_value<float>(pi) - m_new);                            // take
      sc_s[2 * tc + threadIdx.x] = expf(-m_new);
    }
    if (mode == 2 && (int)threadIdx.x < nt) {
      const float dt = softplusf_(as_value<float>(pi) + gate_bias[h]);
      // what the state LOSES, 1 - exp(A dt), straight from expm1: a decay next to one rounds to a float 1e-7 off,
      // and that error, made anew at every token, would add up over the hundreds of tokens such a state remembers
      sc_s[threadIdx.x] = -expm1f(lower[h] * dt);                                            // 1 - keep
      sc_s[tc + threadIdx.x] = dt;                                                           // take
    }
  };

  if (start < end) {
    fetch(start, min(tc, end - start));
    stash(min(tc, end - start), bufs);
  }
  __syncthreads();
  int which = 0;
  for (int t0 = start; t0 < end; t0 += tc, which ^= 1) {
    const int nt = min(tc, end - t0);
    const int next = t0 + tc;
    const int nt_next = min(tc, end - next);
    if (next < end) fetch(next, nt_next);
    const float* buf = bufs + which * buf_floats;
    // a thread's key channels come in fours, `lanes` fours apart: the threads of a column then read neighbouring
    // 16 bytes of the staged operands (one four-float load each, no two on one bank)
    const float* q_s = buf + sub * 4;
    const float* g_s = buf + tc * dkp + sub * 4;
    const float* v_s = buf + 2 * tc * dkp;
    const float* sc_s = v_s + tc * cols;
    float* out_p = out + (int64_t)t0 * out_stride + (int64_t)h * out_cols;
#pragma unroll REC_UNROLL_TOKENS
    for (int tt = 0; tt < nt; ++tt) {
      const float vj = v_s[tt * cols + cix];
      float keep = 0.f, take = 0.f;
      if (mode >= 1) {
        keep = sc_s[tt];
        take = sc_s[tc + tt];
      }
      float o = 0.f;
      const float4* q4 = reinterpret_cast<const float4*>(q_s + tt * dkp);
      const float4* g4 = reinterpret_cast<const float4*>(g_s + tt * dkp);
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; ++i4) {
        const float4 qq = q4[i4 * lanes], gg = g4[i4 * lanes];
        const float qa[4] = {qq.x, qq.y, qq.z, qq.w}, ga[4] = {gg.x, gg.y, gg.z, gg.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i4 * 4 + e;
          const float a = mode >= 1 ? keep : ga[e];
          const float b = mode >= 1 ? take * ga[e] : 1.0f - ga[e];
          if (mode == 2) S[i] += fmaf(b, vj, -(keep * S[i]));       // keep holds 1 - decay here
          else S[i] = a * S[i] + b * vj;
          o = fmaf(S[i], qa[e], o);
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        if (off < lanes) o += __shfl_xor_sync(0xffffffffu, o, off);      // (lanes is the same for the whole grid)
      if (sub == 0 && live) out_p[col] = o;
      if (mode == 1 && blockIdx.x == 0 && threadIdx.x == 0) out_p[dv + 1] = sc_s[2 * tc + tt];
      out_p += out_stride;
    }
    if (next < end) stash(nt_next, bufs + (which ^ 1) * buf_floats);
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = ((i >> 2) * lanes + sub) * 4 + (i & 3);
      if (d < dk) sp[d] = S[i];
    }
  }
}

// --------------------------------------------------------------- one token per request
// Steps in which every request brings a single token (decoding) have no chain to follow: each state element is
// read, updated and written once, so these kernels are laid out for the memory system instead.  A thread owns
// four neighbouring elements of a state row (one 16-byte access each way when the row length allows), takes its
// operands straight from global memory, and the threads that share a row add their parts by shuffles.
template <typename T>
__global__ void __launch_bounds__(128)
selective_scan_step_kernel(const T* __restrict__ xc, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                           const float* __restrict__ A, const T* __restrict__ bc, int64_t bc_stride, int b_off,
                           int c_off, const float* __restrict__ D, const T* __restrict__ xz, int64_t xz_stride,
                           int z_off, float* __restrict__ ssm_state, float* __restrict__ conv_state,
                           const int* __restrict__ cu_q, const int* __restrict__ state_slots, T* __restrict__ out,
                           int channels, int n_state, int taps, int lanes) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int per_block = 128 / lanes;
  const int c = blockIdx.x * per_block + threadIdx.x / lanes;
  const int sub = threadIdx.x % lanes;
  const int t = cu_q[r];
  if (cu_q[r + 1] - t != 1) return;                       // (the host picks this kernel for single tokens only)
  const int slot = state_slots[r];
  const bool live = c < channels;
  const int cc = live ? c : 0;
  const float dt = softplusf_(dt_raw[(int64_t)t * channels + cc] + dt_bias[cc]);
  const float x = to_float(xc[(int64_t)t * channels + cc]);
  const float dx = dt * x;
  const T* brow = bc + (int64_t)t * bc_stride;
  float* sp = ssm_state + ((int64_t)slot * channels + cc) * n_state;
  const bool vec = (n_state & 3) == 0;
  float y = 0.f;
  for (int n0 = sub * 4; n0 < n_state; n0 += lanes * 4) {
    float S[4], a[4];
    if (vec) {
      const float4 s4 = *reinterpret_cast<const float4*>(sp + n0);
      const float4 a4 = *reinterpret_cast<const float4*>(A + (int64_t)cc * n_state + n0);
      S[0] = s4.x; S[1] = s4.y; S[2] = s4.z; S[3] = s4.w;
      a[0] = a4.x; a[1] = a4.y; a[2] = a4.z; a[3] = a4.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const bool ok = n0 + e < n_state;
        S[e] = ok ? sp[n0 + e] : 0.f;
        a[e] = ok ? A[(int64_t)cc * n_state + n0 + e] : 0.f;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (n0 + e < n_state) {
        S[e] = exp2f(dt * (a[e] * 1.4426950408889634f)) * S[e] + dx * to_float(brow[b_off + n0 + e]);
        y = fmaf(S[e], to_float(brow[c_off + n0 + e]), y);
      }
    }
    if (live) {
      if (vec) {
        *reinterpret_cast<float4*>(sp + n0) = make_float4(S[0], S[1], S[2], S[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (n0 + e < n_state) sp[n0 + e] = S[e];
      }
    }
  }
  for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
  if (sub == 0 && live) {
    const float z = to_float(xz[(int64_t)t * xz_stride + z_off + cc]);
    out[(int64_t)t * channels + cc] = from_float<T>((y + D[cc] * x) * siluf_(z));
    const int keep = taps - 1;                           // the convolution's memory moves on by one input
    float* cs = conv_state + (int64_t)slot * keep * channels + cc;
    for (int k = 0; k + 1 < keep; ++k) cs[(int64_t)k * channels] = cs[(int64_t)(k + 1) * channels];
    if (keep > 0) cs[(int64_t)(keep - 1) * channels] = to_float(xz[(int64_t)t * xz_stride + cc]);
  }
}

template <typename T>
__global__ void __launch_bounds__(REC_THREADS)
matrix_recurrence_step_kernel(int mode, const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k,
                              int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
                              const float* __restrict__ gates, int64_t gates_stride, const float* __restrict__ gate_bias,
                              const float* __restrict__ lower, float q_scale, float* __restrict__ state,
                              const int* __restrict__ cu_q,
                              const int* __restrict__ state_slots, float* __restrict__ out, int64_t out_stride, int heads,
                              int dk, int dv, int lanes, int kv_div) {
  pdl_trigger();
  pdl_wait();
  const int cols = REC_THREADS / lanes;
  const int dvx = dv + (mode == 1 ? 1 : 0);
  const int out_cols = dv + (mode == 1 ? 2 : 0);
  const int r = blockIdx.z, h = blockIdx.y;
  const int col = blockIdx.x * cols + threadIdx.x / lanes;
  const int sub = threadIdx.x % lanes;
  const int64_t t = cu_q[r];
  if (cu_q[r + 1] - t != 1) return;
  const int slot = state_slots[r];
  const bool live = col < dvx;
  float keep = 0.f, take = 0.f, m_new = 0.f;
  if (mode == 1) {
    const float* g = gates + t * gates_stride;            // the gate scan's work: i | f | m before | m after
    m_new = g[3 * heads + h];
    keep = expf(g[heads + h] + g[2 * heads + h] - m_new);
    take = expf(g[h] - m_new);
  } else if (mode == 2) {
    take = softplusf_(gates[t * gates_stride + h] + gate_bias[h]);          // the step size
    keep = -expm1f(lower[h] * take);                                        // what the state loses, 1 - decay
  }
  const float vj = !live ? 0.f : (col < dv ? to_float(v[t * v_stride + (int64_t)h * dv + col]) : 1.0f);
  float* sp = state + (((int64_t)slot * heads + h) * dvx + (live ? col : 0)) * dk;
  const bool vec = (dk & 3) == 0;
  float o = 0.f;
  for (int d0 = sub * 4; d0 < dk; d0 += lanes * 4) {
    float S[4];
    if (vec) {
      const float4 s4 = *reinterpret_cast<const float4*>(sp + d0);
      S[0] = s4.x; S[1] = s4.y; S[2] = s4.z; S[3] = s4.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) S[e] = d0 + e < dk ? sp[d0 + e] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = d0 + e;
      if (d < dk) {
        const int hd = h * dk + d, kd = (h / kv_div) * dk + d;
        float a, b, qe;
        if (mode >= 1) {
          a = keep;
          b = take * to_float(k[t * k_stride + kd]);
          qe = to_float(q[t * q_stride + kd]) * q_scale;
        } else {
          const float lo = lower[hd];
          a = lo + (1.0f - lo) * sigmoidf_(gates[t * gates_stride + hd] + gate_bias[hd]);
          b = 1.0f - a;
          qe = siluf_(to_float(q[t * q_stride + hd]));
        }
        if (mode == 2) S[e] += fmaf(b, vj, -(keep * S[e]));
        else S[e] = a * S[e] + b * vj;
        o = fmaf(S[e], qe, o);
      }
    }
    if (live) {
      if (vec) {
        *reinterpret_cast<float4*>(sp + d0) = make_float4(S[0], S[1], S[2], S[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (d0 + e < dk) sp[d0 + e] = S[e];
      }
    }
  }
  for (int off = lanes >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
  float* orow = out + t * out_stride + (int64_t)h * out_cols;
  if (sub == 0 && live) orow[col] = o;
  if (mode == 1 && blockIdx.x == 0 && threadIdx.x == 0) orow[dv + 1] = expf(-m_new);
}

// --------------------------------------------------------------- per-head output norm
// One warp per (token, head): o [dv] (fp32, optionally divided by max(|o[dv]|, o[dv+1]) + den_eps, the
// two extra columns the recurrence wrote), divided by its root mean square, times a weight (shared by
// the heads when w_head_stride is 0), times sigmoid(gate) when a gate is given.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kernel(const float* __restrict__ o, int64_t o_stride, int o_cols, int with_den, float den_eps,
                 const float* __restrict__ w, int w_head_stride, const T* __restrict__ gate, int64_t gate_stride,
                 T* __restrict__ out, int64_t out_stride, int n_tokens, int heads, int dv, float eps) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * 4 + warp;
  if (item >= (int64_t)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (int64_t)t * heads);
  const float* row = o + (int64_t)t * o_stride + (int64_t)h * o_cols;
  float inv_den = 1.0f;
  if (with_den) inv_den = 1.0f / (fmaxf(fabsf(row[dv]), row[dv + 1]) + den_eps);
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float x = with_den ? row[c] * inv_den : row[c];
    ss = fmaf(x, x, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    float x = (with_den ? row[c] * inv_den : row[c]) * inv * w[(int64_t)h * w_head_stride + c];
    if (gate) x *= sigmoidf_(to_float(gate[(int64_t)t * gate_stride + (int64_t)h * dv + c]));
    out[(int64_t)t * out_stride + (int64_t)h * dv + c] = from_float<T>(x);
  }
}

// --------------------------------------------------------------- gated norm over groups of columns
// One block per (token, group of `group_width` neighbouring columns):
//     u[c] = (y[c] + skip[c / head_width] * x[c]) * silu(z[c])        (the skip term only with `skip`)
//     out[c] = u[c] / sqrt(mean over the group of u^2 + eps) * w[c]
// y is the fp32 read-out of a recurrence, x its input and z the gate, both of the activation type.  The gate comes
// BEFORE the norm, and the groups need not be heads.  Two passes over the group's columns; everything in fp32.
template <typename T>
__global__ void __launch_bounds__(1024)
gated_group_norm_kernel(const float* __restrict__ y, int64_t y_stride, const T* __restrict__ x, int64_t x_stride,
                        const float* __restrict__ skip, int head_width, const T* __restrict__ z, int64_t z_stride,
                        const float* __restrict__ w, T* __restrict__ out, int64_t out_stride, int group_width,
                        float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int c0 = blockIdx.y * group_width;
  auto gated = [&](int c) {
    float u = y[t * y_stride + c];
    if (skip) u = fmaf(skip[c / head_width], to_float(x[t * x_stride + c]), u);
    return u * siluf_(to_float(z[t * z_stride + c]));
  };
  float ss = 0.f;
  for (int c = c0 + threadIdx.x; c < c0 + group_width; c += blockDim.x) {
    const float u = gated(c);
    ss = fmaf(u, u, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)group_width + eps);
  for (int c = c0 + threadIdx.x; c < c0 + group_width; c += blockDim.x)
    out[t * out_stride + c] = from_float<T>(gated(c) * inv * w[c]);
}

// The convolution's state after a step: of (old state ++ this step's inputs) the last taps-1 rows, per request.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_advance_kernel(const T* __restrict__ x, int64_t x_stride, float* __restrict__ conv_state,
                          const int* __restrict__ cu_q, const int* __restrict__ state_slots, int channels, int taps) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t0 = cu_q[r], len = cu_q[r + 1] - t0;
  const int keep = taps - 1;
  float* cs = conv_state + (int64_t)state_slots[r] * keep * channels + c;
  for (int j = 0; j < keep; ++j) {           // ascending: a row is read before the row that overwrites it is written
    const int src = j + len;                 // row of (old state ++ inputs)
    cs[(int64_t)j * channels] =
        src < keep ? cs[(int64_t)src * channels] : to_float(x[(int64_t)(t0 + src - keep) * x_stride + c]);
  }
}

inline int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

template <typename T>
int conv_silu_launch(const T* x, int64_t x_stride, const float* w, const float* bias, const float* conv_state,
                     const int* positions, const int* token_row, T* out, int n_tokens, int channels, int taps,
                     cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS || (channels + 255) / 256 > 65535) return (int)cudaErrorInvalidValue;
  return gllm_launch(conv_silu_kernel<T>, dim3(n_tokens, (channels + 255) / 256), dim3(256), 0, stream, x, x_stride, w,
                     bias, conv_state, positions, token_row, out, n_tokens, channels, taps);
}

template <typename T>
int selective_scan_launch(const T* xc, const float* dt_raw, const float* dt_bias, const float* A, const T* bc,
                          int64_t bc_stride, int b_off, int c_off, const float* D, const T* xz, int64_t xz_stride,
                          int z_off, float* ssm_state, float* conv_state, const int* cu_q, const int* state_slots,
                          T* out, int num_requests, int max_q_len, int channels, int n_state, int taps,
                          cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (max_q_len == 1 && taps >= 1 && taps <= MAX_TAPS && num_requests <= 65535) {
    int lanes = pow2_at_least((n_state + 3) / 4);
    if (lanes > 32) lanes = 32;
    const int per_block = 128 / lanes;
    return gllm_launch(selective_scan_step_kernel<T>, dim3((channels + per_block - 1) / per_block, num_requests),
                       dim3(128), 0, stream, xc, dt_raw, dt_bias, A, bc, bc_stride, b_off, c_off, D, xz, xz_stride, z_off,
                       ssm_state, conv_state, cu_q, state_slots, out, channels, n_state, taps, lanes);
  }
  const int npt = n_state <= 64 ? 2 : 8;
  const int lanes = pow2_at_least((n_state + npt - 1) / npt);
  if (lanes > 32 || taps < 1 || taps > MAX_TAPS || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const int threads = (int64_t)channels * lanes >= 4096 ? 512 : 128;
  const int per_block = threads / lanes;
  // tokens per chunk: as many as a thread's look-ahead registers hold of the chunk's values
  int tc = SCAN_MAX_CHUNK;
  while (tc > 1 && (tc * 2 * n_state > threads * SCAN_PF_BC || tc * per_block > threads * SCAN_PF_CH)) tc >>= 1;
  if (tc * 2 * n_state > threads * SCAN_PF_BC || tc * per_block > threads * SCAN_PF_CH)
    return (int)cudaErrorInvalidValue;
  const size_t smem = 2 * sizeof(float) * (size_t)tc * (2 * n_state + 3 * per_block);
  void (*kernel)(const T*, const float*, const float*, const float*, const T*, int64_t, int, int, const float*, const T*,
                 int64_t, int, float*, float*, const int*, const int*, T*, int, int, int, int, int);
  if (threads == 512) kernel = npt == 2 ? selective_scan_kernel<T, 2, 512> : selective_scan_kernel<T, 8, 512>;
  else kernel = npt == 2 ? selective_scan_kernel<T, 2, 128> : selective_scan_kernel<T, 8, 128>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return gllm_launch(kernel, dim3((channels + per_block - 1) / per_block, num_requests), dim3(threads), smem, stream, xc,
                     dt_raw, dt_bias, A, bc, bc_stride, b_off, c_off, D, xz, xz_stride, z_off, ssm_state, conv_state, cu_q,
                     state_slots, out, channels, n_state, taps, lanes, tc);
}

template <typename T>
int matrix_recurrence_launch(int mode, const T* q, int64_t q_stride, const T* k, int64_t k_stride, const T* v,
                             int64_t v_stride, const float* gates, int64_t gates_stride, const float* gate_bias,
                             const float* lower, float cap, float q_scale, float* state, float* mstate, float* work,
                             const int* cu_q, const int* state_slots, float* out, int64_t out_stride,
                             int num_requests, int max_q_len, int heads, int dk, int dv, int kv_div,
                             cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (heads > 65535 || num_requests > 65535 || dk < 1 || dv < 1 || dk > 512 || mode < 0 || mode > 2 || kv_div < 1 ||
      heads % kv_div || (mode == 2 && (k == nullptr || lower == nullptr)))
    return (int)cudaErrorInvalidValue;
  const int dvx = dv + (mode == 1 ? 1 : 0);
  if (mode == 1) {
    if (work == nullptr || mstate == nullptr) return (int)cudaErrorInvalidValue;
    const int rc = gllm_launch(exp_gate_scan_kernel, dim3(num_requests), dim3(128), 0, stream, gates, gates_stride,
                               gate_bias, cap, mstate, cu_q, state_slots, work, heads);
    if (rc != 0) return rc;
    gates = work;
    gates_stride = 4 * (int64_t)heads;
  }
  if (max_q_len == 1) {
    int lanes = pow2_at_least((dk + 3) / 4);
    if (lanes > 32) lanes = 32;
    const int cols = REC_THREADS / lanes;
    return gllm_launch(matrix_recurrence_step_kernel<T>, dim3((dvx + cols - 1) / cols, heads, num_requests),
                       dim3(REC_THREADS), 0, stream, mode, q, q_stride, k, k_stride, v, v_stride, gates, gates_stride,
                       gate_bias, lower, q_scale, state, cu_q, state_slots, out, out_stride, heads, dk, dv, lanes, kv_div);
  }
  int dpt = dk <= 128 ? 4 : 16;
  // the step-sized recurrence has many heads of many value columns: with 65 .. 256 key channels eight per thread
  // measured 1.2x faster than four (1.00 against 1.23 ms for 64 heads of 128 x 64 over 2,048 tokens); up to 64, four
  if (mode == 2 && dk > 64 && dk <= 256) dpt = 8;
  if (const char* e = getenv("GLLM_B200_REC_DPT")) {          // for measurements: key channels a thread keeps
    const int want = atoi(e);
    if ((want == 4 || want == 8 || want == 16) && want * 32 >= dk) dpt = want;
  }
  int lanes = pow2_at_least((dk + dpt - 1) / dpt);
  if (lanes < 2) lanes = 2;
  const int threads = REC_THREADS;
  const int cols = threads / lanes;
  const int dkp = lanes * dpt;
  int tc = REC_MAX_CHUNK;
  while (tc > 1 && (tc * dkp > REC_LOOKAHEAD || tc * cols > REC_LOOKAHEAD)) tc >>= 1;
  if (tc * dkp > REC_LOOKAHEAD || tc * cols > REC_LOOKAHEAD) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * 2 * (size_t)tc * (2 * dkp + cols + 4);
  void (*kernel)(int, const T*, int64_t, const T*, int64_t, const T*, int64_t, const float*, int64_t, const float*,
                 const float*, float, float*, const int*, const int*, float*, int64_t, int, int, int, int, int, int);
#define GLLM_REC_PICK(M)                                                                            \
  kernel = dpt == 4 ? matrix_recurrence_kernel<T, 4, REC_THREADS, M>                                \
                    : (dpt == 8 ? matrix_recurrence_kernel<T, 8, REC_THREADS, M> : matrix_recurrence_kernel<T, 16, REC_THREADS, M>)
  if (mode == 2) GLLM_REC_PICK(2);
  else if (mode == 1) GLLM_REC_PICK(1);
  else GLLM_REC_PICK(0);
#undef GLLM_REC_PICK
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return gllm_launch(kernel, dim3((dvx + cols - 1) / cols, heads, num_requests), dim3(threads), smem, stream, mode, q,
                     q_stride, k, k_stride, v, v_stride, gates, gates_stride, gate_bias, lower, q_scale, state, cu_q,
                     state_slots, out, out_stride, heads, dk, dv, lanes, tc, kv_div);
}

template <typename T>
int head_norm_launch(const float* o, int64_t o_stride, int o_cols, int with_den, float den_eps, const float* w,
                     int w_head_stride, const T* gate, int64_t gate_stride, T* out, int64_t out_stride, int n_tokens,
                     int heads, int dv, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int64_t blocks = ((int64_t)n_tokens * heads + 3) / 4;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(head_norm_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, stream, o, o_stride, o_cols, with_den,
                     den_eps, w, w_head_stride, gate, gate_stride, out, out_stride, n_tokens, heads, dv, eps);
}

template <typename T>
int gated_group_norm_launch(const float* y, int64_t y_stride, const T* x, int64_t x_stride, const float* skip,
                            int head_width, const T* z, int64_t z_stride, const float* w, T* out, int64_t out_stride,
                            int n_tokens, int groups, int group_width, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (groups < 1 || groups > 65535 || group_width < 1 || (skip != nullptr && (x == nullptr || head_width < 1)))
    return (int)cudaErrorInvalidValue;
  // wide groups of few tokens (single decoded tokens: a handful of blocks in all) get 1,024 threads a block, four
  // columns a thread and pass; otherwise 256
  const bool few = (int64_t)n_tokens * groups < 2 * gllm_sm_count();
  const int cap = few ? 1024 : 256;
  const int threads = group_width >= cap ? cap : (group_width + 31) / 32 * 32;
  return gllm_launch(gated_group_norm_kernel<T>, dim3(n_tokens, groups), dim3(threads), 0, stream, y, y_stride, x,
                     x_stride, skip, head_width, z, z_stride, w, out, out_stride, group_width, eps);
}

template <typename T>
int conv_state_advance_launch(const T* x, int64_t x_stride, float* conv_state, const int* cu_q, const int* state_slots,
                              int num_requests, int channels, int taps, cudaStream_t stream) {
  if (num_requests <= 0 || taps <= 1) return 0;
  if (num_requests > 65535 || taps > MAX_TAPS) return (int)cudaErrorInvalidValue;
  return gllm_launch(conv_state_advance_kernel<T>, dim3((channels + 255) / 256, num_requests), dim3(256), 0, stream, x,
                     x_stride, conv_state, cu_q, state_slots, channels, taps);
}
}  // namespace

#define GLLM_RECURRENT_EXPORTS(T, S)                                                                                  \
  GLLM_API int gllm_conv_silu_##S(const T* x, int64_t x_stride, const float* w, const float* bias,                    \
                                  const float* conv_state, const int* positions, const int* token_row, T* out,        \
                                  int n_tokens, int channels, int taps, cudaStream_t stream) {                        \
    return conv_silu_launch<T>(x, x_stride, w, bias, conv_state, positions, token_row, out, n_tokens, channels, taps, \
                               stream);                                                                               \
  }                                                                                                                   \
  GLLM_API int gllm_selective_scan_##S(const T* xc, const float* dt_raw, const float* dt_bias, const float* A,        \
                                       const T* bc, int64_t bc_stride, int b_off, int c_off, const float* D,          \
                                       const T* xz, int64_t xz_stride, int z_off, float* ssm_state, float* conv_state, \
                                       const int* cu_q, const int* state_slots, T* out, int num_requests,             \
                                       int max_q_len, int channels, int n_state, int taps, cudaStream_t stream) {     \
    return selective_scan_launch<T>(xc, dt_raw, dt_bias, A, bc, bc_stride, b_off, c_off, D, xz, xz_stride, z_off,     \
                                    ssm_state, conv_state, cu_q, state_slots, out, num_requests, max_q_len, channels, \
                                    n_state, taps, stream);                                                           \
  }                                                                                                                   \
  GLLM_API int gllm_matrix_recurrence_##S(int mode, const T* q, int64_t q_stride, const T* k, int64_t k_stride,       \
                                          const T* v, int64_t v_stride, const float* gates, int64_t gates_stride,     \
                                          const float* gate_bias, const float* lower, float cap, float q_scale,       \
                                          float* state, float* mstate, float* work, const int* cu_q,                  \
                                          const int* state_slots, float* out, int64_t out_stride, int num_requests,   \
                                          int max_q_len, int heads, int dk, int dv, int kv_div,                       \
                                          cudaStream_t stream) {                                                      \
    return matrix_recurrence_launch<T>(mode, q, q_stride, k, k_stride, v, v_stride, gates, gates_stride, gate_bias,   \
                                       lower, cap, q_scale, state, mstate, work, cu_q, state_slots, out, out_stride,  \
                                       num_requests, max_q_len, heads, dk, dv, kv_div, stream);                       \
  }                                                                                                                   \
  GLLM_API int gllm_head_norm_##S(const float* o, int64_t o_stride, int o_cols, int with_den, float den_eps,          \
                                  const float* w, int w_head_stride, const T* gate, int64_t gate_stride, T* out,      \
                                  int64_t out_stride, int n_tokens, int heads, int dv, float eps,                     \
                                  cudaStream_t stream) {                                                              \
    return head_norm_launch<T>(o, o_stride, o_cols, with_den, den_eps, w, w_head_stride, gate, gate_stride, out,      \
                               out_stride, n_tokens, heads, dv, eps, stream);                                         \
  }                                                                                                                   \
  GLLM_API int gllm_gated_group_norm_##S(const float* y, int64_t y_stride, const T* x, int64_t x_stride,              \
                                         const float* skip, int head_width, const T* z, int64_t z_stride,             \
                                         const float* w, T* out, int64_t out_stride, int n_tokens, int groups,        \
                                         int group_width, float eps, cudaStream_t stream) {                           \
    return gated_group_norm_launch<T>(y, y_stride, x, x_stride, skip, head_width, z, z_stride, w, out, out_stride,    \
                                      n_tokens, groups, group_width, eps, stream);                                    \
  }                                                                                                                   \
  GLLM_API int gllm_conv_state_advance_##S(const T* x, int64_t x_stride, float* conv_state, const int* cu_q,          \
                                           const int* state_slots, int num_requests, int channels, int taps,          \
                                           cudaStream_t stream) {                                                     \
    return conv_state_advance_launch<T>(x, x_stride, conv_state, cu_q, state_slots, num_requests, channels, taps,     \
                                        stream);                                                                      \
  }

GLLM_RECURRENT_EXPORTS(float, f32)
GLLM_RECURRENT_EXPORTS(__nv_bfloat16, bf16)
