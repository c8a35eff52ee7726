// Differential attention of the bf16 path on the tensor cores, over the paged cache (see attention_diff.cu for the
// mechanism and the page layout: [kv_heads, block_size, 2 * dk] keys, two maps side by side, then
// [kv_heads, block_size, dv] values).
//
// Two kernels.  diff_mma: one CTA (4 warps) owns 64 rows = (64 / G') query tokens x G' query heads that share one
// key head, for ONE of the two maps; key and value tiles of 64 keys are fetched page by page with cp.async in two
// stages; S = Q K^T and O += P V run as mma.sync m16n8k16 with fp32 accumulation; the scores are capped,
// cap * tanh(s * scale / cap), with the tanh formed as 1 - 2 / (1 + e^(2y)) from one exponential and one
// reciprocal (absolute error about 1e-7, where tanh.approx would lose three digits of a score near the cap); a
// running maximum and sum per row, probabilities rounded to bf16 for the second product.  A CTA may take only a
// range of a request's key tiles (`splits` > 1: single decoded tokens over long contexts get enough CTAs to stream
// them).  It writes the unnormalised fp32 result with its maximum and sum.  diff_combine: one warp per
// (token, head) merges the ranges of each map, forms o = a1 - lambda * a2, divides by the root mean square over dv,
// multiplies by out_scale and sigmoid(gate), and rounds to bf16.  Everything but the two products' operands is fp32.
// Key tiles are aligned to absolute positions, so a result does not depend on how the request was cut into steps.
#include "mma_utils.cuh"

namespace {
constexpr int BM = 64, BN = 64, DM_THREADS = 128;
static_assert(DM_THREADS == 2 * BN, "two threads fetch a key");
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_BIG = -1e30f;

template <int C>
__device__ __forceinline__ int swz(int row, int piece) {
  if (C % 8 == 0) return piece ^ (row & 7);
  return piece ^ ((row >> 1) & 3);
}

// partial: [split][map][token][head][DV] fp32; stats: [split][map][token][head][2] = (maximum in log2 units, sum)
template <int DK, int DV>
__global__ void __launch_bounds__(DM_THREADS)
diff_mma_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride, float* __restrict__ partial,
                float* __restrict__ stats, int n_tokens, const __nv_bfloat16* __restrict__ cache,
                const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
                const int* __restrict__ ctx_lens, const int* __restrict__ slots, int hq, int hkv, int gp,
                int block_size, int num_pages, float scale, float softcap, int splits, int tiles_per_split,
                int* __restrict__ status) {
  constexpr int CK = DK / 8, CV = DV / 8;
  constexpr int K_BYTES = BN * DK * 2, V_BYTES = BN * DV * 2;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* q_sm = smem_raw;                       // [BM][DK]
  unsigned char* kv_sm = smem_raw + BM * DK * 2;        // [2 stages][K [BN][DK] | V [BN][DV]]

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.z;
  const int map = blockIdx.y & 1, ytile = blockIdx.y >> 1;
  const int group = hq / hkv;
  const int tiles_per_kv = group / gp;
  const int kvh = ytile / tiles_per_kv;
  const int h0 = kvh * group + (ytile - kvh * tiles_per_kv) * gp;
  const int qt = BM / gp;
  const int tok_begin = cu_q[r], q_len = cu_q[r + 1] - tok_begin;
  const int n_qtiles = (q_len + qt - 1) / qt;
  const int split = blockIdx.x % splits;
  const int xt = blockIdx.x / splits;
  if (xt >= n_qtiles) return;
  const int qtile = n_qtiles - 1 - xt;                  // longest rows first
  const int t0 = qtile * qt;
  const int t_count = min(qt, q_len - t0);
  const int ctx = ctx_lens[r];
  const int* bt = block_table + (int64_t)slots[r] * bt_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;

  const int pos_first = ctx + t0, pos_last = ctx + t0 + t_count - 1;
  int tile_first = 0, tile_last = pos_last / BN;
  if (splits > 1) {
    tile_first = split * tiles_per_split;
    tile_last = min(tile_last, tile_first + tiles_per_split - 1);
  }

  const int64_t page_elems = (int64_t)hkv * block_size * (2 * DK + DV);
  const int64_t v_region = (int64_t)hkv * block_size * 2 * DK;

  int qpos[2];
  bool row_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = warp * 16 + g8 + 8 * i;
    const int tl = rr / gp;
    row_ok[i] = tl < t_count;
    qpos[i] = pos_first + tl;
  }
  float o[DV / 8][4];
#pragma unroll
  for (int nd = 0; nd < DV / 8; ++nd)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nd][e] = 0.f;
  float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.f, 0.f};
  const float to_exponent = 2.0f * LOG2E * scale / softcap;      // e^(2y) = 2^(s * to_exponent), y = s * scale / cap
  const float cap2 = softcap * LOG2E;                            // the capped score in log2 units

  if (tile_first <= tile_last) {
    for (int idx = threadIdx.x; idx < BM * CK; idx += DM_THREADS) {
      const int rr = idx / CK, piece = idx - rr * CK;
      const int tl = rr / gp, g = rr - tl * gp;
      const bool ok = tl < t_count;
      const __nv_bfloat16* src =
          q + (int64_t)(tok_begin + t0 + (ok ? tl : 0)) * q_stride + (int64_t)((h0 + g) * 2 + map) * DK + piece * 8;
      cp_async16(smem_u32(q_sm + (rr * CK + swz<CK>(rr, piece)) * 16), src, ok);
    }
    // two threads a key: one page look-up each, then the key's 16-byte pieces in turn (keys first, values after)
    auto load_kv = [&](int tile, int stage) {
      unsigned char* k_dst = kv_sm + stage * (K_BYTES + V_BYTES);
      unsigned char* v_dst = k_dst + K_BYTES;
      const int row = threadIdx.x >> 1, half = threadIdx.x & 1;
      const int key = tile * BN + row;
      bool ok = key <= pos_last;
      int page = 0;
      if (ok) {
        page = bt[key / block_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(status, GLLM_STATUS_PAGE_RANGE);
          ok = false;
          page = 0;
        }
      }
      const int off = key % block_size;
      const __nv_bfloat16* k_src =
          ok ? cache + (int64_t)page * page_elems + ((int64_t)kvh * block_size + off) * 2 * DK + map * DK : cache;
      const __nv_bfloat16* v_src =
          ok ? cache + (int64_t)page * page_elems + v_region + ((int64_t)kvh * block_size + off) * DV : cache;
#pragma unroll
      for (int piece = half; piece < CK; piece += 2)
        cp_async16(smem_u32(k_dst + (row * CK + swz<CK>(row, piece)) * 16), ok ? k_src + piece * 8 : cache, ok);
#pragma unroll
      for (int piece = half; piece < CV; piece += 2)
        cp_async16(smem_u32(v_dst + (row * CV + swz<CV>(row, piece)) * 16), ok ? v_src + piece * 8 : cache, ok);
    };
    load_kv(tile_first, 0);
    cp_async_commit();
    uint32_t qf[DK / 16][4];

    for (int tile = tile_first; tile <= tile_last; ++tile) {
      const int stage = (tile - tile_first) & 1;
      if (tile < tile_last) {
        load_kv(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (tile == tile_first) {
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
          const int mat = lane >> 3, rl = lane & 7;
          const int row = warp * 16 + (mat & 1) * 8 + rl;
          const int piece = 2 * ks + (mat >> 1);
          ldmatrix_x4(qf[ks], smem_u32(q_sm + (row * CK + swz<CK>(row, piece)) * 16));
        }
      }
      const unsigned char* k_sm = kv_sm + stage * (K_BYTES + V_BYTES);
      const unsigned char* v_sm = k_sm + K_BYTES;
      const int kv0 = tile * BN;

      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          const int mat = lane >> 3, rl = lane & 7;
          const int row = np * 16 + (mat >> 1) * 8 + rl;
          const int piece = 2 * ks + (mat & 1);
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(k_sm + (row * CK + swz<CK>(row, piece)) * 16));
          mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
      }
      // ---- capped scores in log2 units; hidden keys are marked
      const bool need_mask = (kv0 + BN - 1 > pos_first) || (t_count < qt);
      float tmax[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const float ex = fast_exp2(s[nt][e] * to_exponent);
          float x = cap2 * (1.0f - __fdividef(2.0f, 1.0f + ex));
          if (need_mask) {
            const int key = kv0 + nt * 8 + 2 * t4 + (e & 1);
            if (!row_ok[i] || key > qpos[i]) x = NEG_BIG;
          }
          s[nt][e] = x;
          tmax[i] = fmaxf(tmax[i], x);
        }
      float corr[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
        tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
        const float m_new = fmaxf(m_run[i], tmax[i]);
        corr[i] = fast_exp2(m_run[i] - m_new);
        m_run[i] = m_new;
        l_run[i] *= corr[i];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const float p = s[nt][e] <= NEG_BIG ? 0.f : fast_exp2(s[nt][e] - m_run[i]);
          s[nt][e] = p;
          l_run[i] += p;
        }
#pragma unroll
      for (int nd = 0; nd < DV / 8; ++nd) {
        o[nd][0] *= corr[0];
        o[nd][1] *= corr[0];
        o[nd][2] *= corr[1];
        o[nd][3] *= corr[1];
      }
      // ---- O += P V
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nd2 = 0; nd2 < DV / 16; ++nd2) {
          const int mat = lane >> 3, rl = lane & 7;
          const int row = kk * 16 + (mat & 1) * 8 + rl;
          const int piece = 2 * nd2 + (mat >> 1);
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_u32(v_sm + (row * CV + swz<CV>(row, piece)) * 16));
          mma_bf16(o[2 * nd2], a, b[0], b[1]);
          mma_bf16(o[2 * nd2 + 1], a, b[2], b[3]);
        }
      }
      __syncthreads();
    }
  }
  // ---- store the unnormalised result with its maximum and sum
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    if (!row_ok[i]) continue;
    const int rr = warp * 16 + g8 + 8 * i;
    const int tl = rr / gp, g = rr - tl * gp;
    const int64_t token = tok_begin + t0 + tl;
    const int64_t item = (((int64_t)split * 2 + map) * n_tokens + token) * hq + (h0 + g);
    float* dst = partial + item * DV;
#pragma unroll
    for (int nd = 0; nd < DV / 8; ++nd)
      *reinterpret_cast<float2*>(dst + nd * 8 + 2 * t4) = make_float2(o[nd][2 * i], o[nd][2 * i + 1]);
    if (t4 == 0) *reinterpret_cast<float2*>(stats + item * 2) = make_float2(m_run[i], l_run[i]);
  }
}

// One warp per (token, head).
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ partial, const float* __restrict__ stats,
                    const __nv_bfloat16* __restrict__ gate, int64_t gate_stride, __nv_bfloat16* __restrict__ out,
                    int64_t out_stride, int n_tokens, int hq, int dv, int splits, float lambda, float eps,
                    float out_scale) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * 4 + warp;
  if (item >= (int64_t)n_tokens * hq) return;
  const int64_t per_map = (int64_t)n_tokens * hq;
  float o[8], ss = 0.f;                                 // dv <= 256
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = 0.f;
#pragma unroll
  for (int map = 0; map < 2; ++map) {
    // lane s holds the maximum and sum of range s (at most 32 ranges): one load each, all at once
    float2 st = make_float2(NEG_BIG, 0.f);
    if (lane < splits) st = *reinterpret_cast<const float2*>(stats + ((((int64_t)lane * 2 + map) * per_map + item) * 2));
    const float big = warp_max(st.y > 0.f ? st.x : NEG_BIG);
    const float w_mine = st.y > 0.f ? exp2f(st.x - big) : 0.f;
    const float total = warp_sum(st.y * w_mine);         // (lanes beyond the ranges add zeros)
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {                  // ascending ranges: one order of the sums
      const float w = __shfl_sync(0xffffffffu, w_mine, s);
      const float* row = partial + (((int64_t)s * 2 + map) * per_map + item) * dv;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) a[i] = fmaf(row[c], w, a[i]);
      }
    }
    const float inv = total > 0.f ? (map == 0 ? 1.0f : -lambda) / total : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = fmaf(a[i], inv, o[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(o[i], o[i], ss);
  ss = warp_sum(ss);
  const float mult = out_scale / sqrtf(ss / (float)dv + eps);
  const int64_t t = item / hq;
  const int h = (int)(item - t * hq);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) {
      float v = o[i] * mult;
      if (gate) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[t * gate_stride + (int64_t)h * dv + c])));
      out[t * out_stride + (int64_t)h * dv + c] = __float2bfloat16_rn(v);
    }
  }
}

template <int DK, int DV>
int diff_mma_launch(const __nv_bfloat16* q, int64_t q_stride, float* partial, float* stats, int n_tokens,
                    const __nv_bfloat16* cache, const int* block_table, int bt_stride, const int* cu_q,
                    const int* ctx_lens, const int* slots, int num_requests, int max_q_len, int hq, int hkv,
                    int block_size, int num_pages, float scale, float softcap, int splits, int tiles_per_split,
                    int* status, cudaStream_t stream) {
  const int group = hq / hkv;
  const int gp = (group <= BM && BM % group == 0) ? group : 1;
  const int qt = BM / gp;
  const size_t smem = (size_t)BM * DK * 2 + 2 * (size_t)BN * (DK + DV) * 2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(diff_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(((max_q_len + qt - 1) / qt) * splits, 2 * hkv * (group / gp), num_requests);
  return gllm_launch(diff_mma_kernel<DK, DV>, grid, dim3(DM_THREADS), smem, stream, q, q_stride, partial, stats,
                     n_tokens, cache, block_table, bt_stride, cu_q, ctx_lens, slots, hq, hkv, gp, block_size, num_pages,
                     scale, softcap, splits, tiles_per_split, status);
}
}  // namespace

GLLM_API int gllm_attention_diff_mma_supports(int dk, int dv) {
  return (dk == 32 || dk == 64 || dk == 128) && (dv == 32 || dv == 64 || dv == 96 || dv == 128);
}

// How many query tokens one CTA covers (the caller sizes its split decision with it).
GLLM_API int gllm_attention_diff_mma_tokens_per_tile(int hq, int hkv) {
  const int group = hq / hkv;
  return (group <= BM && BM % group == 0) ? BM / group : BM;
}

// partial: fp32 [splits][2][n_tokens][hq][dv]; stats: fp32 [splits][2][n_tokens][hq][2]; both are scratch.
GLLM_API int gllm_attention_diff_mma(const __nv_bfloat16* q, int64_t q_stride, const __nv_bfloat16* gate,
                                     int64_t gate_stride, __nv_bfloat16* out, int64_t out_stride, float* partial,
                                     float* stats, int n_tokens, const __nv_bfloat16* cache, const int* block_table,
                                     int bt_stride, const int* cu_q, const int* ctx_lens, const int* slots,
                                     int num_requests, int max_q_len, int hq, int hkv, int dk, int dv, int block_size,
                                     int num_pages, float scale, float softcap, float lambda, float eps,
                                     float out_scale, int splits, int tiles_per_split, int* status,
                                     cudaStream_t stream) {
  if (num_requests <= 0 || max_q_len <= 0 || n_tokens <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || hq % hkv || num_requests > 65535 || (q_stride % 8) || splits < 1 ||
      (splits > 1 && tiles_per_split < 1) || partial == nullptr || stats == nullptr || !(softcap > 0.f) ||
      splits > 32 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15))
    return (int)cudaErrorInvalidValue;
  int rc = (int)cudaErrorInvalidValue;
#define GLLM_DM(A, B)                                                                                               \
  if (dk == A && dv == B)                                                                                           \
    rc = diff_mma_launch<A, B>(q, q_stride, partial, stats, n_tokens, cache, block_table, bt_stride, cu_q, ctx_lens, \
                               slots, num_requests, max_q_len, hq, hkv, block_size, num_pages, scale, softcap,      \
                               splits, tiles_per_split, status, stream);
#define GLLM_DM_ROW(A) GLLM_DM(A, 32) GLLM_DM(A, 64) GLLM_DM(A, 96) GLLM_DM(A, 128)
  GLLM_DM_ROW(32) GLLM_DM_ROW(64) GLLM_DM_ROW(128)
#undef GLLM_DM_ROW
#undef GLLM_DM
  if (rc != 0) return rc;
  const int64_t blocks = ((int64_t)n_tokens * hq + 3) / 4;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(diff_combine_kernel, dim3((unsigned)blocks), dim3(128), 0, stream, partial, stats, gate,
                     gate_stride, out, out_stride, n_tokens, hq, dv, splits, lambda, eps, out_scale);
}
