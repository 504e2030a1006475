// Flash-attention forward for sm_100a: packed variable-length sequences (cu_seqlens), causal or
// full, grouped-query heads, head_dim 128, bf16 in / bf16 out, log-sum-exp saved for backward.
//
// One CTA per (128-row query tile, query head):
//   warp 0     : TMA producer   (Q once; K and V tiles in two 2-deep rings)
//   warp 1     : tcgen05 issuer (S = Q K^T into one of two TMEM buffers; O += P V)
//   warps 2..5 : softmax        (one query row per thread: tcgen05.ld of the S row, online max /
//                                sum in registers, P written to shared memory in the 128B-swizzled
//                                K-major layout the second MMA reads, O rescaled in TMEM only when
//                                a row maximum moved)
// S_{j+1} is issued before the softmax of S_j finishes, so the tensor core overlaps the
// exponentials.  Every mbarrier wait is bounded.
// Replaces the FlashAttention-3/4 wheels used by the reference
// (src/xorl/models/layers/attention/backend/flash_attention.py:382-531).
#include "common.cuh"

namespace xb_attn_fwd_ns {

constexpr int D = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int TILE_BYTES = 128 * D * 2;  // 32 KB: two 64-wide chunks of [128 rows][128 B]
constexpr int CHUNK_BYTES = 128 * 128;   // 16 KB
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int S_COL0 = 0, O_COL = 256;
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + TILE_BYTES;      // 2 stages
constexpr int SMEM_V = SMEM_K + 2 * TILE_BYTES;  // 2 stages
constexpr int SMEM_P = SMEM_V + 2 * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_P + TILE_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR + 256 + 1024;

struct Params {
  __nv_bfloat16* out;
  long long ldo;
  float* lse;  // [Hq, T]
  const int* cu_seqlens;
  const int* k_starts;  // optional: first K/V row of every sequence (defaults to cu_seqlens)
  int num_seqs;
  int T, Hq, Hkv;
  int causal;
  int window;          // > 0: a query sees only keys with q_pos - k_pos < window
  const float* sinks;  // optional fp32 [Hq]: one more logit per head in the softmax denominator
  float scale_log2;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, pv_done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  // ---- which (sequence, query tile) does this CTA own?  Heavy (late) tiles are scheduled first.
  const int tile_id = (int)gridDim.x - 1 - (int)blockIdx.x;
  int seq = -1, qt = 0, seq_start = 0, seq_len = 0;
  {
    int acc = 0;
    for (int b = 0; b < p.num_seqs; ++b) {
      const int s0 = p.cu_seqlens[b], s1 = p.cu_seqlens[b + 1];
      const int nt = (s1 - s0 + BQ - 1) / BQ;
      if (tile_id < acc + nt) {
        seq = b; qt = tile_id - acc; seq_start = s0; seq_len = s1 - s0;
        break;
      }
      acc += nt;
    }
  }
  if (seq < 0) return;  // uniform for the whole CTA, nothing allocated yet
  const int k_start = p.k_starts ? p.k_starts[seq] : seq_start;
  if (k_start < 0) return;  // this query block takes no part in the call
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q_row0 = qt * BQ;  // position inside the sequence
  const int kv_end = p.causal ? min(seq_len, q_row0 + BQ) : seq_len;
  // first key tile any row of this query tile can see under a sliding window
  const int kt0 = p.window > 0 ? max(0, q_row0 - p.window + 1) / BKV : 0;
  const int n_kv = max(0, (kv_end + BKV - 1) / BKV - kt0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + SMEM_BAR);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->s_empty[s], 128);
    }
    mbar_init(&bars->p_full, 128);
    mbar_init(&bars->pv_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, TILE_BYTES);
      tma_load_3d(smem + SMEM_Q, &tmap_q, &bars->q_full, 0, head, seq_start + q_row0);
      tma_load_3d(smem + SMEM_Q + CHUNK_BYTES, &tmap_q, &bars->q_full, 64, head,
                  seq_start + q_row0);
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int tok = k_start + (kt0 + j) * BKV;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_FWD, 100 + s)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        tma_load_3d(smem + SMEM_K + s * TILE_BYTES, &tmap_k, &bars->k_full[s], 0, kv_head, tok);
        tma_load_3d(smem + SMEM_K + s * TILE_BYTES + CHUNK_BYTES, &tmap_k, &bars->k_full[s], 64,
                    kv_head, tok);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_FWD, 110 + s)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        tma_load_3d(smem + SMEM_V + s * TILE_BYTES, &tmap_v, &bars->v_full[s], 0, kv_head, tok);
        tma_load_3d(smem + SMEM_V + s * TILE_BYTES + CHUNK_BYTES, &tmap_v, &bars->v_full[s], 64,
                    kv_head, tok);
        issued = j + 1;
      }
      if (!ok) {
        // bounded drain of copies that may still be landing in this CTA's shared memory
        const uint64_t t0 = xb_globaltimer();
        for (int j = max(0, issued - 2); j < issued; ++j) {
          while (!mbar_try_wait(&bars->k_full[j & 1], (j >> 1) & 1) &&
                 xb_globaltimer() - t0 < 200000000ull) {}
          while (!mbar_try_wait(&bars->v_full[j & 1], (j >> 1) & 1) &&
                 xb_globaltimer() - t0 < 200000000ull) {}
        }
        while (!mbar_try_wait(&bars->q_full, 0) && xb_globaltimer() - t0 < 200000000ull) {}
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = xb_idesc(1, 1, BQ, BKV, 0, 0);  // Q K^T : both K-major
      constexpr uint32_t idesc_o = xb_idesc(1, 1, BQ, D, 0, 1);    // P V   : V is MN-major
      constexpr uint64_t kmaj = xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t mnmaj = xb_smem_desc_base_sw128(CHUNK_BYTES, 1024);
      const uint32_t sq = xb_smem_u32(smem + SMEM_Q);
      const uint32_t sp = xb_smem_u32(smem + SMEM_P);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.status, XB_K_ATTN_FWD, 200);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->k_full[s], ph, abort_flag, p.status, XB_K_ATTN_FWD, 210 + s))
          return false;
        if (!mbar_wait(&bars->s_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_FWD, 220 + s))
          return false;
        tc_fence_after();
        const uint32_t sk = xb_smem_u32(smem + SMEM_K + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + S_COL0 + s * BKV, xb_smem_desc(kmaj, sq + off),
                        xb_smem_desc(kmaj, sk + off), idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->k_empty[s]);
        tc_commit(&bars->s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          if (!issue_s(j + 1)) { ok = false; break; }
        }
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->p_full, j & 1, abort_flag, p.status, XB_K_ATTN_FWD, 230)) {
          ok = false;
          break;
        }
        if (!mbar_wait(&bars->v_full[s], ph, abort_flag, p.status, XB_K_ATTN_FWD, 240 + s)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sv = xb_smem_u32(smem + SMEM_V + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint32_t a_off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;  // P: K-major over kv
          const uint32_t b_off = k * 2048;                               // V: 16 kv rows per step
          tc_mma_f16_ss(tmem_base + O_COL, xb_smem_desc(kmaj, sp + a_off),
                        xb_smem_desc(mnmaj, sv + b_off), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&bars->v_empty[s]);
        tc_commit(&bars->pv_done);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- softmax / epilogue -------------------------------
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;       // row inside the tile == TMEM lane
    const int row_pos = q_row0 + r;     // position inside the sequence
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    uint8_t* sp = smem + SMEM_P;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      // votes keep the warp together: tcgen05.ld / tcgen05.st below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], (j >> 1) & 1, abort_flag, p.status,
                                             XB_K_ATTN_FWD, 300 + s))) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sc[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t t[32];
        tmem_ld_32x32(tmem_base + lane_addr + S_COL0 + s * BKV + c * 32, t);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) sc[c * 32 + i] = __uint_as_float(t[i]);     // raw scores
      }
      tc_fence_before();
      mbar_arrive(&bars->s_empty[s]);

      const int col0 = (kt0 + j) * BKV;
      const bool need_mask = (col0 + BKV > seq_len) || (p.causal && col0 + BKV - 1 > q_row0) ||
                             (p.window > 0 && col0 < q_row0 + BQ - p.window);
      if (need_mask) {
        const int lim = p.causal ? min(seq_len - 1, row_pos) : seq_len - 1;  // last valid column
        const int lo = p.window > 0 ? row_pos - p.window + 1 : 0;            // first valid column
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (col0 + i > lim || col0 + i < lo) sc[i] = -INFINITY;
      }
      float mx_raw = -INFINITY;
#pragma unroll
      for (int i = 0; i < BKV; ++i) mx_raw = fmaxf(mx_raw, sc[i]);
      // m is the reference maximum (log2 units) that l and the O accumulator are relative to.  It
      // only moves when the running maximum grows by more than 2^8: P then stays below 256, exact
      // enough in bf16 with fp32 accumulation, and most steps skip the rescaling of O in TMEM.
      const float mx_t = mx_raw * p.scale_log2;              // -inf stays -inf (scale > 0)
      const float mx = (m == -INFINITY) ? mx_t : ((mx_t - m > 8.f) ? mx_t : m);
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = (m == -INFINITY || mx == m) ? 1.f : xb_ex2(m - m_use);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < BKV; ++i) {
        sc[i] = xb_ex2(fmaf(sc[i], p.scale_log2, -m_use));
        sum += sc[i];
      }
      l = l * alpha + sum;
      m = mx;

      if (j > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (j - 1) & 1, abort_flag, p.status, XB_K_ATTN_FWD, 310))) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t t[32];
            tmem_ld_32x32(tmem_base + lane_addr + O_COL + c * 32, t);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
            tmem_st_32x32(tmem_base + lane_addr + O_COL + c * 32, t);
          }
          tc_wait_st();
        }
      }
      // P (bf16) -> shared memory, 128B-swizzled K-major: 16-byte slot index XOR (row & 7)
#pragma unroll
      for (int c16 = 0; c16 < BKV / 8; ++c16) {
        uint4 v;
        v.x = pack_bf16x2(sc[c16 * 8 + 0], sc[c16 * 8 + 1]);
        v.y = pack_bf16x2(sc[c16 * 8 + 2], sc[c16 * 8 + 3]);
        v.z = pack_bf16x2(sc[c16 * 8 + 4], sc[c16 * 8 + 5]);
        v.w = pack_bf16x2(sc[c16 * 8 + 6], sc[c16 * 8 + 7]);
        const int half = c16 >> 3, slot = (c16 & 7) ^ (r & 7);
        *reinterpret_cast<uint4*>(sp + half * CHUNK_BYTES + r * 128 + slot * 16) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_full);
    }
    if (ok && n_kv > 0) {
      ok = mbar_wait(&bars->pv_done, (n_kv - 1) & 1, abort_flag, p.status, XB_K_ATTN_FWD, 320);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const bool valid = row_pos < seq_len;
      if (p.sinks != nullptr) {
        // the sink logit joins the denominator (and the LSE) and contributes no value
        const float sk = __ldg(p.sinks + head) * 1.4426950408889634f;
        if (m == -INFINITY) { m = sk; l = 1.f; }
        else l += xb_ex2(sk - m);
      }
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow =
          p.out + (size_t)(seq_start + row_pos) * p.ldo + (size_t)head * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t t[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tmem_base + lane_addr + O_COL + c * 32, t);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0;
        }
        if (valid) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t[v4 * 8 + 0]) * inv, __uint_as_float(t[v4 * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(t[v4 * 8 + 2]) * inv, __uint_as_float(t[v4 * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(t[v4 * 8 + 4]) * inv, __uint_as_float(t[v4 * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(t[v4 * 8 + 6]) * inv, __uint_as_float(t[v4 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = o;
          }
        }
      }
      if (valid) {
        // natural-log LSE of the scaled scores
        const float lse = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        p.lse[(size_t)head * p.T + seq_start + row_pos] = lse;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace xb_attn_fwd_ns

// q: [T, Hq, 128] with token stride ldq;  k, v: [T, Hkv, 128] with token strides ldk, ldv;
// out: [T, Hq, 128] token stride ldo;  lse: [Hq, T] fp32;  cu_seqlens: int32 [num_seqs + 1] on the
// device.  All strides in elements, multiples of 8; base pointers 16-byte aligned.
XB_API int xb_attn_fwd_ex(const void* q, const void* k, const void* v, void* out, float* lse,
                          const int* cu_seqlens, const int* k_starts, long long ldq, long long ldk,
                          long long ldv, long long ldo, int num_seqs, int T, int Tk, int Hq, int Hkv,
                          int D, int causal, float scale, int max_tiles, void* stream);
XB_API int xb_attn_fwd_sink(const void* q, const void* k, const void* v, void* out, float* lse,
                            const int* cu_seqlens, const int* k_starts, const float* sinks, long long ldq,
                            long long ldk, long long ldv, long long ldo, int num_seqs, int T, int Tk, int Hq,
                            int Hkv, int D, int causal, float scale, int max_tiles, void* stream);

XB_API int xb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                       const int* cu_seqlens, long long ldq, long long ldk, long long ldv,
                       long long ldo, int num_seqs, int T, int Hq, int Hkv, int D, int causal,
                       float scale, int max_tiles, void* stream) {
  return xb_attn_fwd_ex(q, k, v, out, lse, cu_seqlens, nullptr, ldq, ldk, ldv, ldo, num_seqs, T, T,
                        Hq, Hkv, D, causal, scale, max_tiles, stream);
}

// As xb_attn_fwd, but the K/V rows of sequence b start at k_starts[b] (device int32 array, may be
// null) in K/V tensors of Tk rows.  Query and key lengths of a sequence are equal.  This is the
// block-pair form used by ring attention: any query block against any key block.
XB_API int xb_attn_fwd_ex(const void* q, const void* k, const void* v, void* out, float* lse,
                          const int* cu_seqlens, const int* k_starts, long long ldq, long long ldk,
                          long long ldv, long long ldo, int num_seqs, int T, int Tk, int Hq, int Hkv,
                          int D, int causal, float scale, int max_tiles, void* stream) {
  return xb_attn_fwd_sink(q, k, v, out, lse, cu_seqlens, k_starts, nullptr, ldq, ldk, ldv, ldo, num_seqs, T,
                          Tk, Hq, Hkv, D, causal, scale, max_tiles, stream);
}

// As xb_attn_fwd_ex with two more features.  ``causal``: bit 0 is the causal flag, the bits above it
// hold a sliding-window length (0: none): a query sees the keys with q_pos - k_pos < window.
// ``sinks``: optional fp32 [Hq] device array of per-head sink logits.
XB_API int xb_attn_fwd_sink(const void* q, const void* k, const void* v, void* out, float* lse,
                            const int* cu_seqlens, const int* k_starts, const float* sinks, long long ldq,
                            long long ldk, long long ldv, long long ldo, int num_seqs, int T, int Tk, int Hq,
                            int Hkv, int D, int causal, float scale, int max_tiles, void* stream) {
  using namespace xb_attn_fwd_ns;
  if (D != 128) return -1;
  if (T <= 0 || num_seqs <= 0) return 0;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || Hq % Hkv) return -1;
  CUtensorMap tq, tk, tv;
  if (xb_make_tmap_3d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, Hq, D, ldq, D, BQ, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (xb_make_tmap_3d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, Hkv, D, ldk, D, BKV, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (xb_make_tmap_3d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, Hkv, D, ldv, D, BKV, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -4;
  Params p;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.lse = lse; p.cu_seqlens = cu_seqlens; p.k_starts = k_starts;
  p.num_seqs = num_seqs; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal & 1;
  p.window = causal >> 1; p.sinks = sinks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = xb_status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  // upper bound on the number of query tiles: every sequence adds at most one partial tile
  const int tiles = max_tiles > 0 ? max_tiles : (T + BQ - 1) / BQ + num_seqs;
  dim3 grid(tiles, Hq);
  attn_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
