// dK / dV of flash-attention backward (sm_100a; packed varlen, causal or full, GQA, head_dim 128).
//
// One CTA owns a 64-row key/value tile of one KV head and walks every query tile (128 rows) of
// every query head of the group that can see it.  Per step four tcgen05 GEMM groups:
//     S   = Q K^T            (128 x 64,  K = d)        dP  = dO V^T        (128 x 64,  K = d)
//     dV^T += dO^T P         (128 x 64,  K = q rows)   dK^T += Q^T dS      (128 x 64,  K = q rows)
// dV^T / dK^T stay in TMEM for the CTA's lifetime (d on the lanes); transposed operands are MN-major
// descriptors over the TMA-written tiles.  dQ is produced by attn_bwd_dq.cu.
//
// The step is software-pipelined over two buffers of everything that crosses between the tensor
// core and the row threads: S / dP in TMEM and P / dS in shared memory.  The MMA thread issues
// S, dP of step t+1 before it waits for P, dS of step t, so the tensor core multiplies while the
// row threads exponentiate, and the dV / dK MMAs of step t overlap the row work of step t+1.
// Eight row warps (two threads per query row, 32 key columns each) put two warps on every
// scheduler, and lse / delta of the next step are fetched one step ahead, so neither arithmetic nor
// global-load latency is exposed.
//   warp 0 : TMA producer (K,V once; Q,dO two-stage ring)    warp 1 : MMA issuer    warps 2..9 : rows
#include "common.cuh"

namespace xb_attn_dkv_ns {

constexpr int D = 128;
constexpr int BQ = 128;
constexpr int BKV = 64;
constexpr int NUM_THREADS = 320;
constexpr int ROW_THREADS = 256;
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0;        // + 128 * buf
constexpr int COL_DP = 64;      // + 128 * buf
constexpr int COL_DV = 256, COL_DK = 320;
constexpr int KV_TILE_BYTES = BKV * D * 2;    // 16 KB : two d-chunks of [64 rows][128 B]
constexpr int KV_CHUNK_BYTES = BKV * 128;
constexpr int Q_TILE_BYTES = BQ * D * 2;      // 32 KB : two d-chunks of [128 rows][128 B]
constexpr int Q_CHUNK_BYTES = BQ * 128;
constexpr int PS_BYTES = BQ * BKV * 2;        // 16 KB : [128 q rows][64 kv = 128 B]
constexpr int SMEM_K = 0;
constexpr int SMEM_V = SMEM_K + KV_TILE_BYTES;
constexpr int SMEM_Q = SMEM_V + KV_TILE_BYTES;        // 2 stages
constexpr int SMEM_DO = SMEM_Q + 2 * Q_TILE_BYTES;    // 2 stages
constexpr int SMEM_P = SMEM_DO + 2 * Q_TILE_BYTES;    // 2 buffers
constexpr int SMEM_DS = SMEM_P + 2 * PS_BYTES;        // 2 buffers
constexpr int SMEM_BAR = SMEM_DS + 2 * PS_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR + 256 + 1024;

struct Params {
  const float* lse;     // [Hq, T]
  const float* delta;   // [Hq, T]
  float* dk;            // [Tk, Hkv, D] fp32
  __nv_bfloat16* dv;    // [Tk, Hkv, D] with token stride lddv
  long long lddv;
  const int* cu_seqlens;
  const int* k_starts;
  int num_seqs;
  int T, Hq, Hkv;
  int causal;
  int window;
  float scale, scale_log2;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t kv_full;
  uint64_t q_full[2], q_empty[2];
  uint64_t sdp_full[2], sdp_empty[2];   // S and dP ready in TMEM / read out by the row threads
  uint64_t pds_full[2], pds_free[2];    // P and dS written to shared memory / consumed by the MMAs
  uint64_t all_done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const Params p) {
  const int tile_id = blockIdx.x;
  int seq = -1, kt = 0, seq_start = 0, seq_len = 0;
  {
    int acc = 0;
    for (int b = 0; b < p.num_seqs; ++b) {
      const int s0 = p.cu_seqlens[b], s1 = p.cu_seqlens[b + 1];
      const int nt = (s1 - s0 + BKV - 1) / BKV;
      if (tile_id < acc + nt) {
        seq = b; kt = tile_id - acc; seq_start = s0; seq_len = s1 - s0;
        break;
      }
      acc += nt;
    }
  }
  if (seq < 0) return;
  const int k_start = p.k_starts ? p.k_starts[seq] : seq_start;
  if (k_start < 0) return;  // this query block takes no part in the call
  const int kv_head = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int kv0 = kt * BKV;                         // position inside the sequence
  const int n_q_tiles = (seq_len + BQ - 1) / BQ;
  const int qt0 = p.causal ? kv0 / BQ : 0;           // first query tile that sees this KV tile
  // last query that sees key k under a window is k + window - 1
  const int qt_end = p.window > 0 ? min(n_q_tiles, (kv0 + BKV + p.window - 2) / BQ + 1) : n_q_tiles;
  const int per_head = max(0, qt_end - qt0);
  const int n_steps = per_head * G;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + SMEM_BAR);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 1);
      mbar_init(&bars->sdp_full[s], 1);
      mbar_init(&bars->sdp_empty[s], ROW_THREADS);
      mbar_init(&bars->pds_full[s], ROW_THREADS);
      mbar_init(&bars->pds_free[s], 1);
    }
    mbar_init(&bars->all_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
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
      const int tok = k_start + kv0;
      mbar_expect_tx(&bars->kv_full, 2 * KV_TILE_BYTES);
      tma_load_3d(smem + SMEM_K, &tmap_k, &bars->kv_full, 0, kv_head, tok);
      tma_load_3d(smem + SMEM_K + KV_CHUNK_BYTES, &tmap_k, &bars->kv_full, 64, kv_head, tok);
      tma_load_3d(smem + SMEM_V, &tmap_v, &bars->kv_full, 0, kv_head, tok);
      tma_load_3d(smem + SMEM_V + KV_CHUNK_BYTES, &tmap_v, &bars->kv_full, 64, kv_head, tok);
      bool ok = true;
      int issued = 0;
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        const int head = kv_head * G + t / per_head;
        const int qtok = seq_start + (qt0 + t % per_head) * BQ;
        if (!mbar_wait(&bars->q_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 800 + s)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&bars->q_full[s], 2 * Q_TILE_BYTES);
        uint8_t* sq = smem + SMEM_Q + s * Q_TILE_BYTES;
        uint8_t* sdo = smem + SMEM_DO + s * Q_TILE_BYTES;
        tma_load_3d(sq, &tmap_q, &bars->q_full[s], 0, head, qtok);
        tma_load_3d(sq + Q_CHUNK_BYTES, &tmap_q, &bars->q_full[s], 64, head, qtok);
        tma_load_3d(sdo, &tmap_do, &bars->q_full[s], 0, head, qtok);
        tma_load_3d(sdo + Q_CHUNK_BYTES, &tmap_do, &bars->q_full[s], 64, head, qtok);
        issued = t + 1;
      }
      if (!ok) {
        const uint64_t t0 = xb_globaltimer();
        while (!mbar_try_wait(&bars->kv_full, 0) && xb_globaltimer() - t0 < 200000000ull) {}
        for (int t = max(0, issued - 2); t < issued; ++t)
          while (!mbar_try_wait(&bars->q_full[t & 1], (t >> 1) & 1) &&
                 xb_globaltimer() - t0 < 200000000ull) {}
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = xb_idesc(1, 1, BQ, BKV, 0, 0);   // Q K^T, dO V^T
      constexpr uint32_t idesc_t = xb_idesc(1, 1, D, BKV, 1, 1);    // dO^T P, Q^T dS (both MN-major)
      constexpr uint64_t kmaj = xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t mn_q = xb_smem_desc_base_sw128(Q_CHUNK_BYTES, 1024);    // Q/dO as A^T
      constexpr uint64_t mn_ps = xb_smem_desc_base_sw128(PS_BYTES, 1024);        // P/dS as B (1 chunk)
      const uint32_t sk = xb_smem_u32(smem + SMEM_K), sv = xb_smem_u32(smem + SMEM_V);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, p.status, XB_K_ATTN_BWD, 810);
      auto issue_sdp = [&](int t) -> bool {
        const int s = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&bars->q_full[s], ph, abort_flag, p.status, XB_K_ATTN_BWD, 820 + s)) return false;
        if (!mbar_wait(&bars->sdp_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 830 + s)) return false;
        tc_fence_after();
        const uint32_t sq = xb_smem_u32(smem + SMEM_Q + s * Q_TILE_BYTES);
        const uint32_t sdo = xb_smem_u32(smem + SMEM_DO + s * Q_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * Q_CHUNK_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + COL_S + 128 * s, xb_smem_desc(kmaj, sq + a_off),
                        xb_smem_desc(kmaj, sk + b_off), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * Q_CHUNK_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + COL_DP + 128 * s, xb_smem_desc(kmaj, sdo + a_off),
                        xb_smem_desc(kmaj, sv + b_off), idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->sdp_full[s]);
        return true;
      };
      if (ok && n_steps > 0) ok = issue_sdp(0);
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t & 1;
        if (t + 1 < n_steps) {
          if (!issue_sdp(t + 1)) { ok = false; break; }
        }
        if (!mbar_wait(&bars->pds_full[s], (t >> 1) & 1, abort_flag, p.status, XB_K_ATTN_BWD, 840 + s)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sq = xb_smem_u32(smem + SMEM_Q + s * Q_TILE_BYTES);
        const uint32_t sdo = xb_smem_u32(smem + SMEM_DO + s * Q_TILE_BYTES);
        const uint32_t spp = xb_smem_u32(smem + SMEM_P + s * PS_BYTES);
        const uint32_t sds = xb_smem_u32(smem + SMEM_DS + s * PS_BYTES);
        // dV^T += dO^T P ; dK^T += Q^T dS   (reduction over the 128 query rows, 16 per MMA)
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          tc_mma_f16_ss(tmem_base + COL_DV, xb_smem_desc(mn_q, sdo + k * 2048),
                        xb_smem_desc(mn_ps, spp + k * 2048), idesc_t, (t > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          tc_mma_f16_ss(tmem_base + COL_DK, xb_smem_desc(mn_q, sq + k * 2048),
                        xb_smem_desc(mn_ps, sds + k * 2048), idesc_t, (t > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&bars->q_empty[s]);
        tc_commit(&bars->pds_free[s]);
      }
      if (ok) tc_commit(&bars->all_done);
    }
    __syncwarp();
  } else {
    // ------------------------------- row threads --------------------------------------
    const int q4 = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;        // which 32 of the 64 key columns
    const int r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    // lse / delta of the step about to run, fetched one step ahead
    float lse_n = 0.f, delta_n = 0.f;
    auto fetch = [&](int t) {
      lse_n = 0.f; delta_n = 0.f;
      if (t < n_steps) {
        const int head = kv_head * G + t / per_head;
        const int q_pos = (qt0 + t % per_head) * BQ + r;
        if (q_pos < seq_len) {
          const size_t tok = (size_t)seq_start + q_pos;
          lse_n = __ldg(p.lse + (size_t)head * p.T + tok) * LOG2E;
          delta_n = __ldg(p.delta + (size_t)head * p.T + tok);
        }
      }
    };
    fetch(0);
    for (int t = 0; t < n_steps && ok; ++t) {
      const int s = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      const int q_pos = (qt0 + t % per_head) * BQ + r;
      const bool row_valid = q_pos < seq_len;
      const float lse = lse_n, delta = delta_n;
      fetch(t + 1);
      // votes keep the warp together: the tcgen05.ld below is warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->sdp_full[s], ph, abort_flag, p.status, XB_K_ATTN_BWD, 900 + s))) {
        ok = false;
        break;
      }
      tc_fence_after();
      float pv[32], ds[32];
      {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tmem_base + lane_addr + COL_S + 128 * s + half * 32, a);
        tmem_ld_32x32(tmem_base + lane_addr + COL_DP + 128 * s + half * 32, b);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&bars->sdp_empty[s]);
        // dS here is P o (dP - delta); the softmax scale is applied once, to dK, at the end.
        // Tiles entirely below the diagonal and inside the sequence (the common case) need no mask.
        const int q_lo = (qt0 + t % per_head) * BQ;
        const bool no_mask = (q_lo + BQ <= seq_len) && (kv0 + BKV <= seq_len) && (!p.causal || kv0 + BKV - 1 <= q_lo) &&
                             (p.window <= 0 || kv0 >= q_lo + BQ - p.window);
        if (no_mask) {                               // CTA-uniform
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pe = xb_ex2(fmaf(__uint_as_float(a[i]), p.scale_log2, -lse));
            pv[i] = pe;
            ds[i] = pe * (__uint_as_float(b[i]) - delta);
          }
        } else {
          const int lim = p.causal ? min(seq_len - 1, q_pos) : seq_len - 1;  // last visible kv position
          const int nvis = row_valid ? (lim - (kv0 + half * 32) + 1) : 0;     // visible columns of this thread
          const int nlo = p.window > 0 ? (q_pos - p.window + 1) - (kv0 + half * 32) : 0;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pe = (i < nvis && i >= nlo) ? xb_ex2(fmaf(__uint_as_float(a[i]), p.scale_log2, -lse)) : 0.f;
            pv[i] = pe;
            ds[i] = pe * (__uint_as_float(b[i]) - delta);
          }
        }
      }
      // the dV / dK MMAs of step t-2 read this P / dS buffer: wait until they are done
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->pds_free[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 910 + s))) {
        ok = false;
        break;
      }
      // P and dS rows (bf16) -> shared memory, [128 rows][128 B] with the 128B swizzle
      uint8_t* sp = smem + SMEM_P + s * PS_BYTES + r * 128;
      uint8_t* sd = smem + SMEM_DS + s * PS_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 v, w;
        v.x = pack_bf16x2(pv[c * 8 + 0], pv[c * 8 + 1]);
        v.y = pack_bf16x2(pv[c * 8 + 2], pv[c * 8 + 3]);
        v.z = pack_bf16x2(pv[c * 8 + 4], pv[c * 8 + 5]);
        v.w = pack_bf16x2(pv[c * 8 + 6], pv[c * 8 + 7]);
        w.x = pack_bf16x2(ds[c * 8 + 0], ds[c * 8 + 1]);
        w.y = pack_bf16x2(ds[c * 8 + 2], ds[c * 8 + 3]);
        w.z = pack_bf16x2(ds[c * 8 + 4], ds[c * 8 + 5]);
        w.w = pack_bf16x2(ds[c * 8 + 6], ds[c * 8 + 7]);
        const int slot = (half * 4 + c) ^ (r & 7);
        *reinterpret_cast<uint4*>(sp + slot * 16) = v;
        *reinterpret_cast<uint4*>(sd + slot * 16) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->pds_full[s]);
    }
    if (ok && n_steps > 0) ok = mbar_wait(&bars->all_done, 0, abort_flag, p.status, XB_K_ATTN_BWD, 920);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      // dV^T / dK^T: this thread holds feature d = r for 32 of the 64 kv rows of the tile.  For a
      // fixed kv row the 32 lanes of a warp write 32 consecutive features.
      uint32_t a[32], b[32];
      if (n_steps > 0) {                          // CTA-uniform
        tmem_ld_32x32(tmem_base + lane_addr + COL_DV + half * 32, a);
        tmem_ld_32x32(tmem_base + lane_addr + COL_DK + half * 32, b);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) { a[i] = 0; b[i] = 0; }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int kv_pos = kv0 + half * 32 + i;
        if (kv_pos < seq_len) {
          const size_t tok = (size_t)k_start + kv_pos;
          p.dv[tok * p.lddv + (size_t)kv_head * D + r] = __float2bfloat16(__uint_as_float(a[i]));
          p.dk[(tok * p.Hkv + kv_head) * D + r] = __uint_as_float(b[i]) * p.scale;
        }
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

}  // namespace xb_attn_dkv_ns

// dk fp32 [Tk, Hkv, 128], dv bf16 [Tk, Hkv, 128] (token stride lddv) for the K/V rows covered by the
// call; lse / delta [Hq, T] must be ready.  max_tiles bounds the number of 64-row key tiles (0 =
// derive from T).
XB_API int xb_attn_bwd_dkv(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                           const float* delta, float* dk, void* dv, const int* cu_seqlens, const int* k_starts,
                           long long ldq, long long ldk, long long ldv, long long lddo, long long lddv,
                           int num_seqs, int T, int Tk, int Hq, int Hkv, int causal, float scale, int max_tiles,
                           void* stream) {
  using namespace xb_attn_dkv_ns;
  if (T <= 0 || num_seqs <= 0) return 0;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || Hq % Hkv) return -1;
  CUtensorMap tq, tk, tv, tdo;
  if (xb_make_tmap_3d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, Hq, D, ldq, D, BQ, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (xb_make_tmap_3d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, Hkv, D, ldk, D, BKV, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (xb_make_tmap_3d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, Hkv, D, ldv, D, BKV, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -4;
  if (xb_make_tmap_3d(&tdo, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, Hq, D, lddo, D, BQ, 1, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -5;
  Params p;
  p.lse = lse; p.delta = delta; p.dk = dk; p.dv = (__nv_bfloat16*)dv; p.lddv = lddv;
  p.cu_seqlens = cu_seqlens; p.k_starts = k_starts; p.num_seqs = num_seqs;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal & 1; p.window = causal >> 1; p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = xb_status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  const int tiles = max_tiles > 0 ? max_tiles : (T + BKV - 1) / BKV + num_seqs;
  dim3 grid(tiles, Hkv);
  attn_bwd_dkv_kernel<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
