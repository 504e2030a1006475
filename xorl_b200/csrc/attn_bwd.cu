// Flash-attention backward for sm_100a (packed varlen, causal or full, GQA, head_dim 128).
//
// One CTA owns a 64-row key/value tile of one KV head and walks every query tile (128 rows) of
// every query head of that group that can see it.  Per step, five tcgen05 GEMMs:
//     S   = Q K^T            (128 x 64,  K = d)        dP  = dO V^T        (128 x 64,  K = d)
//     dV^T += dO^T P         (128 x 64,  K = q rows)   dK^T += Q^T dS      (128 x 64,  K = q rows)
//     dQ  = dS K             (128 x 128, K = kv rows)
// dV^T / dK^T stay in TMEM for the whole CTA lifetime (d on the lanes), so the M = 128 MMA shape is
// used throughout; transposed operands are expressed with MN-major descriptors over the very same
// TMA-written tiles, nothing is transposed in memory.  dQ tiles are added to an fp32 buffer with
// vector reductions; dK is written fp32 and dV bf16 when the CTA finishes.
//   warp 0 : TMA producer (K,V once; Q,dO two-stage ring)    warp 1 : MMA issuer
//   warps 2..5 : one query row per thread (P, dS, dQ read-out)
// Replaces the FlashAttention backward of the reference's wheels
// (src/xorl/models/layers/attention/backend/flash_attention.py:382-531).
#include "common.cuh"

namespace xb_attn_bwd_ns {

constexpr int D = 128;
constexpr int BQ = 128;
constexpr int BKV = 64;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_DP = 64, COL_DQ = 128, COL_DV = 256, COL_DK = 320;
constexpr int KV_TILE_BYTES = BKV * D * 2;    // 16 KB : two d-chunks of [64 rows][128 B]
constexpr int KV_CHUNK_BYTES = BKV * 128;     // 8 KB
constexpr int Q_TILE_BYTES = BQ * D * 2;      // 32 KB : two d-chunks of [128 rows][128 B]
constexpr int Q_CHUNK_BYTES = BQ * 128;       // 16 KB
constexpr int PS_BYTES = BQ * BKV * 2;        // 16 KB : [128 q rows][64 kv = 128 B]
constexpr int SMEM_K = 0;
constexpr int SMEM_V = SMEM_K + KV_TILE_BYTES;
constexpr int SMEM_Q = SMEM_V + KV_TILE_BYTES;        // 2 stages
constexpr int SMEM_DO = SMEM_Q + 2 * Q_TILE_BYTES;    // 2 stages
constexpr int SMEM_P = SMEM_DO + 2 * Q_TILE_BYTES;
constexpr int SMEM_DS = SMEM_P + PS_BYTES;
constexpr int SMEM_BAR = SMEM_DS + PS_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR + 256 + 1024;

struct Params {
  const float* lse;     // [Hq, T]
  const float* delta;   // [Hq, T]
  float* dq_accum;      // [T, Hq, D] fp32, zeroed by the caller
  float* dk;            // [T, Hkv, D] fp32
  __nv_bfloat16* dv;    // [T, Hkv, D] with token stride lddv
  long long lddv;
  const int* cu_seqlens;
  const int* k_starts;  // optional first K/V row per sequence
  int num_seqs;
  int T, Hq, Hkv;
  int causal;
  float scale, scale_log2;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t kv_full;
  uint64_t q_full[2], q_empty[2];
  uint64_t sdp_full, sdp_empty;   // S and dP ready in TMEM / read out by the row threads
  uint64_t pds_full;              // P and dS written to shared memory
  uint64_t dq_full, dq_empty;     // dQ tile ready in TMEM / read out
  uint64_t all_done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
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
  const int per_head = n_q_tiles - qt0;
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
    }
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->sdp_empty, 128);
    mbar_init(&bars->pds_full, 128);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_empty, 128);
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
        if (!mbar_wait(&bars->q_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 100 + s)) {
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
      constexpr uint32_t idesc_q = xb_idesc(1, 1, BQ, D, 0, 1);     // dS K (K tile MN-major)
      constexpr uint64_t kmaj = xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t mn_q = xb_smem_desc_base_sw128(Q_CHUNK_BYTES, 1024);    // Q/dO as A^T
      constexpr uint64_t mn_ps = xb_smem_desc_base_sw128(PS_BYTES, 1024);        // P/dS as B (1 chunk)
      constexpr uint64_t mn_kv = xb_smem_desc_base_sw128(KV_CHUNK_BYTES, 1024);  // K as B of dQ
      const uint32_t sk = xb_smem_u32(smem + SMEM_K), sv = xb_smem_u32(smem + SMEM_V);
      const uint32_t spp = xb_smem_u32(smem + SMEM_P), sds = xb_smem_u32(smem + SMEM_DS);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, p.status, XB_K_ATTN_BWD, 200);
      auto issue_sdp = [&](int t) -> bool {
        const int s = t & 1;
        if (!mbar_wait(&bars->q_full[s], (t >> 1) & 1, abort_flag, p.status, XB_K_ATTN_BWD,
                       210 + s))
          return false;
        if (!mbar_wait(&bars->sdp_empty, (t & 1) ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 220))
          return false;
        tc_fence_after();
        const uint32_t sq = xb_smem_u32(smem + SMEM_Q + s * Q_TILE_BYTES);
        const uint32_t sdo = xb_smem_u32(smem + SMEM_DO + s * Q_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * Q_CHUNK_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + COL_S, xb_smem_desc(kmaj, sq + a_off),
                        xb_smem_desc(kmaj, sk + b_off), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * Q_CHUNK_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + COL_DP, xb_smem_desc(kmaj, sdo + a_off),
                        xb_smem_desc(kmaj, sv + b_off), idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->sdp_full);
        return true;
      };
      if (ok && n_steps > 0) ok = issue_sdp(0);
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t & 1;
        // P/dS of step t in shared memory (this also implies S/dP of step t were read out)
        if (!mbar_wait(&bars->pds_full, t & 1, abort_flag, p.status, XB_K_ATTN_BWD, 230)) {
          ok = false;
          break;
        }
        // dQ accumulator of the previous step must have been read out
        if (!mbar_wait(&bars->dq_empty, (t & 1) ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 240)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sq = xb_smem_u32(smem + SMEM_Q + s * Q_TILE_BYTES);
        const uint32_t sdo = xb_smem_u32(smem + SMEM_DO + s * Q_TILE_BYTES);
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
        // dQ = dS K   (reduction over the 64 kv rows)
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          tc_mma_f16_ss(tmem_base + COL_DQ, xb_smem_desc(kmaj, sds + k * 32),
                        xb_smem_desc(mn_kv, sk + k * 2048), idesc_q, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->q_empty[s]);
        tc_commit(&bars->dq_full);
        // S/dP of the next step can be computed while the row threads drain dQ
        if (t + 1 < n_steps) {
          if (!issue_sdp(t + 1)) { ok = false; break; }
        }
      }
      if (ok) tc_commit(&bars->all_done);
    }
    __syncwarp();
  } else {
    // ------------------------------- row threads --------------------------------------
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    for (int t = 0; t < n_steps && ok; ++t) {
      const int head = kv_head * G + t / per_head;
      const int qt = qt0 + t % per_head;
      const int q_pos = qt * BQ + r;
      const bool row_valid = q_pos < seq_len;
      const size_t tok = (size_t)seq_start + q_pos;
      float lse = 0.f, delta = 0.f;
      if (row_valid) {
        lse = p.lse[(size_t)head * p.T + tok] * LOG2E;
        delta = p.delta[(size_t)head * p.T + tok];
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->sdp_full, t & 1, abort_flag, p.status, XB_K_ATTN_BWD, 300))) {
        ok = false;
        break;
      }
      tc_fence_after();
      float pv[BKV], ds[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tmem_base + lane_addr + COL_S + c * 32, a);
        tmem_ld_32x32(tmem_base + lane_addr + COL_DP + c * 32, b);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          pv[c * 32 + i] = __uint_as_float(a[i]);
          ds[c * 32 + i] = __uint_as_float(b[i]);
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->sdp_empty);
      const int lim = p.causal ? min(seq_len - 1, q_pos) : seq_len - 1;  // last visible kv position
#pragma unroll
      for (int i = 0; i < BKV; ++i) {
        const bool vis = row_valid && (kv0 + i <= lim);
        const float pe = vis ? exp2f(pv[i] * p.scale_log2 - lse) : 0.f;
        pv[i] = pe;
        ds[i] = pe * (ds[i] - delta) * p.scale;
      }
      // previous step's MMAs (which read P/dS from shared memory) are done once dq_full fired
      if (t > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->dq_full, (t - 1) & 1, abort_flag, p.status, XB_K_ATTN_BWD, 310))) {
          ok = false;
          break;
        }
        tc_fence_after();
        // drain dQ of step t-1 into the fp32 accumulation buffer
        const int head_p = kv_head * G + (t - 1) / per_head;
        const int qpos_p = (qt0 + (t - 1) % per_head) * BQ + r;
        float* dst = p.dq_accum + ((size_t)(seq_start + qpos_p) * p.Hq + head_p) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t a[32];
          tmem_ld_32x32(tmem_base + lane_addr + COL_DQ + c * 32, a);
          tc_wait_ld();
          if (qpos_p < seq_len) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 32 + i),
                           "f"(__uint_as_float(a[i])), "f"(__uint_as_float(a[i + 1])),
                           "f"(__uint_as_float(a[i + 2])), "f"(__uint_as_float(a[i + 3]))
                           : "memory");
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&bars->dq_empty);
      }
      // P and dS rows (bf16) -> shared memory, [128 rows][128 B] with the 128B swizzle
      uint8_t* sp = smem + SMEM_P + r * 128;
      uint8_t* sd = smem + SMEM_DS + r * 128;
#pragma unroll
      for (int c16 = 0; c16 < BKV / 8; ++c16) {
        uint4 v, w;
        v.x = pack_bf16x2(pv[c16 * 8 + 0], pv[c16 * 8 + 1]);
        v.y = pack_bf16x2(pv[c16 * 8 + 2], pv[c16 * 8 + 3]);
        v.z = pack_bf16x2(pv[c16 * 8 + 4], pv[c16 * 8 + 5]);
        v.w = pack_bf16x2(pv[c16 * 8 + 6], pv[c16 * 8 + 7]);
        w.x = pack_bf16x2(ds[c16 * 8 + 0], ds[c16 * 8 + 1]);
        w.y = pack_bf16x2(ds[c16 * 8 + 2], ds[c16 * 8 + 3]);
        w.z = pack_bf16x2(ds[c16 * 8 + 4], ds[c16 * 8 + 5]);
        w.w = pack_bf16x2(ds[c16 * 8 + 6], ds[c16 * 8 + 7]);
        const int slot = c16 ^ (r & 7);
        *reinterpret_cast<uint4*>(sp + slot * 16) = v;
        *reinterpret_cast<uint4*>(sd + slot * 16) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->pds_full);
    }
    if (ok && n_steps > 0) {
      // last dQ tile
      const int t = n_steps - 1;
      if (__all_sync(0xffffffffu, mbar_wait(&bars->dq_full, t & 1, abort_flag, p.status, XB_K_ATTN_BWD, 320))) {
        tc_fence_after();
        const int head_p = kv_head * G + t / per_head;
        const int qpos_p = (qt0 + t % per_head) * BQ + r;
        float* dst = p.dq_accum + ((size_t)(seq_start + qpos_p) * p.Hq + head_p) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t a[32];
          tmem_ld_32x32(tmem_base + lane_addr + COL_DQ + c * 32, a);
          tc_wait_ld();
          if (qpos_p < seq_len) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 32 + i),
                           "f"(__uint_as_float(a[i])), "f"(__uint_as_float(a[i + 1])),
                           "f"(__uint_as_float(a[i + 2])), "f"(__uint_as_float(a[i + 3]))
                           : "memory");
            }
          }
        }
      } else {
        ok = false;
      }
    }
    if (ok && n_steps > 0) ok = mbar_wait(&bars->all_done, 0, abort_flag, p.status, XB_K_ATTN_BWD, 330);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      // dV^T / dK^T: this thread holds feature d = r for the 64 kv rows of the tile.  For a fixed
      // kv row the 32 lanes of a warp write 32 consecutive features.
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t a[32], b[32];
        if (n_steps > 0) {
          tmem_ld_32x32(tmem_base + lane_addr + COL_DV + c * 32, a);
          tmem_ld_32x32(tmem_base + lane_addr + COL_DK + c * 32, b);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0; b[i] = 0; }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv_pos = kv0 + c * 32 + i;
          if (kv_pos < seq_len) {
            const size_t tok = (size_t)k_start + kv_pos;
            p.dv[tok * p.lddv + (size_t)kv_head * D + r] = __float2bfloat16(__uint_as_float(a[i]));
            p.dk[(tok * p.Hkv + kv_head) * D + r] = __uint_as_float(b[i]);
          }
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

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]; one warp per (t, h)
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo,
                  const __nv_bfloat16* __restrict__ dout, long long lddo, float* __restrict__ delta,
                  int T, int Hq) {
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (wid >= (long long)T * Hq) return;
  const int t = (int)(wid / Hq), h = (int)(wid % Hq);
  const int lane = threadIdx.x & 31;
  const uint2 a = reinterpret_cast<const uint2*>(o + (size_t)t * ldo + (size_t)h * D)[lane];
  const uint2 b = reinterpret_cast<const uint2*>(dout + (size_t)t * lddo + (size_t)h * D)[lane];
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y);
  const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) delta[(size_t)h * T + t] = s;
}

static int g_split = 1;

}  // namespace xb_attn_bwd_ns

// 1 (default): dK / dV from the key-stationary kernel in attn_bwd_dkv.cu and dQ from the
// query-stationary kernel in attn_bwd_dq.cu (no atomics); 0: the single kernel of this file, which
// adds dQ partials to global memory with fp32 vector reductions.  Returns the previous setting.
XB_API int xb_attn_bwd_set_split(int split) {
  const int prev = xb_attn_bwd_ns::g_split;
  xb_attn_bwd_ns::g_split = split ? 1 : 0;
  return prev;
}

XB_API int xb_attn_bwd_dq(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                          const float* delta, float* dq, const int* cu_seqlens, const int* k_starts,
                          long long ldq, long long ldk, long long ldv, long long lddo, int num_seqs, int T,
                          int Tk, int Hq, int Hkv, int causal, float scale, int accumulate, int max_q_tiles,
                          void* stream);
XB_API int xb_attn_bwd_dkv(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                           const float* delta, float* dk, void* dv, const int* cu_seqlens, const int* k_starts,
                           long long ldq, long long ldk, long long ldv, long long lddo, long long lddv,
                           int num_seqs, int T, int Tk, int Hq, int Hkv, int causal, float scale, int max_tiles,
                           void* stream);

// Inputs as in xb_attn_fwd plus out / dout [T, Hq, 128] and lse [Hq, T].
// Scratch: delta fp32 [Hq * T]; dq_accum fp32 [T * Hq * 128] (this call zeroes it).
// Outputs: dq_accum (fp32 dQ), dk fp32 [T, Hkv, 128], dv bf16 [T, Hkv, 128] (token stride lddv).
XB_API int xb_attn_bwd_ex(const void* q, const void* k, const void* v, const void* out,
                          const void* dout, const float* lse, float* delta, float* dq_accum,
                          float* dk, void* dv, const int* cu_seqlens, const int* k_starts,
                          long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
                          long long lddv, int num_seqs, int T, int Tk, int Hq, int Hkv, int D,
                          int causal, float scale, int flags, int max_tiles, void* stream);

XB_API int xb_attn_bwd(const void* q, const void* k, const void* v, const void* out,
                       const void* dout, const float* lse, float* delta, float* dq_accum, float* dk,
                       void* dv, const int* cu_seqlens, long long ldq, long long ldk, long long ldv,
                       long long ldo, long long lddo, long long lddv, int num_seqs, int T, int Hq,
                       int Hkv, int D, int causal, float scale, int max_tiles, void* stream) {
  return xb_attn_bwd_ex(q, k, v, out, dout, lse, delta, dq_accum, dk, dv, cu_seqlens, nullptr, ldq,
                        ldk, ldv, ldo, lddo, lddv, num_seqs, T, T, Hq, Hkv, D, causal, scale, 0,
                        max_tiles, stream);
}

// Block-pair form (see xb_attn_fwd_ex).  flags bit 0: dq_accum already holds partial sums, do not
// clear it; bit 1: delta is already computed, do not recompute it.  dk / dv have Tk rows and
// are written (not accumulated) for the K/V rows this call covers.
XB_API int xb_attn_bwd_ex(const void* q, const void* k, const void* v, const void* out,
                          const void* dout, const float* lse, float* delta, float* dq_accum,
                          float* dk, void* dv, const int* cu_seqlens, const int* k_starts,
                          long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
                          long long lddv, int num_seqs, int T, int Tk, int Hq, int Hkv, int D,
                          int causal, float scale, int flags, int max_tiles, void* stream) {
  using namespace xb_attn_bwd_ns;
  if (D != 128) return -1;
  if (T <= 0 || num_seqs <= 0) return 0;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || (lddo % 8) || Hq % Hkv) return -1;
  cudaStream_t st = (cudaStream_t)stream;
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
  if (xb_make_tmap_3d(&tdo, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, Hq, D, lddo, D, BQ, 1,
                      64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -5;
  if (!(flags & 1)) {
    if (cudaMemsetAsync(dq_accum, 0, (size_t)T * Hq * D * sizeof(float), st) != cudaSuccess)
      return -6;
  }
  if (!(flags & 2)) {
    const long long rows = (long long)T * Hq;
    attn_delta_kernel<<<(int)((rows + 7) / 8), 256, 0, st>>>(
        (const __nv_bfloat16*)out, ldo, (const __nv_bfloat16*)dout, lddo, delta, T, Hq);
  }
  if (g_split || (causal >> 1)) {     // sliding windows are implemented by the split kernels only
    // dq_accum is written with plain stores (added to when flags bit 0 is set); rows outside every
    // sequence keep the zeros of the memset above
    int rc = xb_attn_bwd_dkv(q, k, v, dout, lse, delta, dk, dv, cu_seqlens, k_starts, ldq, ldk, ldv, lddo, lddv,
                             num_seqs, T, Tk, Hq, Hkv, causal, scale, max_tiles, stream);
    if (rc) return rc;
    const int q_tiles = max_tiles > 0 ? (max_tiles + 1) / 2 + num_seqs : 0;
    return xb_attn_bwd_dq(q, k, v, dout, lse, delta, dq_accum, cu_seqlens, k_starts, ldq, ldk, ldv, lddo,
                          num_seqs, T, Tk, Hq, Hkv, causal, scale, (flags & 1) ? 1 : 0, q_tiles, stream);
  }
  Params p;
  p.lse = lse; p.delta = delta; p.dq_accum = dq_accum; p.dk = dk;
  p.dv = (__nv_bfloat16*)dv; p.lddv = lddv; p.cu_seqlens = cu_seqlens; p.k_starts = k_starts; p.num_seqs = num_seqs;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = xb_status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  const int tiles = max_tiles > 0 ? max_tiles : (T + BKV - 1) / BKV + num_seqs;
  dim3 grid(tiles, Hkv);
  attn_bwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
