// dQ of flash-attention backward without atomics (sm_100a; packed varlen, causal or full, GQA,
// head_dim 128).
//
// One CTA owns a 128-row query tile of one query head and walks the 64-row key/value tiles it can
// see.  Per step three tcgen05 GEMM groups:
//     S  = Q K^T   (128 x 64, K = d)      dP = dO V^T   (128 x 64, K = d)
//     dQ += dS K   (128 x 128, K = 64 kv rows)          dS = P o (dP - delta) * scale
// dQ stays in TMEM for the CTA's lifetime and is written once, with plain stores: every (row,
// head) of dQ belongs to exactly one CTA.  S / dP are double-buffered in TMEM and dS in shared
// memory, so the MMAs of step j+1 run while the row threads turn step j into dS.
// Together with the dK/dV kernel (attn_bwd.cu with its dQ part switched off) this replaces the
// single kernel that added 128 x 128 fp32 dQ partials to global memory with vector reductions at
// every step; the price is a second evaluation of S and dP.
//   warp 0 : TMA producer (Q, dO once; K, V three-stage ring)     warp 1 : MMA issuer
//   warps 2..9 : two threads per query row (32 of the 64 key columns each), two warps per scheduler
//                so that dependent-issue latency of the softmax arithmetic is hidden
#include "common.cuh"

namespace xb_attn_dq_ns {

constexpr int D = 128;
constexpr int BQ = 128;
constexpr int BKV = 64;
constexpr int NS = 3;                          // K/V ring stages
constexpr int NUM_THREADS = 320;
constexpr int ROW_THREADS = 256;
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0;                       // + 128 * buf
constexpr int COL_DP = 64;                     // + 128 * buf
constexpr int COL_DQ = 256;
constexpr int KV_TILE_BYTES = BKV * D * 2;     // 16 KB : two d-chunks of [64 rows][128 B]
constexpr int KV_CHUNK_BYTES = BKV * 128;
constexpr int Q_TILE_BYTES = BQ * D * 2;       // 32 KB : two d-chunks of [128 rows][128 B]
constexpr int Q_CHUNK_BYTES = BQ * 128;
constexpr int DS_BYTES = BQ * BKV * 2;         // 16 KB : [128 q rows][64 kv = 128 B]
constexpr int SMEM_Q = 0;
constexpr int SMEM_DO = SMEM_Q + Q_TILE_BYTES;
constexpr int SMEM_KV = SMEM_DO + Q_TILE_BYTES;                 // NS x (K tile, V tile)
constexpr int SMEM_DS = SMEM_KV + NS * 2 * KV_TILE_BYTES;       // 2 buffers
constexpr int SMEM_BAR = SMEM_DS + 2 * DS_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR + 256 + 1024;

struct Params {
  const float* lse;     // [Hq, T]
  const float* delta;   // [Hq, T]
  float* dq;            // [T, Hq, D] fp32
  const int* cu_seqlens;
  const int* k_starts;
  int num_seqs;
  int T, Hq, Hkv;
  int causal;
  int window;
  int accumulate;       // dq already holds partial sums of earlier key blocks: add to it
  float scale, scale_log2;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t q_full;
  uint64_t kv_full[NS], kv_empty[NS];
  uint64_t sdp_full[2], sdp_empty[2];
  uint64_t ds_full[2], ds_free[2];
  uint64_t dq_done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const Params p) {
  // tiles are numbered so that, inside a sequence, the last (most expensive under a causal mask)
  // query tile comes first
  const int tile_id = blockIdx.x;
  int seq = -1, qt = 0, seq_start = 0, seq_len = 0;
  {
    int acc = 0;
    for (int b = 0; b < p.num_seqs; ++b) {
      const int s0 = p.cu_seqlens[b], s1 = p.cu_seqlens[b + 1];
      const int nt = (s1 - s0 + BQ - 1) / BQ;
      if (tile_id < acc + nt) {
        seq = b; qt = nt - 1 - (tile_id - acc); seq_start = s0; seq_len = s1 - s0;
        break;
      }
      acc += nt;
    }
  }
  if (seq < 0) return;
  const int k_start = p.k_starts ? p.k_starts[seq] : seq_start;
  if (k_start < 0) return;
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qt * BQ;
  const int n_kv_all = (seq_len + BKV - 1) / BKV;
  const int n_hi = p.causal ? min(n_kv_all, (min(q0 + BQ, seq_len) - 1) / BKV + 1) : n_kv_all;
  const int jt0 = p.window > 0 ? max(0, q0 - p.window + 1) / BKV : 0;   // first key tile inside the window
  const int n_steps = max(0, n_hi - jt0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + SMEM_BAR);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->sdp_full[b], 1);
      mbar_init(&bars->sdp_empty[b], ROW_THREADS);
      mbar_init(&bars->ds_full[b], ROW_THREADS);
      mbar_init(&bars->ds_free[b], 1);
    }
    mbar_init(&bars->dq_done, 1);
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
      const int qtok = seq_start + q0;
      mbar_expect_tx(&bars->q_full, 2 * Q_TILE_BYTES);
      tma_load_3d(smem + SMEM_Q, &tmap_q, &bars->q_full, 0, head, qtok);
      tma_load_3d(smem + SMEM_Q + Q_CHUNK_BYTES, &tmap_q, &bars->q_full, 64, head, qtok);
      tma_load_3d(smem + SMEM_DO, &tmap_do, &bars->q_full, 0, head, qtok);
      tma_load_3d(smem + SMEM_DO + Q_CHUNK_BYTES, &tmap_do, &bars->q_full, 64, head, qtok);
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_steps && ok; ++j) {
        const int s = j % NS;
        const uint32_t ph = (j / NS) & 1;
        if (!mbar_wait(&bars->kv_empty[s], ph ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 500 + s)) {
          ok = false;
          break;
        }
        const int tok = k_start + (jt0 + j) * BKV;
        uint8_t* sk = smem + SMEM_KV + s * 2 * KV_TILE_BYTES;
        uint8_t* sv = sk + KV_TILE_BYTES;
        mbar_expect_tx(&bars->kv_full[s], 2 * KV_TILE_BYTES);
        tma_load_3d(sk, &tmap_k, &bars->kv_full[s], 0, kv_head, tok);
        tma_load_3d(sk + KV_CHUNK_BYTES, &tmap_k, &bars->kv_full[s], 64, kv_head, tok);
        tma_load_3d(sv, &tmap_v, &bars->kv_full[s], 0, kv_head, tok);
        tma_load_3d(sv + KV_CHUNK_BYTES, &tmap_v, &bars->kv_full[s], 64, kv_head, tok);
        issued = j + 1;
      }
      if (!ok) {
        // no bulk copy may still be in flight into shared memory when the CTA exits
        const uint64_t t0 = xb_globaltimer();
        while (!mbar_try_wait(&bars->q_full, 0) && xb_globaltimer() - t0 < 200000000ull) {}
        for (int j = max(0, issued - NS); j < issued; ++j)
          while (!mbar_try_wait(&bars->kv_full[j % NS], (j / NS) & 1) &&
                 xb_globaltimer() - t0 < 200000000ull) {}
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = xb_idesc(1, 1, BQ, BKV, 0, 0);   // Q K^T, dO V^T
      constexpr uint32_t idesc_q = xb_idesc(1, 1, BQ, D, 0, 1);     // dS K (K tile MN-major)
      constexpr uint64_t kmaj = xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t mn_kv = xb_smem_desc_base_sw128(KV_CHUNK_BYTES, 1024);
      const uint32_t sq = xb_smem_u32(smem + SMEM_Q), sdo = xb_smem_u32(smem + SMEM_DO);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.status, XB_K_ATTN_BWD, 600);
      auto issue_sdp = [&](int j) -> bool {
        const int s = j % NS, b = j & 1;
        if (!mbar_wait(&bars->kv_full[s], (j / NS) & 1, abort_flag, p.status, XB_K_ATTN_BWD, 610 + s))
          return false;
        if (!mbar_wait(&bars->sdp_empty[b], ((j >> 1) & 1) ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 620 + b))
          return false;
        tc_fence_after();
        const uint32_t sk = xb_smem_u32(smem + SMEM_KV + s * 2 * KV_TILE_BYTES);
        const uint32_t sv = sk + KV_TILE_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * Q_CHUNK_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + COL_S + 128 * b, xb_smem_desc(kmaj, sq + a_off),
                        xb_smem_desc(kmaj, sk + b_off), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * Q_CHUNK_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + COL_DP + 128 * b, xb_smem_desc(kmaj, sdo + a_off),
                        xb_smem_desc(kmaj, sv + b_off), idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->sdp_full[b]);
        return true;
      };
      if (ok && n_steps > 0) ok = issue_sdp(0);
      for (int j = 0; j < n_steps && ok; ++j) {
        const int s = j % NS, b = j & 1;
        if (j + 1 < n_steps) {
          if (!issue_sdp(j + 1)) { ok = false; break; }
        }
        if (!mbar_wait(&bars->ds_full[b], (j >> 1) & 1, abort_flag, p.status, XB_K_ATTN_BWD, 630 + b)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sk = xb_smem_u32(smem + SMEM_KV + s * 2 * KV_TILE_BYTES);
        const uint32_t sds = xb_smem_u32(smem + SMEM_DS + b * DS_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          tc_mma_f16_ss(tmem_base + COL_DQ, xb_smem_desc(kmaj, sds + k * 32),
                        xb_smem_desc(mn_kv, sk + k * 2048), idesc_q, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&bars->kv_empty[s]);   // K_j (and V_j, read earlier) no longer needed
        tc_commit(&bars->ds_free[b]);
      }
      if (ok) tc_commit(&bars->dq_done);
    }
    __syncwarp();
  } else {
    // ------------------------------- row threads --------------------------------------
    const int q4 = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;        // which 32 of the 64 key columns (and which half of d)
    const int r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    const int q_pos = q0 + r;
    const bool row_valid = q_pos < seq_len;
    const size_t tok = (size_t)seq_start + q_pos;
    float lse = 0.f, delta = 0.f;
    if (row_valid) {
      lse = p.lse[(size_t)head * p.T + tok] * LOG2E;
      delta = p.delta[(size_t)head * p.T + tok];
    }
    const int lim = p.causal ? min(seq_len - 1, q_pos) : seq_len - 1;
    bool ok = true;
    for (int j = 0; j < n_steps && ok; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      // votes keep the warp together: the tcgen05.ld below is warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->sdp_full[b], ph, abort_flag, p.status, XB_K_ATTN_BWD, 700 + b))) {
        ok = false;
        break;
      }
      tc_fence_after();
      float ds[32];
      const int kv0 = (jt0 + j) * BKV + half * 32;
      {
        uint32_t a[32], d2[32];
        tmem_ld_32x32(tmem_base + lane_addr + COL_S + 128 * b + half * 32, a);
        tmem_ld_32x32(tmem_base + lane_addr + COL_DP + 128 * b + half * 32, d2);
        tc_wait_ld();
        // dS here is P o (dP - delta); the softmax scale is applied once, to dQ, at the end
        const int kt = (jt0 + j) * BKV;
        const bool no_mask = (q0 + BQ <= seq_len) && (kt + BKV <= seq_len) && (!p.causal || kt + BKV - 1 <= q0) &&
                             (p.window <= 0 || kt >= q0 + BQ - p.window);     // CTA-uniform
        if (no_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            ds[i] = xb_ex2(fmaf(__uint_as_float(a[i]), p.scale_log2, -lse)) * (__uint_as_float(d2[i]) - delta);
        } else {
          const int nvis = row_valid ? (lim - kv0 + 1) : 0;
          const int nlo = p.window > 0 ? (q_pos - p.window + 1) - kv0 : 0;   // columns below it are outside the window
#pragma unroll
          for (int i = 0; i < 32; ++i)
            ds[i] = (i < nvis && i >= nlo) ? xb_ex2(fmaf(__uint_as_float(a[i]), p.scale_log2, -lse)) *
                                   (__uint_as_float(d2[i]) - delta)
                             : 0.f;
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->sdp_empty[b]);
      // the dQ MMAs of step j-2 read this dS buffer: wait until they are done
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->ds_free[b], ph ^ 1, abort_flag, p.status, XB_K_ATTN_BWD, 710 + b))) {
        ok = false;
        break;
      }
      uint8_t* sd = smem + SMEM_DS + b * DS_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int c16 = half * 4 + c;
        uint4 w;
        w.x = pack_bf16x2(ds[c * 8 + 0], ds[c * 8 + 1]);
        w.y = pack_bf16x2(ds[c * 8 + 2], ds[c * 8 + 3]);
        w.z = pack_bf16x2(ds[c * 8 + 4], ds[c * 8 + 5]);
        w.w = pack_bf16x2(ds[c * 8 + 6], ds[c * 8 + 7]);
        *reinterpret_cast<uint4*>(sd + ((c16 ^ (r & 7)) * 16)) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->ds_full[b]);
    }
    if (ok && n_steps > 0) ok = mbar_wait(&bars->dq_done, 0, abort_flag, p.status, XB_K_ATTN_BWD, 720);
    // tcgen05.ld is warp-collective (.sync.aligned): every lane of the warp executes it, whether or
    // not its row exists; only the stores are per-row
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      float* dst = p.dq + (tok * p.Hq + head) * D + half * 64;     // this thread: 64 of the 128 features
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t a[32];
        if (n_steps > 0) {                                          // CTA-uniform
          tmem_ld_32x32(tmem_base + lane_addr + COL_DQ + half * 64 + c * 32, a);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 o = make_float4(__uint_as_float(a[i]) * p.scale, __uint_as_float(a[i + 1]) * p.scale,
                                   __uint_as_float(a[i + 2]) * p.scale, __uint_as_float(a[i + 3]) * p.scale);
            float4* d4 = reinterpret_cast<float4*>(dst + c * 32 + i);
            if (p.accumulate) {
              const float4 old = *d4;
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *d4 = o;
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

}  // namespace xb_attn_dq_ns

// dq[T, Hq, 128] fp32 (= or +=) dS K for every query row; same tensor-map inputs as xb_attn_bwd_ex.
// max_q_tiles bounds the grid (>= sum over sequences of ceil(len / 128)); 0 = derive from T.
XB_API int xb_attn_bwd_dq(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                          const float* delta, float* dq, const int* cu_seqlens, const int* k_starts,
                          long long ldq, long long ldk, long long ldv, long long lddo, int num_seqs, int T,
                          int Tk, int Hq, int Hkv, int causal, float scale, int accumulate, int max_q_tiles,
                          void* stream) {
  using namespace xb_attn_dq_ns;
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
  p.lse = lse; p.delta = delta; p.dq = dq; p.cu_seqlens = cu_seqlens; p.k_starts = k_starts;
  p.num_seqs = num_seqs; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal & 1; p.window = causal >> 1; p.accumulate = accumulate;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = xb_status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  const int tiles = max_q_tiles > 0 ? max_q_tiles : (T + BQ - 1) / BQ + num_seqs;
  dim3 grid(tiles, Hq);
  attn_bwd_dq_kernel<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
