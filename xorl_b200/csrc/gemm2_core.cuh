// Shared pieces of the CTA-pair bf16 GEMM kernels (tile constants, work-item decoding, cluster-scope
// barrier waits, cta_group::2 TMA / MMA / commit wrappers).  Used by gemm2.cu (plain GEMM) and
// gemm_fused.cu (GEMM with an all-gather of one operand and / or a reduce-scatter of the result
// over peer memory in the same kernel).
#pragma once
#include "common.cuh"

namespace xb_gemm2 {

constexpr int BM = 128;          // rows of one A sub-tile (per CTA)
constexpr int BN = 256;          // columns of a full tile
constexpr int BNH = 128;         // columns of B loaded by one CTA for a full tile
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = 2 * A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 320;   // TMA warp, MMA warp, 2 x 4 epilogue warps
constexpr int TMEM_COLS = 512;
// Epilogue staging: one 16 KB slab (128 rows x 128 bytes, 128B-swizzled) per epilogue warp group.
constexpr int SLAB_BYTES = BM * 128;
constexpr int OFF_SLAB = STAGES * STAGE_BYTES;
constexpr int OFF_BARS = OFF_SLAB + 2 * SLAB_BYTES;
constexpr int SMEM_BYTES = OFF_BARS + 1024 + 256;

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  int accumulate;
  int num_m_blocks, num_n_blocks, group_m;   // grid of full 512 x 256 tiles
  int full_items;                            // tiles [0, full_items) are processed whole
  int split_m, split_n;                      // the remaining tiles are cut split_m x split_n ways
  int num_items;
  int tma_epilogue;                          // C is written through shared memory and TMA stores
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Item {
  int m0, n0;      // origin of the pair's item
  int nsub;        // 128-row A sub-tiles per CTA (2: 512 rows per pair, 1: 256 rows)
  int ncols;       // 256 or 128
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cl(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(xb_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait with cluster-scope acquire (the signal may come from the peer CTA).
__device__ __forceinline__ bool mbar_wait_cl(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                             int* status, int detail) {
  if (mbar_try_wait_cl(bar, parity)) return true;
  const uint64_t t0 = xb_globaltimer();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_cl(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (xb_globaltimer() - t0 > XB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        xb_report(status, XB_ERR_MBAR_TIMEOUT, XB_K_GEMM, detail);
        return false;
      }
    }
  }
}
// Warp-collective wait for long waits (epilogue warps sit out a whole main loop): one lane polls,
// with a sleep between polls, so that the barrier word in shared memory is not hammered by 32
// threads per warp while the tensor core streams its operands from the same shared memory.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int detail) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    if (!mbar_try_wait_cl(bar, parity)) {
      const uint64_t t0 = xb_globaltimer();
      for (uint32_t it = 1;; ++it) {
        __nanosleep(40);
        if (mbar_try_wait_cl(bar, parity)) break;
        if ((it & 15u) == 0u) {
          if (*abort_flag) { ok = 0; break; }
          if (xb_globaltimer() - t0 > XB_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            xb_report(status, XB_ERR_MBAR_TIMEOUT, XB_K_GEMM, detail);
            ok = 0;
            break;
          }
        }
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}
// TMA load whose completion is signalled on a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      ::"r"(xb_smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   xb_smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma2_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at a cluster address once all MMAs issued so far by this thread are done.
__device__ __forceinline__ void tc_commit2(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_cluster_addr)
               : "memory");
}

// All MMAs of one K block, fully unrolled for a compile-time number of A sub-tiles.
template <bool A_MN, bool B_MN, int NSUB>
__device__ __forceinline__ void issue_kblock(uint32_t tmem_base, uint32_t sa, uint32_t sb, uint32_t idesc,
                                             bool first) {
  constexpr uint64_t a_base = A_MN ? xb_smem_desc_base_sw128(BK * 128, 1024) : xb_smem_desc_base_sw128(16, 1024);
  constexpr uint64_t b_base = B_MN ? xb_smem_desc_base_sw128(BK * 128, 1024) : xb_smem_desc_base_sw128(16, 1024);
  constexpr uint32_t a_kstep = A_MN ? (UMMA_K * 128) : (UMMA_K * 2);
  constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
#pragma unroll
  for (int k = 0; k < BK / UMMA_K; ++k) {
    const uint64_t db = xb_smem_desc(b_base, sb + k * b_kstep);
#pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tc_mma2_f16_ss(tmem_base + u * BN, xb_smem_desc(a_base, sa + u * A_BYTES + k * a_kstep), db, idesc,
                     (first && k == 0) ? 0u : 1u);
  }
}

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& mb, int& nb) {
  const int per_group = p.group_m * p.num_n_blocks;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.num_m_blocks - first_m);
  const int t = tile - g * per_group;
  mb = first_m + t % gsz;
  nb = t / gsz;
}

__device__ __forceinline__ Item decode_item(const Params& p, int w) {
  Item it;
  int tile, um = 0, un = 0;
  if (w < p.full_items) {
    tile = w;
    it.nsub = 2;
    it.ncols = BN;
  } else {
    const int parts = p.split_m * p.split_n;
    const int j = w - p.full_items;
    tile = p.full_items + j / parts;
    const int sub = j % parts;
    um = sub % p.split_m;
    un = sub / p.split_m;
    it.nsub = p.split_m == 2 ? 1 : 2;
    it.ncols = BN / p.split_n;
  }
  int mb, nb;
  tile_coords(p, tile, mb, nb);
  it.m0 = mb * 512 + um * 256;
  it.n0 = nb * BN + un * it.ncols;
  return it;
}

// Cuts the tiles of the last, partial wave when that shortens it: a piece of a tile cut f ways takes
// about 1/f of a tile's time (a little more, hence the penalties), and T tiles cut f ways need
// ceil(T f / P) rounds on P pairs.
static inline void plan_items(Params& p, int pairs, bool can_split_n) {
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int tail = tiles % pairs;
  p.full_items = tiles - tail;
  p.split_m = p.split_n = 1;
  if (tail) {
    const float penalty[3] = {1.00f, 1.10f, 1.50f};
    const int f[3] = {1, 2, 4};
    float best = 1e30f;
    for (int i = 0; i < (can_split_n ? 3 : 2); ++i) {
      const int rounds = (tail * f[i] + pairs - 1) / pairs;
      const float cost = penalty[i] * (float)rounds / (float)f[i];
      if (cost < best - 1e-6f) {
        best = cost;
        p.split_m = f[i] >= 2 ? 2 : 1;
        p.split_n = f[i] == 4 ? 2 : 1;
      }
    }
  }
  p.num_items = p.full_items + tail * p.split_m * p.split_n;
}

}  // namespace xb_gemm2
