// Dense bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] (+)= op(A)[M,K] * op(B)[N,K]^T.
//
// Two CTAs of a cluster share one 256x256 output tile.  Each loads its own 128 rows of A and its
// own 128 columns of B (TMA, 128B swizzle, no multicast), so a CTA moves 32 KB per 64-deep K block
// instead of 48 KB, the shared-memory ring has 6 stages instead of 4, and every B element is read
// from L2 once per pair.  The leader CTA's MMA thread issues tcgen05.mma.cta_group::2 (M = 256
// across the pair, N = 256); each CTA's tensor memory receives the accumulator rows of its half
// and each CTA's epilogue warps write them out.
//
// Barriers: the peer's TMA loads complete on the leader's `full` barrier (one barrier tracks both
// halves of a stage); `empty` and `tmem_full` exist in both CTAs and the leader commits to each
// with its own tcgen05.commit; `tmem_empty` lives in the leader and receives arrivals from the
// epilogue threads of both CTAs.  Every wait is bounded; after a timeout all roles of both CTAs
// drain and the tensor memory is freed.
//
// MSUB = 2 doubles the rows per CTA (pair tile 512 x 256): every B stage is used by two MMAs, which
// cuts the operand bytes per flop by a quarter and doubles the time a stage of the ring covers
// (4 stages of 48 KB).  Both accumulators of a CTA (all 512 tensor-memory columns) then belong to
// one tile, so the epilogue does not overlap the next tile's MMAs, only its loads.
// Same operand layouts and contract as the single-CTA kernel in gemm.cu (a_mn / b_mn).
#include "common.cuh"

namespace xb_gemm2 {

constexpr int BM = 128;          // rows of A per CTA (256 per pair)
constexpr int BN = 256;          // columns of the pair's tile
constexpr int BNH = 128;         // columns of B loaded by one CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;          // one 128-row A sub-tile
constexpr int B_BYTES = BNH * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int MAX_STAGES = 6;
template <int MSUB> struct Cfg {
  static constexpr int STAGES = MSUB == 1 ? 6 : 4;
  static constexpr int STAGE_BYTES = MSUB * A_BYTES + B_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int NUM_ACC = 2 / MSUB;       // accumulator sets in tensor memory
  static constexpr int ACC_COLS = BN * MSUB;
  static constexpr int TILE_M = 256 * MSUB;      // rows of the pair's tile
};

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  int accumulate;
  int num_m_blocks, num_n_blocks, group_m;   // in units of pair tiles
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
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

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& mb, int& nb) {
  const int per_group = p.group_m * p.num_n_blocks;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.num_m_blocks - first_m);
  const int t = tile - g * per_group;
  mb = first_m + t % gsz;
  nb = t / gsz;
}

template <bool A_MN, bool B_MN, int MSUB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const Params p) {
  constexpr int STAGES = Cfg<MSUB>::STAGES;
  constexpr int STAGE_BYTES = Cfg<MSUB>::STAGE_BYTES;
  constexpr int NUM_ACC = Cfg<MSUB>::NUM_ACC;
  constexpr int ACC_COLS = Cfg<MSUB>::ACC_COLS;
  constexpr int TILE_M = Cfg<MSUB>::TILE_M;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 256);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc2(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();           // barriers of both CTAs initialised, tensor memory allocated
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int mb, nb;
        tile_coords(p, tile, mb, nb);
        const int m0 = mb * TILE_M + (int)cta * BM;     // sub-tile j adds 256 * j
        const int n0 = nb * BN + (int)cta * BNH;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cl(&bars->empty[s], ph ^ 1, abort_flag, p.status, 100 + s)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + MSUB * A_BYTES;
          const uint32_t full_leader = mapa_u32(xb_smem_u32(&bars->full[s]), 0);
          if (cta == 0) mbar_expect_tx(&bars->full[s], 2 * STAGE_BYTES);
          const int k0 = kb * BK;
#pragma unroll
          for (int u = 0; u < MSUB; ++u) {
            if (!A_MN) {
              tma_load_2d_pair(sa + u * A_BYTES, &tmap_a, full_leader, k0, m0 + 256 * u);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d_pair(sa + u * A_BYTES + j * (BK * 128), &tmap_a, full_leader,
                                 m0 + 256 * u + 64 * j, k0);
            }
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, full_leader, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &tmap_b, full_leader, n0 + 64 * j, k0);
          }
        }
      }
      if (!ok && cta == 0) {
        // Wait (bounded) for stages that were armed: no bulk copy may still be in flight into
        // shared memory when the CTAs exit.  The peer's copies complete on these barriers too.
        const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t i2 = it - 1 - j;
          const uint64_t t0 = xb_globaltimer();
          while (!mbar_try_wait_cl(&bars->full[i2 % STAGES], (i2 / STAGES) & 1)) {
            if (xb_globaltimer() - t0 > 200000000ull) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) ---------------------
    if (cta == 0 && lane == 0) {
      constexpr uint32_t idesc = xb_idesc(1, 1, 256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint64_t a_base = A_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t b_base = B_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint32_t a_kstep = A_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
        const int acc = tcount % NUM_ACC;
        const uint32_t acc_ph = (tcount / NUM_ACC) & 1;
        if (!mbar_wait_cl(&bars->tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, 200 + acc)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cl(&bars->full[s], ph, abort_flag, p.status, 300 + s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = xb_smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + MSUB * A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t db = xb_smem_desc(b_base, sb + k * b_kstep);
#pragma unroll
            for (int u = 0; u < MSUB; ++u) {
              const uint64_t da = xb_smem_desc(a_base, sa + u * A_BYTES + k * a_kstep);
              tc_mma2_f16_ss(d_tmem + u * BN, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          const uint32_t e = xb_smem_u32(&bars->empty[s]);
          tc_commit2(mapa_u32(e, 0));
          tc_commit2(mapa_u32(e, 1));
        }
        if (ok) {
          const uint32_t f = xb_smem_u32(&bars->tmem_full[acc]);
          tc_commit2(mapa_u32(f, 0));
          tc_commit2(mapa_u32(f, 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (both CTAs, own 128 rows) ----------------
    const int q = warp & 3;
    uint32_t tcount = 0;
    bool ok = true;
    const bool vec_ok = p.out_fp32
                            ? ((p.ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0)
                            : ((p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
      int mb, nb;
      tile_coords(p, tile, mb, nb);
      const int acc = tcount % NUM_ACC;
      const uint32_t acc_ph = (tcount / NUM_ACC) & 1;
      if (!mbar_wait_cl(&bars->tmem_full[acc], acc_ph, abort_flag, p.status, 400 + acc)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = mb * TILE_M + (int)cta * BM + q * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < ACC_COLS / 32; ++c) {
        const int row = row0 + 256 * (c / (BN / 32));
        const int col0 = n0 + (c % (BN / 32)) * 32;
        if (col0 >= p.N) continue;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        if (row < p.M) {
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + 4 * v);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + 4 * v) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float o = __uint_as_float(r[j]);
                  if (p.accumulate) o += dst[j];
                  dst[j] = o;
                }
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * v + j]);
                if (p.accumulate) {
                  const uint4 old = *reinterpret_cast<const uint4*>(dst + 8 * v);
                  const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y),
                               o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst + 8 * v) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float o = __uint_as_float(r[j]);
                  if (p.accumulate) o += __bfloat162float(dst[j]);
                  dst[j] = __float2bfloat16(o);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(mapa_u32(xb_smem_u32(&bars->tmem_empty[acc]), 0));
    }
  }

  // Both CTAs must be done with tensor memory (and with each other's barriers) before it is freed.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int MSUB>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, cudaStream_t stream) {
  static int pairs_for_dev[64] = {0};
  constexpr int SMEM_BYTES = Cfg<MSUB>::SMEM_BYTES;
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm2_kernel<A_MN, B_MN, MSUB>;
  if (!pairs_for_dev[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -10;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (xb_sm_count() / 2));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = xb_sm_count() / 2;
    }
    if (clusters > xb_sm_count() / 2) clusters = xb_sm_count() / 2;
    pairs_for_dev[dev & 63] = clusters;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int pairs = tiles < pairs_for_dev[dev & 63] ? tiles : pairs_for_dev[dev & 63];
  kern<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace xb_gemm2

// Same contract as xb_gemm_bf16.  msub = 1: pair tile 256 x 256 with double-buffered accumulators;
// msub = 2: pair tile 512 x 256.
XB_API int xb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                             int accumulate, int msub, void* stream) {
  using namespace xb_gemm2;
  if (msub != 1 && msub != 2) return -1;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) ||
      (reinterpret_cast<uintptr_t>(B) % 16))
    return -1;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn)
    rc = xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -2;
  if (!b_mn)
    rc = xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BNH, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -3;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.num_m_blocks = (M + 256 * msub - 1) / (256 * msub);
  p.num_n_blocks = (N + BN - 1) / BN;
  p.group_m = 8 / msub;
  p.status = xb_status_ptr();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (msub == 1) {
    if (!a_mn && !b_mn) return launch<false, false, 1>(ta, tb, p, st);
    if (!a_mn && b_mn) return launch<false, true, 1>(ta, tb, p, st);
    if (a_mn && !b_mn) return launch<true, false, 1>(ta, tb, p, st);
    return launch<true, true, 1>(ta, tb, p, st);
  }
  if (!a_mn && !b_mn) return launch<false, false, 2>(ta, tb, p, st);
  if (!a_mn && b_mn) return launch<false, true, 2>(ta, tb, p, st);
  if (a_mn && !b_mn) return launch<true, false, 2>(ta, tb, p, st);
  return launch<true, true, 2>(ta, tb, p, st);
}
