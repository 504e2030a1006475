// Dense bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] (+)= op(A)[M,K] * op(B)[N,K]^T.
//
// Two CTAs of a cluster share one 512 x 256 output tile.  Each CTA loads two 128-row sub-tiles of
// A and its own 128 columns of B per 64-deep K block (TMA, 128B swizzle, no multicast); the leader
// CTA's MMA thread issues tcgen05.mma.cta_group::2 (M = 256 across the pair, N = 256) once per A
// sub-tile, so every B stage feeds two MMAs.  Compared with one CTA per 128 x 256 tile this moves
// half the operand bytes per flop through L2 and shared memory, and a 4-stage ring of 48 KB covers
// twice the load latency.  Each CTA's tensor memory holds its 2 x (128 x 256) fp32 accumulators
// (all 512 columns); eight epilogue warps drain them, one set of four per sub-tile, and the MMA
// thread restarts on a sub-tile as soon as that sub-tile has been drained.
//
// Work items: the tiles that fill whole waves of the resident pairs are full 512 x 256 tiles; the
// tiles of the last, partial wave are cut in two (256 rows) or four (256 rows x 128 columns) when
// that shortens the tail, and all items are dealt round-robin to the pairs.
//
// Barriers: the peer's TMA loads complete on the leader's `full` barrier (one barrier tracks both
// halves of a stage); `empty` and `tmem_full` exist in both CTAs and the leader commits to each
// with its own tcgen05.commit; `tmem_empty[u]` lives in the leader and receives arrivals from the
// epilogue threads of both CTAs.  Every wait is bounded; after a timeout all roles of both CTAs
// drain and the tensor memory is freed.
// Same operand layouts and contract as the single-CTA kernel in gemm.cu (a_mn / b_mn).
#include <stdlib.h>

#include "gemm2_core.cuh"

namespace xb_gemm2 {

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const __grid_constant__ CUtensorMap tmap_b64, const __grid_constant__ CUtensorMap tmap_c,
             const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + OFF_BARS);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tmem_full, 1);
    mbar_init(&bars->tmem_empty[0], 256);
    mbar_init(&bars->tmem_empty[1], 256);
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_b64);
    if (p.tma_epilogue) tma_prefetch_desc(&tmap_c);
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
      for (int w = pair; w < p.num_items && ok; w += num_pairs) {
        const Item item = decode_item(p, w);
        const int m0 = item.m0 + (int)cta * BM;              // sub-tile u adds 256 * u
        const int bcols = item.ncols / 2;                     // B columns loaded by this CTA
        const int n0 = item.n0 + (int)cta * bcols;
        const uint32_t stage_tx = 2u * (uint32_t)(item.nsub * A_BYTES + bcols * BK * 2);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cl(&bars->empty[s], ph ^ 1, abort_flag, p.status, 100 + s)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + 2 * A_BYTES;
          const uint32_t full_leader = mapa_u32(xb_smem_u32(&bars->full[s]), 0);
          if (cta == 0) mbar_expect_tx(&bars->full[s], stage_tx);
          const int k0 = kb * BK;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (u >= item.nsub) break;
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
            tma_load_2d_pair(sb, bcols == BNH ? &tmap_b : &tmap_b64, full_leader, k0, n0);
          } else {
            for (int j = 0; j < bcols / 64; ++j)
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
      constexpr uint64_t a_base = A_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t b_base = B_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint32_t a_kstep = A_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      // cluster addresses of a barrier in the two CTAs differ from its local address by constants
      const uint32_t bars_local = xb_smem_u32(bars);
      const uint32_t off0 = mapa_u32(bars_local, 0) - bars_local;
      const uint32_t off1 = mapa_u32(bars_local, 1) - bars_local;
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      for (int w = pair; w < p.num_items && ok; w += num_pairs, ++tcount) {
        const Item item = decode_item(p, w);
        constexpr uint32_t idesc256 = xb_idesc(1, 1, 256, 256, A_MN ? 1 : 0, B_MN ? 1 : 0);
        constexpr uint32_t idesc128 = xb_idesc(1, 1, 256, 128, A_MN ? 1 : 0, B_MN ? 1 : 0);
        const uint32_t idesc = item.ncols == 256 ? idesc256 : idesc128;
        const uint32_t acc_ph = tcount & 1;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cl(&bars->full[s], ph, abort_flag, p.status, 300 + s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = xb_smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + 2 * A_BYTES;
          if (kb == 0) {
            // sub-tile by sub-tile, so that the first can start while the second is still drained
            for (int u = 0; u < 2; ++u) {
              if (!mbar_wait_cl(&bars->tmem_empty[u], acc_ph ^ 1, abort_flag, p.status, 200 + u)) {
                ok = false;
                break;
              }
              tc_fence_after();
              if (u < item.nsub) {
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                  tc_mma2_f16_ss(tmem_base + u * BN, xb_smem_desc(a_base, sa + u * A_BYTES + k * a_kstep),
                                 xb_smem_desc(b_base, sb + k * b_kstep), idesc, k > 0 ? 1u : 0u);
              }
            }
            if (!ok) break;
          } else if (item.nsub == 2) {
            issue_kblock<A_MN, B_MN, 2>(tmem_base, sa, sb, idesc, false);
          } else {
            issue_kblock<A_MN, B_MN, 1>(tmem_base, sa, sb, idesc, false);
          }
          const uint32_t e = xb_smem_u32(&bars->empty[s]);
          tc_commit2(e + off0);
          tc_commit2(e + off1);
        }
        if (ok) {
          const uint32_t f = xb_smem_u32(&bars->tmem_full);
          tc_commit2(f + off0);
          tc_commit2(f + off1);
        }
      }
    }
    __syncwarp();
  } else {
    // --------------- epilogue (both CTAs; warps 2-5 sub-tile 0, warps 6-9 sub-tile 1) ----------
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int u = (warp - 2) >> 2;          // sub-tile drained by this warp
    uint32_t tcount = 0;
    bool ok = true;
    const bool vec_ok = p.out_fp32
                            ? ((p.ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0)
                            : ((p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0);
    for (int w = pair; w < p.num_items && ok; w += num_pairs, ++tcount) {
      const Item item = decode_item(p, w);
      if (!mbar_wait_warp(&bars->tmem_full, tcount & 1, abort_flag, p.status, 400 + u)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t empty_leader = mapa_u32(xb_smem_u32(&bars->tmem_empty[u]), 0);
      const int row = item.m0 + 256 * u + (int)cta * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + u * BN + ((uint32_t)(q * 32) << 16);
      const int nchunks = u < item.nsub ? item.ncols / 32 : 0;
      if (p.tma_epilogue) {
        // Slabs of 128 rows x 128 bytes (64 bf16 or 32 fp32 columns) go through 128B-swizzled shared
        // memory and one TMA store (or TMA add, when accumulating into fp32) each: global memory sees
        // whole 128-byte row segments and no thread waits on a global store.
        uint8_t* slab = smem + OFF_SLAB + u * SLAB_BYTES;
        const int r = q * 32 + lane;
        uint8_t* srow = slab + r * 128;
        const bool leader = (warp - 2 - 4 * u) == 0 && lane == 0;
        const int row0 = item.m0 + 256 * u + (int)cta * BM;
        const int per_slab = p.out_fp32 ? 1 : 2;             // 32-column chunks per slab
#pragma unroll 1
        for (int c = 0; c < nchunks; c += per_slab) {
          const int col0 = item.n0 + c * 32;
          if (col0 >= p.N) break;
          uint32_t v[2][32];
          tmem_ld_32x32(taddr + c * 32, v[0]);
          if (per_slab == 2) tmem_ld_32x32(taddr + c * 32 + 32, v[1]);
          tc_wait_ld();
          if (leader) tma_store_wait_read<0>();               // the previous slab has left shared memory
          if (u == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
          else asm volatile("bar.sync 3, 128;" ::: "memory");
          if (p.out_fp32) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(srow + ((j ^ (r & 7)) * 16)) =
                  make_uint4(v[0][4 * j], v[0][4 * j + 1], v[0][4 * j + 2], v[0][4 * j + 3]);
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[h][8 * j]), __uint_as_float(v[h][8 * j + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[h][8 * j + 2]), __uint_as_float(v[h][8 * j + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[h][8 * j + 4]), __uint_as_float(v[h][8 * j + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[h][8 * j + 6]), __uint_as_float(v[h][8 * j + 7]));
                *reinterpret_cast<uint4*>(srow + (((h * 4 + j) ^ (r & 7)) * 16)) = o;
              }
          }
          fence_proxy_async_smem();
          if (u == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
          else asm volatile("bar.sync 3, 128;" ::: "memory");
          if (leader) {
            if (p.accumulate) tma_reduce_add_2d(&tmap_c, slab, col0, row0);
            else tma_store_2d(&tmap_c, slab, col0, row0);
            tma_store_commit();
          }
        }
        tc_fence_before();
        mbar_arrive_cluster(empty_leader);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < nchunks; ++c) {
        const int col0 = item.n0 + c * 32;
        if (col0 >= p.N) break;
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
      mbar_arrive_cluster(empty_leader);
    }
    if (p.tma_epilogue && (warp - 2 - 4 * u) == 0 && lane == 0) tma_store_wait<0>();
  }

  // Both CTAs must be done with tensor memory (and with each other's barriers) before it is freed.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

// Batch-invariant mode: every output tile is a full 512 x 256 pair tile issued with the same MMA
// shapes whatever M and N are (the tiles of a partial last wave are not cut), so the value of an
// output row does not depend on how many other rows the call carries.
static int g_batch_invariant = 0;

static int resident_pairs_cache[64] = {0};

template <bool A_MN, bool B_MN>
static int resident_pairs() {
  int dev = 0;
  cudaGetDevice(&dev);
  static bool configured[64] = {false};
  auto kern = gemm2_kernel<A_MN, B_MN>;
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -1;
    configured[dev & 63] = true;
  }
  if (!resident_pairs_cache[dev & 63]) {
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
    resident_pairs_cache[dev & 63] = clusters;
  }
  return resident_pairs_cache[dev & 63];
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb64, const CUtensorMap& tc,
                  Params& p, cudaStream_t stream) {
  const int pairs_max = resident_pairs<A_MN, B_MN>();
  if (pairs_max <= 0) return -10;
  plan_items(p, pairs_max, true);
  if (g_batch_invariant) {
    p.full_items = p.num_m_blocks * p.num_n_blocks;
    p.split_m = p.split_n = 1;
    p.num_items = p.full_items;
  }
  const int pairs = p.num_items < pairs_max ? p.num_items : pairs_max;
  gemm2_kernel<A_MN, B_MN><<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tb64, tc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace xb_gemm2

XB_API int xb_gemm_set_batch_invariant(int on) {
  const int prev = xb_gemm2::g_batch_invariant;
  xb_gemm2::g_batch_invariant = on ? 1 : 0;
  return prev;
}

// Same contract as xb_gemm_bf16.
XB_API int xb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                             int accumulate, void* stream) {
  using namespace xb_gemm2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) ||
      (reinterpret_cast<uintptr_t>(B) % 16))
    return -1;
  CUtensorMap ta, tb, tb64;
  int rc;
  if (!a_mn)
    rc = xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -2;
  if (!b_mn) {
    rc = xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BNH, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc)
      rc = xb_make_tmap_2d(&tb64, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, 64, BK,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    rc = xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
    tb64 = tb;
  }
  if (rc) return -3;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.num_m_blocks = (M + 511) / 512;
  p.num_n_blocks = (N + BN - 1) / BN;
  p.group_m = 4;
  p.status = xb_status_ptr();
  // Output through shared memory + TMA when C can be described by a tensor map (16-byte aligned base
  // and row pitch) and the mode has a TMA form: plain store, or fp32 add for accumulation.
  CUtensorMap tc = ta;
  const int es = out_fp32 ? 4 : 2;
  p.tma_epilogue = 0;
  static const bool tma_epi_enabled = []() {
    const char* e = getenv("XORL_B200_GEMM_TMA_EPILOGUE");
    return !(e && e[0] == '0');
  }();
  if (tma_epi_enabled && (ldc * es) % 16 == 0 && reinterpret_cast<uintptr_t>(C) % 16 == 0 && (!accumulate || out_fp32)) {
    if (xb_make_tmap_2d(&tc, C, out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, es, M, N,
                        ldc, BM, 128 / es, CU_TENSOR_MAP_SWIZZLE_128B) == 0)
      p.tma_epilogue = 1;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch<false, false>(ta, tb, tb64, tc, p, st);
  if (!a_mn && b_mn) return launch<false, true>(ta, tb, tb64, tc, p, st);
  if (a_mn && !b_mn) return launch<true, false>(ta, tb, tb64, tc, p, st);
  return launch<true, true>(ta, tb, tb64, tc, p, st);
}
