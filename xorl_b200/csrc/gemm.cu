// Dense bf16 GEMM for sm_100a: C[M,N] (+)= op(A)[M,K] * op(B)[N,K]^T, fp32 accumulation in TMEM.
//
// One persistent CTA per SM, warp specialised:
//   warp 0      : TMA producer  (cp.async.bulk.tensor, 128B swizzle, 4-stage ring, no multicast)
//   warp 1      : MMA issuer    (one thread issues tcgen05.mma 128x256x16, commits to mbarriers)
//   warps 2..5  : epilogue      (tcgen05.ld from the finished accumulator -> registers -> global)
// Two 256-column accumulators (all 512 TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.
//
// Operand layouts ("major-ness"), chosen per call so that forward, dgrad and wgrad of a linear
// layer all run without a transpose pass:
//   a_mn = 0 : A stored [M, lda] with K contiguous      (K-major)
//   a_mn = 1 : A stored [K, lda] with M contiguous      (MN-major)
//   b_mn = 0 : B stored [N, ldb] with K contiguous      (K-major, i.e. an nn.Linear weight)
//   b_mn = 1 : B stored [K, ldb] with N contiguous      (MN-major)
// Replaces the cuBLAS `F.linear` calls and the CuTe-DSL GemmSm100 of the reference
// (src/xorl/ops/quack/gemm_sm100.py); unlike the latter it never uses multicast loads.
#include "common.cuh"

namespace xb_gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  int accumulate;
  int num_m_blocks, num_n_blocks, group_m;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& mb, int& nb) {
  // Group `group_m` row blocks together and walk N inside the group, so that the CTAs that run
  // concurrently share a compact set of A and B panels in L2.
  const int per_group = p.group_m * p.num_n_blocks;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.num_m_blocks - first_m);
  const int t = tile - g * per_group;
  mb = first_m + t % gsz;
  nb = t / gsz;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 128);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
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
      uint32_t it = 0;  // global k-block counter across tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(p, tile, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, p.status, XB_K_GEMM, 100 + s)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&bars->full[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, &tmap_a, &bars->full[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmap_a, &bars->full[s], m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmap_b, &bars->full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmap_b, &bars->full[s], n0 + 64 * j, k0);
          }
        }
      }
      if (!ok) {
        // Leave no bulk copy in flight into this CTA's shared memory: wait (bounded) for the
        // stages that were armed but possibly not yet landed.
        const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t i2 = it - 1 - j;
          const uint64_t t0 = xb_globaltimer();
          while (!mbar_try_wait(&bars->full[i2 % STAGES], (i2 / STAGES) & 1)) {
            if (xb_globaltimer() - t0 > 200000000ull) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = xb_idesc(1, 1, BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint64_t a_base = A_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t b_base = B_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint32_t a_kstep = A_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int acc = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, XB_K_GEMM,
                       200 + acc)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, abort_flag, p.status, XB_K_GEMM, 300 + s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = xb_smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = xb_smem_desc(a_base, sa + k * a_kstep);
            const uint64_t db = xb_smem_desc(b_base, sb + k * b_kstep);
            tc_mma_f16_ss(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&bars->empty[s]);  // frees the smem stage once these MMAs have read it
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue -----------------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tcount = 0;
    bool ok = true;
    const bool vec_ok = p.out_fp32
                            ? ((p.ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0)
                            : ((p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      int mb, nb;
      tile_coords(p, tile, mb, nb);
      const int acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[acc], acc_ph, abort_flag, p.status, XB_K_GEMM, 400 + acc))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = mb * BM + q * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
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
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
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
      mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p,
                  cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_kernel<A_MN, B_MN>;
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < xb_sm_count() ? tiles : xb_sm_count();
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace xb_gemm

// C[M,N] (+)= op(A) * op(B)^T.  See the header comment for a_mn / b_mn.  Leading dimensions are in
// elements and must be multiples of 8; A and B must be 16-byte aligned.  Returns 0 on success.
XB_API int xb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                        long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                        int accumulate, void* stream) {
  using namespace xb_gemm;
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
    rc = xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BN, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -3;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.num_m_blocks = (M + BM - 1) / BM;
  p.num_n_blocks = (N + BN - 1) / BN;
  p.group_m = 16;
  p.status = xb_status_ptr();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch<false, false>(ta, tb, p, st);
  if (!a_mn && b_mn) return launch<false, true>(ta, tb, p, st);
  if (a_mn && !b_mn) return launch<true, false>(ta, tb, p, st);
  return launch<true, true>(ta, tb, p, st);
}
