// Grouped (per-expert) bf16 GEMMs for MoE on tcgen05, over a token buffer whose expert segments
// start at multiples of 128 rows (segment table `seg[E+1]`, int32, on the device — no host sync).
//
//   rows mode  : C[rows of e, :] = A[rows of e, :] @ op(B[e])      forward (B stored [E,K,N]) and
//                                                                   dgrad  (B stored [E,N,K])
//   wgrad mode : C[e] (+)= A[rows of e, :]^T @ B[rows of e, :]     per-expert weight gradient
//
// Same warp-specialised persistent structure as csrc/gemm.cu (TMA producer / MMA issuer / four
// epilogue warps, 4-stage ring, two TMEM accumulators).  In rows mode the epilogue stages 64-column
// bf16 slabs in swizzled shared memory and writes them with TMA stores.  Because segments are 128-row aligned a
// 128-row tile never straddles two experts, and a 64-row reduction block never mixes experts.
// Replaces the Triton group_gemm_same_nk / same_mn kernels of the reference
// (src/xorl/ops/group_gemm/kernel/group_gemm.py:80-377).
#include "common.cuh"

namespace xb_ggemm {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192, TMEM_COLS = 512;
constexpr int MAX_E = 512;
constexpr int SLAB_COLS = 64;                      // rows-mode epilogue staging: 128 rows x 64 columns bf16
constexpr int SLAB_BYTES = BM * SLAB_COLS * 2;
constexpr int OFF_SLAB = STAGES * STAGE_BYTES;
constexpr int OFF_BARS = OFF_SLAB + SLAB_BYTES;
constexpr int SMEM_BYTES = OFF_BARS + 1024 + 256 + (MAX_E + 1) * 4;

struct Params {
  int mode;  // 0 rows, 1 wgrad
  int E, R, M, N, K;
  const int* seg;
  void* C;
  long long ldc;       // rows mode: row stride of C; wgrad: N (row stride inside one expert)
  int out_fp32, accumulate;
  int b_mn;            // rows mode: B stored [E,K,N] (1) or [E,N,K] (0)
  int num_m_blocks, num_n_blocks;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Tile {
  int e, m0, n0, k0, num_kb;
  bool valid;
};

__device__ __forceinline__ Tile get_tile(const Params& p, const int* sseg, int t) {
  Tile r;
  if (p.mode == 0) {
    // groups of GROUP_M row blocks, inside a group row block fastest: the CTAs running at any time
    // share a few B tiles and one group of A rows (resident in L2) instead of streaming all of A once
    // per column block
    constexpr int GROUP_M = 16;
    const int per_group = GROUP_M * p.num_n_blocks;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, p.num_m_blocks - first_m);
    const int u = t - g * per_group;
    const int mb = first_m + u % gsz, nb = u / gsz;
    r.m0 = mb * BM;
    r.n0 = nb * BN;
    r.k0 = 0;
    r.num_kb = (p.K + BK - 1) / BK;
    int e = -1;
    for (int i = 0; i < p.E; ++i)
      if (r.m0 >= sseg[i] && r.m0 < sseg[i + 1]) { e = i; break; }
    r.e = e;
    r.valid = e >= 0;
  } else {
    const int per_e = p.num_m_blocks * p.num_n_blocks;
    r.e = t / per_e;
    const int u = t - r.e * per_e;
    r.m0 = (u % p.num_m_blocks) * BM;
    r.n0 = (u / p.num_m_blocks) * BN;
    r.k0 = sseg[r.e];
    r.num_kb = (sseg[r.e + 1] - sseg[r.e]) / BK;
    r.valid = true;
  }
  return r;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
ggemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + OFF_BARS);
  int* sseg = reinterpret_cast<int*>(smem + OFF_BARS + 256);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.mode == 0 ? p.num_m_blocks * p.num_n_blocks
                                    : p.E * p.num_m_blocks * p.num_n_blocks;
  for (int i = threadIdx.x; i <= p.E; i += NUM_THREADS) sseg[i] = p.seg[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->tmem_full[a], 1); mbar_init(&bars->tmem_empty[a], 128); }
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.mode == 0) tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const bool a_mn = p.mode == 1;
  const bool b_mn = p.mode == 1 || p.b_mn;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = get_tile(p, sseg, t);
        if (!tl.valid) continue;
        for (int kb = 0; kb < tl.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&bars->empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.status,
                         XB_K_GROUPED_GEMM, 100 + s)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&bars->full[s], STAGE_BYTES);
          const int k0 = tl.k0 + kb * BK;
          if (!a_mn) {
            tma_load_2d(sa, &tmap_a, &bars->full[s], k0, tl.m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmap_a, &bars->full[s], tl.m0 + 64 * j, k0);
          }
          if (p.mode == 1) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmap_b, &bars->full[s], tl.n0 + 64 * j, k0);
          } else if (b_mn) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (BK * 128), &tmap_b, &bars->full[s], tl.n0 + 64 * j, k0, tl.e);
          } else {
            tma_load_3d(sb, &tmap_b, &bars->full[s], k0, tl.n0, tl.e);
          }
        }
      }
      if (!ok) {
        const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        const uint64_t t0 = xb_globaltimer();
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t i2 = it - 1 - j;
          while (!mbar_try_wait(&bars->full[i2 % STAGES], (i2 / STAGES) & 1) &&
                 xb_globaltimer() - t0 < 200000000ull) {}
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = xb_idesc(1, 1, BM, BN, a_mn ? 1 : 0, b_mn ? 1 : 0);
      const uint64_t a_base = a_mn ? xb_smem_desc_base_sw128(BK * 128, 1024) : xb_smem_desc_base_sw128(16, 1024);
      const uint64_t b_base = b_mn ? xb_smem_desc_base_sw128(BK * 128, 1024) : xb_smem_desc_base_sw128(16, 1024);
      const uint32_t a_kstep = a_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      const uint32_t b_kstep = b_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = get_tile(p, sseg, t);
        if (!tl.valid || tl.num_kb == 0) continue;
        const int acc = tcount & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], ((tcount >> 1) & 1) ^ 1, abort_flag, p.status,
                       XB_K_GROUPED_GEMM, 200 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < tl.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&bars->full[s], (it / STAGES) & 1, abort_flag, p.status, XB_K_GROUPED_GEMM,
                         300 + s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = xb_smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16_ss(d_tmem, xb_smem_desc(a_base, sa + k * a_kstep),
                          xb_smem_desc(b_base, sb + k * b_kstep), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->empty[s]);
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
        ++tcount;
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    uint32_t tcount = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile tl = get_tile(p, sseg, t);
      if (!tl.valid) continue;
      const bool has_acc = tl.num_kb > 0;
      const int acc = tcount & 1;
      if (has_acc) {
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[acc], (tcount >> 1) & 1, abort_flag, p.status,
                       XB_K_GROUPED_GEMM, 400 + acc))) { ok = false; break; }
        tc_fence_after();
      } else if (p.accumulate) {
        continue;  // nothing to add for an expert without tokens
      }
      if (p.mode == 0) {
        // rows mode (bf16 out, no accumulation): stage 64-column slabs in 128B-swizzled shared memory
        // and let TMA write them, so that global memory sees whole 128-byte row segments
        const int r = q * 32 + lane;
        const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
        uint8_t* slab = smem + OFF_SLAB;
        uint8_t* srow = slab + r * 128;
#pragma unroll 1
        for (int sl = 0; sl < BN / SLAB_COLS; ++sl) {
          const int col0 = tl.n0 + sl * SLAB_COLS;
          if (col0 >= p.N) break;
          uint32_t v[2][32];
          tmem_ld_32x32(taddr + sl * SLAB_COLS, v[0]);
          tmem_ld_32x32(taddr + sl * SLAB_COLS + 32, v[1]);
          tc_wait_ld();
          if (warp == 2 && lane == 0) tma_store_wait_read<0>();
          asm volatile("bar.sync 2, 128;" ::: "memory");
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
          fence_proxy_async_smem();
          asm volatile("bar.sync 2, 128;" ::: "memory");
          if (warp == 2 && lane == 0) {
            tma_store_2d(&tmap_c, slab, col0, tl.m0);
            tma_store_commit();
          }
        }
        tc_fence_before();
        mbar_arrive(&bars->tmem_empty[acc]);
        ++tcount;
        continue;
      }
      const int row = tl.m0 + q * 32 + lane;
      const int row_limit = p.mode == 0 ? p.R : p.M;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const long long base = p.mode == 0 ? 0 : (long long)tl.e * p.M * p.N;
      const int es = p.out_fp32 ? 4 : 2;
      const bool vec_ok = (p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tl.n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        if (has_acc) {
          tmem_ld_32x32(taddr + c * 32, r);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (row < row_limit) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(p.C) + (base + (long long)row * p.ldc + col0) * es;
          const bool full = vec_ok && col0 + 32 <= p.N;
          if (p.out_fp32) {
            float* d = reinterpret_cast<float*>(dst);
            for (int j = 0; j < 32; j += 4) {
              if (full) {
                float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                       __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(d + j);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(d + j) = o;
              } else {
                for (int u = j; u < j + 4; ++u)
                  if (col0 + u < p.N) d[u] = __uint_as_float(r[u]) + (p.accumulate ? d[u] : 0.f);
              }
            }
          } else {
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst);
            for (int j = 0; j < 32; j += 8) {
              if (full) {
                float f[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) f[u] = __uint_as_float(r[j + u]);
                if (p.accumulate) {
                  const uint4 old = *reinterpret_cast<const uint4*>(d + j);
                  const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y),
                               o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(d + j) = o;
              } else {
                for (int u = j; u < j + 8; ++u)
                  if (col0 + u < p.N)
                    d[u] = __float2bfloat16(__uint_as_float(r[u]) +
                                            (p.accumulate ? __bfloat162float(d[u]) : 0.f));
              }
            }
          }
        }
      }
      if (has_acc) {
        tc_fence_before();
        mbar_arrive(&bars->tmem_empty[acc]);
        ++tcount;
      }
    }
    if (p.mode == 0 && warp == 2 && lane == 0) tma_store_wait<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const Params& p,
                  cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(ggemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess) return -10;
    configured[dev & 63] = true;
  }
  const int tiles = p.mode == 0 ? p.num_m_blocks * p.num_n_blocks : p.E * p.num_m_blocks * p.num_n_blocks;
  if (tiles <= 0) return 0;
  const int grid = tiles < xb_sm_count() ? tiles : xb_sm_count();
  ggemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, tc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace xb_ggemm

// A [R, K] (row stride lda), B [E, K, N] (b_mn = 1) or [E, N, K] (b_mn = 0), C [R, N] (stride ldc),
// seg int32 [E+1] with 128-aligned entries and seg[E] <= R.  Rows >= seg[E] are not written.
XB_API int xb_grouped_gemm_rows(const void* A, const void* B, void* C, const int* seg, int E,
                                long long R, int N, int K, long long lda, long long ldc, int b_mn,
                                void* stream) {
  using namespace xb_ggemm;
  if (E <= 0 || R <= 0) return 0;
  if (E > MAX_E || (R % BM) || (lda % 8) || (K % 8) || (N % 8) || (ldc % 8) ||
      (reinterpret_cast<uintptr_t>(C) % 16)) return -1;
  CUtensorMap ta, tb, tc;
  if (xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, lda, BM, BK,
                      CU_TENSOR_MAP_SWIZZLE_128B)) return -2;
  if (xb_make_tmap_2d(&tc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, ldc, BM, SLAB_COLS,
                      CU_TENSOR_MAP_SWIZZLE_128B)) return -4;
  int rc;
  if (b_mn)
    rc = xb_make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, E, K, N, (uint64_t)K * N, N, 1,
                         BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = xb_make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, E, N, K, (uint64_t)K * N, K, 1,
                         BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -3;
  Params p{};
  p.mode = 0; p.E = E; p.R = (int)R; p.M = (int)R; p.N = N; p.K = K; p.seg = seg; p.C = C; p.ldc = ldc;
  p.out_fp32 = 0; p.accumulate = 0; p.b_mn = b_mn;
  p.num_m_blocks = (int)(R / BM); p.num_n_blocks = (N + BN - 1) / BN;
  p.status = xb_status_ptr();
  return launch(ta, tb, tc, p, (cudaStream_t)stream);
}

// A [R, M] (lda), B [R, N] (ldb), C [E, M, N] contiguous; C[e] (+)= A[seg[e]:seg[e+1]]^T @ B[same].
XB_API int xb_grouped_gemm_wgrad(const void* A, const void* B, void* C, const int* seg, int E,
                                 long long R, int M, int N, long long lda, long long ldb,
                                 int out_fp32, int accumulate, void* stream) {
  using namespace xb_ggemm;
  if (E <= 0) return 0;
  if (E > MAX_E || (lda % 8) || (ldb % 8) || (M % 8) || (N % 8)) return -1;
  CUtensorMap ta, tb;
  if (xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, M, lda, BK, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B)) return -2;
  if (xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, ldb, BK, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  Params p{};
  p.mode = 1; p.E = E; p.R = (int)R; p.M = M; p.N = N; p.K = 0; p.seg = seg; p.C = C; p.ldc = N;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.b_mn = 1;
  p.num_m_blocks = (M + BM - 1) / BM; p.num_n_blocks = (N + BN - 1) / BN;
  p.status = xb_status_ptr();
  return launch(ta, tb, ta, p, (cudaStream_t)stream);   // no output tensor map in wgrad mode
}
