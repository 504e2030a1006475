// Block-scaled fp8 (e4m3) GEMM and quantisation kernels for sm_100a.
//
//   xb_block_fp8_gemm     C[M,N] bf16 = sum_kb (A_kb B_kb^T) * sa[m,kb] * sb[n/128,kb]
//                         A [M,K] e4m3 with one fp32 scale per row and 128-wide K block,
//                         B [N,K] e4m3 with one fp32 scale per 128x128 block.
//   xb_quant_fp8_rows     bf16 [M,K]  -> e4m3 + 1x128 scales      (activations)
//   xb_quant_fp8_blocks   bf16 [N,K]  -> e4m3 + 128x128 scales    (weights)
//   xb_dequant_fp8_blocks e4m3 + 128x128 scales -> bf16
//
// The GEMM is a persistent warp-specialised kernel like the bf16 one, with BK = 128 fp8 elements
// (one 128-byte swizzle atom) so that one shared-memory stage is exactly one scale block.  The
// tensor core accumulates a single K block into one of two 128-column TMEM buffers
// (tcgen05.mma kind::f8f6f4, accumulate cleared at every block); the epilogue warps drain that
// buffer while the next block is being multiplied, apply sa*sb and add into fp32 registers --
// "promotion" of partial sums, which keeps fp32 scales of any magnitude exact without the power
// of two scale format the hardware block-scaled MMA needs.
// Counterparts in the reference: the Triton block-fp8 GEMM and quantisers
// (src/xorl/ops/quantize/block_fp8_quantize.py:155-203, fp8_kernels.py) and the quack block-scaled
// interface (src/xorl/ops/quack/gemm_blockscaled_interface.py).
#include <cuda_fp8.h>

#include "common.cuh"

namespace xb_fp8 {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 128;       // bytes == fp8 elements
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* sa;
  long long sa_ld;   // elements between consecutive rows of sa
  const float* sb;
  long long sb_ld;   // elements between consecutive 128-row blocks of sb
  int num_m_blocks, num_n_blocks, group_m;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& mb, int& nb) {
  const int per_group = p.group_m * p.num_n_blocks;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.num_m_blocks - first_m);
  const int t = tile - g * per_group;
  mb = first_m + t % gsz;
  nb = t / gsz;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int num_kb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 128);
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
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(p, tile, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, p.status, XB_K_FP8_GEMM, 100 + s)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          mbar_expect_tx(&bars->full[s], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &bars->full[s], kb * BK, mb * BM);
          tma_load_2d(sa + A_BYTES, &tmap_b, &bars->full[s], kb * BK, nb * BN);
        }
      }
      if (!ok) {
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
    if (lane == 0) {
      constexpr uint32_t idesc = xb_idesc(0, 0, BM, BN, 0, 0);   // e4m3 x e4m3 -> f32, both K-major
      constexpr uint64_t desc_base = xb_smem_desc_base_sw128(16, 1024);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const int buf = it & 1;
          if (!mbar_wait(&bars->acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status,
                         XB_K_FP8_GEMM, 200 + buf) ||
              !mbar_wait(&bars->full[s], (it / STAGES) & 1, abort_flag, p.status, XB_K_FP8_GEMM,
                         300 + s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = xb_smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            tc_mma_f8_ss(d_tmem, xb_smem_desc(desc_base, sa + k * UMMA_K),
                         xb_smem_desc(desc_base, sb + k * UMMA_K), idesc, k > 0 ? 1u : 0u);
          }
          tc_commit(&bars->empty[s]);
          tc_commit(&bars->acc_full[buf]);
        }
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    uint32_t it = 0;
    bool ok = true;
    const bool vec_ok = (p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mb, nb;
      tile_coords(p, tile, mb, nb);
      const int row = mb * BM + q * 32 + lane;
      const int rrow = row < p.M ? row : p.M - 1;
      const float* sa_row = p.sa + (long long)rrow * p.sa_ld;
      const float* sb_row = p.sb + (long long)nb * p.sb_ld;
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int buf = it & 1;
        const float scale = __ldg(sa_row + kb) * __ldg(sb_row + kb);
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->acc_full[buf], (it >> 1) & 1, abort_flag, p.status, XB_K_FP8_GEMM,
                       400 + buf))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(scale, __uint_as_float(r[j]), acc[c * 32 + j]);
        }
        tc_fence_before();
        mbar_arrive(&bars->acc_empty[buf]);
      }
      if (ok && row < p.M) {
        const int n0 = nb * BN;
        __nv_bfloat16* dst = p.C + (long long)row * p.ldc + n0;
        if (vec_ok && n0 + BN <= p.N) {
#pragma unroll
          for (int v = 0; v < BN / 8; ++v) {
            uint4 o;
            o.x = pack_bf16x2(acc[8 * v], acc[8 * v + 1]);
            o.y = pack_bf16x2(acc[8 * v + 2], acc[8 * v + 3]);
            o.z = pack_bf16x2(acc[8 * v + 4], acc[8 * v + 5]);
            o.w = pack_bf16x2(acc[8 * v + 6], acc[8 * v + 7]);
            *reinterpret_cast<uint4*>(dst + 8 * v) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < BN; ++j)
            if (n0 + j < p.N) dst[j] = __float2bfloat16(acc[j]);
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

// ---- quantisation -------------------------------------------------------------------------------
constexpr float FP8_MAX = 448.f;

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}

// one warp per (row, 128-wide block): lane owns 4 consecutive elements
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                  float* __restrict__ s, long long lds, int M, int KB) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)M * KB) return;
  const int row = (int)(w / KB), kb = (int)(w % KB);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (long long)row * ldx + kb * 128 + lane * 4);
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / FP8_MAX;
  const float inv = 1.f / scale;
  uint32_t out = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) |
                 ((uint32_t)to_e4m3(b.y * inv) << 24);
  *reinterpret_cast<uint32_t*>(q + (long long)row * ldq + kb * 128 + lane * 4) = out;
  if (lane == 0) s[(long long)row * lds + kb] = scale;
}

// one CTA (256 threads) per 128x128 block; edges are treated as zeros and not written
__global__ void __launch_bounds__(256)
quant_blocks_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, long long ldq,
                    float* __restrict__ s, long long lds, int N, int K) {
  const int nb = blockIdx.y, kb = blockIdx.x;
  const int t = threadIdx.x;
  const int c4 = (t & 31) * 4;          // column (4 elements) inside the block
  const int r0 = t >> 5;                // rows r0, r0+8, ...
  float v[16][4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int row = nb * 128 + r0 + 8 * i;
    const int col = kb * 128 + c4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f = 0.f;
      if (row < N && col + j < K) f = __bfloat162float(w[(long long)row * ldw + col + j]);
      v[i][j] = f;
      amax = fmaxf(amax, fabsf(f));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __shared__ float red[8];
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float scale = fmaxf(amax, 1e-12f) / FP8_MAX;
  const float inv = 1.f / scale;
  if (t == 0) s[(long long)nb * lds + kb] = scale;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int row = nb * 128 + r0 + 8 * i;
    const int col = kb * 128 + c4;
    if (row >= N) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (col + j < K) q[(long long)row * ldq + col + j] = to_e4m3(v[i][j] * inv);
  }
}

__global__ void __launch_bounds__(256)
dequant_blocks_kernel(const uint8_t* __restrict__ q, long long ldq, const float* __restrict__ s, long long lds,
                      __nv_bfloat16* __restrict__ w, long long ldw, int N, int K) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)N * K;
  for (long long i = idx; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / K), col = (int)(i % K);
    const float sc = s[(long long)(row >> 7) * lds + (col >> 7)];
    w[(long long)row * ldw + col] = __float2bfloat16(from_e4m3(q[(long long)row * ldq + col]) * sc);
  }
}

}  // namespace xb_fp8

// A [M,K] e4m3 (row stride lda bytes), B [N,K] e4m3 (row stride ldb bytes), K a multiple of 128,
// lda/ldb multiples of 16, both 16-byte aligned.  sa [M, K/128] (row stride sa_ld), sb
// [ceil(N/128), K/128] (row stride sb_ld).  C bf16 [M,N] with row stride ldc elements.
XB_API int xb_block_fp8_gemm_ex(const void* A, const void* B, void* C, const float* sa, const float* sb,
                                int M, int N, int K, long long lda, long long ldb, long long ldc,
                                long long sa_ld, long long sb_ld, void* stream) {
  using namespace xb_fp8;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % BK) || (lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) % 16) ||
      (reinterpret_cast<uintptr_t>(B) % 16))
    return -1;
  CUtensorMap ta, tb;
  if (xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, BK,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (xb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BN, BK,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.sa = sa; p.sa_ld = sa_ld;
  p.sb = sb; p.sb_ld = sb_ld;
  p.num_m_blocks = (M + BM - 1) / BM;
  p.num_n_blocks = (N + BN - 1) / BN;
  p.group_m = 16;
  p.status = xb_status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < xb_sm_count() ? tiles : xb_sm_count();
  fp8_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_block_fp8_gemm(const void* A, const void* B, void* C, const float* sa, const float* sb, int M,
                             int N, int K, void* stream) {
  return xb_block_fp8_gemm_ex(A, B, C, sa, sb, M, N, K, K, K, N, K / 128, K / 128, stream);
}

XB_API int xb_quant_fp8_rows(const void* x, long long ldx, void* q, long long ldq, float* s, long long lds,
                             int M, int K, void* stream) {
  if (K % 128 || ldx % 4 || ldq % 4 || (reinterpret_cast<uintptr_t>(x) % 8) ||
      (reinterpret_cast<uintptr_t>(q) % 4))
    return -1;
  const long long warps = (long long)M * (K / 128);
  if (warps == 0) return 0;
  const long long blocks = (warps * 32 + 255) / 256;
  xb_fp8::quant_rows_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<uint8_t*>(q), ldq, s, lds, M, K / 128);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_quant_fp8_blocks(const void* w, long long ldw, void* q, long long ldq, float* s, long long lds,
                               int N, int K, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  dim3 grid((K + 127) / 128, (N + 127) / 128);
  xb_fp8::quant_blocks_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(w), ldw, reinterpret_cast<uint8_t*>(q), ldq, s, lds, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_dequant_fp8_blocks(const void* q, long long ldq, const float* s, long long lds, void* w,
                                 long long ldw, int N, int K, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  const long long total = (long long)N * K;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  xb_fp8::dequant_blocks_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(q), ldq, s, lds, reinterpret_cast<__nv_bfloat16*>(w), ldw, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
