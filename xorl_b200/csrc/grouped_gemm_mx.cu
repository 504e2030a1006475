// Grouped (per-expert) block-scaled fp8 GEMM for MoE on the tcgen05 block-scaled tensor-core path.
//
//   C[rows of e, :] (bf16) = A[rows of e, :] @ B[e]^T
//     A  e4m3 [R, K]      one power-of-two scale per row and 128-wide K block   (1 x 128)
//     B  e4m3 [E, N, K]   one power-of-two scale per 128 x 128 block            (128 x 128)
//
// Scales are UE8M0 bytes (value 2^(b - 127)).  With power-of-two scales the products are scaled
// by the tensor core itself (`tcgen05.mma.kind::mxf8f6f4.block_scale`, one scale per operand row
// and 32-deep K block, read from tensor memory), so the accumulator of a tile stays in TMEM for
// the whole K loop -- no per-block promotion through registers as in the fp32-scale kernel of
// quant.cu -- and the main loop runs at the fp8 rate.  A 1 x 128 (128 x 128) scale is presented to
// the hardware as four equal 1 x 32 scales (the same byte for every row of the block).
//
// Roles of a CTA (320 threads, one 128 x 192 output tile at a time, persistent):
//   warp 0      TMA producer: A [128 x 128 B] and B [192 x 128 B] per stage, 5-stage ring
//   warp 1      MMA issuer: 4 block-scaled MMAs (K = 32) per stage into one of two TMEM accumulators
//   warps 2-5   epilogue: TMEM -> registers -> bf16 in a 128B-swizzled shared-memory slab (128 rows x 64
//               columns) -> one TMA store per slab, so global memory sees full 128-byte row segments
//   warps 6-9   scale warps: keep the tile's scale bytes for 16 K blocks at a time in registers (rows of
//               the scale arrays are padded to 16 bytes, one vector load per row) and, per stage,
//               write them into that stage's TMEM scale slot with tcgen05.st
// Scale layout in TMEM (found by measurement: a probe against a CPU restatement): for an operand
// row r, lane 32 q + (r % 32) of every lane quarter q, column base + r / 32, byte i = scale of the
// i-th 32-deep K block of the stage; the instruction descriptor's a_sf_id / b_sf_id pick the byte.
//
// The quantisers at the end of the file produce these operands: rows (activations) and stacked
// expert weights in both orientations ([E, N, K] for forward, [E, K, N] for the input gradient).
// Counterparts in the reference: src/xorl/fp8_training/grouped.py:116-330 (Triton, fp32 scales).
#include <cuda_fp8.h>

#include "common.cuh"

namespace xb_ggemm_mx {

constexpr int BM = 128, BN = 192, BK = 128, UMMA_K = 32, STAGES = 5;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int ACC_COLS = BN;                 // two accumulators: columns [0, 192) and [192, 384)
constexpr int SF_BASE = 2 * ACC_COLS;        // scale slots from column 384
constexpr int SF_SLOT = 12;                  // per stage: 4 columns for A, 8 (6 used) for B
constexpr int MAX_E = 512;
constexpr int SLAB_COLS = 64;                // epilogue staging: one 128-row x 64-column bf16 slab (16 KB)
constexpr int SLAB_BYTES = BM * SLAB_COLS * 2;
constexpr int OFF_SLAB = STAGES * STAGE_BYTES;
constexpr int OFF_BARS = OFF_SLAB + SLAB_BYTES;
constexpr int OFF_SEG = OFF_BARS + 256;
constexpr int SMEM_BYTES = OFF_SEG + (MAX_E + 1) * 4 + 1024;

struct Params {
  int E, R, N, K;
  const int* seg;
  const uint8_t* sfa;      // [R, sfa_ld]               row strides: multiples of 16 >= K/128
  const uint8_t* sfb;      // [E, ceil(N/128), sfb_ld]
  int sfa_ld, sfb_ld;
  __nv_bfloat16* C;
  long long ldc;
  int num_m_blocks, num_n_blocks;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Tile {
  int e, m0, n0;
  bool valid;
};

// Tiles are walked in groups of GROUP_M row blocks: inside a group all row blocks of one column block,
// then the next column block.  The CTAs running at any time then share a few B tiles and one group of A
// rows (a few MB, resident in L2) instead of streaming all of A once per column block.
constexpr int GROUP_M = 16;

__device__ __forceinline__ Tile get_tile(const Params& p, const int* sseg, int t) {
  Tile r;
  const int per_group = GROUP_M * p.num_n_blocks;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, p.num_m_blocks - first_m);
  const int u = t - g * per_group;
  const int mb = first_m + u % gsz, nb = u / gsz;
  r.m0 = mb * BM;
  r.n0 = nb * BN;
  int e = -1;
  for (int i = 0; i < p.E; ++i)
    if (r.m0 >= sseg[i] && r.m0 < sseg[i + 1]) { e = i; break; }
  r.e = e;
  r.valid = e >= 0;
  return r;
}

// D[tmem] (+)= (A * sfa) (B * sfb)^T, e4m3 operands in shared memory, UE8M0 scales in tensor memory.
__device__ __forceinline__ void mma_mx(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, uint32_t a, uint32_t b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
// byte i (0..15) of a 16-byte vector, replicated into all four bytes of a word
__device__ __forceinline__ uint32_t rep_byte(const uint4& v, int i) {
  const int w = i >> 2;
  const uint32_t x = w == 0 ? v.x : (w == 1 ? v.y : (w == 2 ? v.z : v.w));
  return 0x01010101u * ((x >> ((i & 3) * 8)) & 0xffu);
}

// Block-scaled instruction descriptor: e4m3 x e4m3 (formats 0), both K-major, N >> 3 at bit 17, UE8M0
// scale format at bit 23, M >> 4 at bit 24; b_sf_id at bit 4 and a_sf_id at bit 29 are added per MMA.
__host__ __device__ constexpr uint32_t mx_idesc(int m, int n) {
  return ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
ggemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + OFF_BARS);
  int* sseg = reinterpret_cast<int*>(smem + OFF_SEG);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int num_kb = p.K / BK;
  const int NB = (p.N + 127) / 128;
  for (int i = threadIdx.x; i <= p.E; i += NUM_THREADS) sseg[i] = p.seg[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->full[s], 5); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->tmem_full[a], 1); mbar_init(&bars->tmem_empty[a], 128); }
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------ TMA producer -------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = get_tile(p, sseg, t);
        if (!tl.valid) continue;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&bars->empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.status, XB_K_GROUPED_GEMM,
                         100 + s)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          mbar_expect_tx(&bars->full[s], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &bars->full[s], kb * BK, tl.m0);
          tma_load_3d(sa + A_BYTES, &tmap_b, &bars->full[s], kb * BK, tl.n0, tl.e);
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
    // ------------------------------------ MMA issuer ---------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc0 = mx_idesc(BM, BN);
      constexpr uint64_t desc_base = xb_smem_desc_base_sw128(16, 1024);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = get_tile(p, sseg, t);
        if (!tl.valid) continue;
        const int acc = tcount & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], ((tcount >> 1) & 1) ^ 1, abort_flag, p.status, XB_K_GROUPED_GEMM,
                       200 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&bars->full[s], (it / STAGES) & 1, abort_flag, p.status, XB_K_GROUPED_GEMM, 300 + s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = xb_smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
          const uint32_t sfa_t = tmem_base + SF_BASE + s * SF_SLOT, sfb_t = sfa_t + 4;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            mma_mx(d_tmem, xb_smem_desc(desc_base, sa + k * UMMA_K), xb_smem_desc(desc_base, sb + k * UMMA_K),
                   idesc0 | ((uint32_t)k << 4) | ((uint32_t)k << 29), sfa_t, sfb_t, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->empty[s]);
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
        ++tcount;
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------ epilogue -----------------------------------------
    const int q = warp & 3;
    uint8_t* slab = smem + OFF_SLAB;
    uint32_t tcount = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile tl = get_tile(p, sseg, t);
      if (!tl.valid) continue;
      const int acc = tcount & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[acc], (tcount >> 1) & 1, abort_flag, p.status,
                                             XB_K_GROUPED_GEMM, 400 + acc))) { ok = false; break; }
      tc_fence_after();
      const int r = q * 32 + lane;                          // row of the tile held by this thread
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      uint8_t* srow = slab + r * 128;
#pragma unroll 1
      for (int sl = 0; sl < BN / SLAB_COLS; ++sl) {
        const int col0 = tl.n0 + sl * SLAB_COLS;
        if (col0 >= p.N) break;                             // uniform over the CTA
        uint32_t v[2][32];
        tmem_ld_32x32(taddr + sl * SLAB_COLS, v[0]);
        tmem_ld_32x32(taddr + sl * SLAB_COLS + 32, v[1]);
        tc_wait_ld();
        // the previous slab's TMA store must have read the staging buffer
        if (warp == 2 && lane == 0) tma_store_wait_read<0>();
        epi_sync();
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
        epi_sync();
        if (warp == 2 && lane == 0) {
          tma_store_2d(&tmap_c, slab, col0, tl.m0);
          tma_store_commit();
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->tmem_empty[acc]);
      ++tcount;
    }
    if (warp == 2 && lane == 0) tma_store_wait<0>();        // global writes complete before the CTA exits
  } else {
    // ------------------------------------ scale warps --------------------------------------
    const int q = warp & 3;                  // lane quarter of tensor memory this warp may write
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile tl = get_tile(p, sseg, t);
      if (!tl.valid) continue;
      const int sub = tl.n0 & 127;           // offset of the tile inside its first 128-column block
      const int nb0 = tl.n0 >> 7;
      const int nb1 = min(nb0 + 1, NB - 1);
      const uint8_t* b0p = p.sfb + ((long long)tl.e * NB + nb0) * p.sfb_ld;
      const uint8_t* b1p = p.sfb + ((long long)tl.e * NB + nb1) * p.sfb_ld;
      uint4 va[4], vb0, vb1;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((kb & 15) == 0) {
          // scales of the next 16 K blocks: rows lane, 32 + lane, 64 + lane, 96 + lane of the tile
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = min(tl.m0 + j * 32 + lane, p.R - 1);
            va[j] = __ldg(reinterpret_cast<const uint4*>(p.sfa + (long long)row * p.sfa_ld + kb));
          }
          vb0 = __ldg(reinterpret_cast<const uint4*>(b0p + kb));
          vb1 = __ldg(reinterpret_cast<const uint4*>(b1p + kb));
        }
        const int s = it % STAGES;
        int got = 1;
        if (lane == 0)
          got = mbar_wait(&bars->empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.status, XB_K_GROUPED_GEMM, 500 + s);
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        tc_fence_after();
        const int i = kb & 15;
        const uint32_t b0 = rep_byte(vb0, i), b1 = rep_byte(vb1, i);
        uint32_t wb[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) wb[j] = (sub + j * 32) < 128 ? b0 : b1;
        const uint32_t slot = tmem_base + SF_BASE + s * SF_SLOT + ((uint32_t)(q * 32) << 16);
        tmem_st4(slot, rep_byte(va[0], i), rep_byte(va[1], i), rep_byte(va[2], i), rep_byte(va[3], i));
        tmem_st4(slot + 4, wb[0], wb[1], wb[2], wb[3]);
        tmem_st2(slot + 8, wb[4], wb[5]);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->full[s]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------
// quantisers (power-of-two scales)
// ------------------------------------------------------------------------------------------------
constexpr float FP8_MAX = 448.f;

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
// Smallest power of two s with amax / s <= 448, as a UE8M0 byte (127 -> 1.0); inv = 1 / s.
__device__ __forceinline__ uint8_t pow2_scale(float amax, float& inv) {
  int e = -127;
  if (amax > 0.f) {
    int ex;
    const float m = frexpf(amax / FP8_MAX, &ex);      // amax / 448 = m * 2^ex, m in [0.5, 1)
    e = (m == 0.5f) ? ex - 1 : ex;
    e = max(-126, min(126, e));
  } else {
    e = 0;
  }
  inv = exp2f((float)-e);
  return (uint8_t)(e + 127);
}

// One warp per row; a pass covers 256 elements (two scale blocks): lane owns 8 consecutive elements
// (one 16-byte load, one 8-byte store), the block maximum is taken over 16 lanes.
__global__ void __launch_bounds__(256)
quant_mx_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                     uint8_t* __restrict__ sf, int sf_ld, long long M, int KB, const int* __restrict__ row_limit) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row_limit != nullptr) M = min(M, (long long)*row_limit);
  if (row >= M) return;
  const __nv_bfloat16* xr = x + row * ldx;
  uint8_t* qr = q + row * ldq;
  const int K = KB * 128;
#pragma unroll 4
  for (int k0 = 0; k0 < K; k0 += 256) {
    const int k = k0 + lane * 8;
    const bool in = k < K;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (in) raw = *reinterpret_cast<const uint4*>(xr + k);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
    float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                       fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float inv;
    const uint8_t byte = pow2_scale(amax, inv);
    if (in) {
      uint2 out;
      out.x = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) | ((uint32_t)to_e4m3(b.y * inv) << 24);
      out.y = to_e4m3(c.x * inv) | (to_e4m3(c.y * inv) << 8) | (to_e4m3(d.x * inv) << 16) | ((uint32_t)to_e4m3(d.y * inv) << 24);
      *reinterpret_cast<uint2*>(qr + k) = out;
      if ((lane & 15) == 0) sf[row * sf_ld + (k >> 7)] = byte;
    }
  }
}

// One CTA per 128 x 128 block of one expert's weight W[e] [K, N] (N contiguous): writes the block
// quantised in place order (q_kn [E, K, N], scales [E, K/128, N/128]) and transposed
// (q_nk [E, N, K], scales [E, N/128, K/128]).
__global__ void __launch_bounds__(256)
quant_mx_weight_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q_kn, uint8_t* __restrict__ sf_kn,
                       int ld_kn, uint8_t* __restrict__ q_nk, uint8_t* __restrict__ sf_nk, int ld_nk, int K, int N) {
  __shared__ uint8_t tile[128][132];
  __shared__ float red[8];
  const int nb = blockIdx.x, kb = blockIdx.y, e = blockIdx.z;
  const int KB = K / 128, NB = N / 128;
  const int t = threadIdx.x;
  const int c4 = (t & 31) * 4, r0 = t >> 5;
  const __nv_bfloat16* src = w + ((long long)e * K + (long long)kb * 128) * N + (long long)nb * 128;
  float v[16][4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + (long long)(r0 + 8 * i) * N + c4);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    v[i][0] = a.x; v[i][1] = a.y; v[i][2] = b.x; v[i][3] = b.y;
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
  }
  amax = warp_max(amax);
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  float inv;
  const uint8_t byte = pow2_scale(amax, inv);
  if (t == 0) {
    sf_kn[((long long)e * KB + kb) * ld_kn + nb] = byte;
    sf_nk[((long long)e * NB + nb) * ld_nk + kb] = byte;
  }
  uint8_t* dkn = q_kn + ((long long)e * K + (long long)kb * 128) * N + (long long)nb * 128;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = r0 + 8 * i;
    const uint8_t q0 = to_e4m3(v[i][0] * inv), q1 = to_e4m3(v[i][1] * inv), q2 = to_e4m3(v[i][2] * inv),
                  q3 = to_e4m3(v[i][3] * inv);
    *reinterpret_cast<uint32_t*>(dkn + (long long)r * N + c4) = q0 | (q1 << 8) | (q2 << 16) | ((uint32_t)q3 << 24);
    tile[r][c4] = q0; tile[r][c4 + 1] = q1; tile[r][c4 + 2] = q2; tile[r][c4 + 3] = q3;
  }
  __syncthreads();
  // transposed write: output row n (of this block), 128 contiguous k bytes
  uint8_t* dnk = q_nk + ((long long)e * N + (long long)nb * 128) * K + (long long)kb * 128;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int n = r0 + 8 * i;
    const uint32_t o = tile[c4][n] | (tile[c4 + 1][n] << 8) | (tile[c4 + 2][n] << 16) | ((uint32_t)tile[c4 + 3][n] << 24);
    *reinterpret_cast<uint32_t*>(dnk + (long long)n * K + c4) = o;
  }
}

}  // namespace xb_ggemm_mx

// A e4m3 [R, K] (row stride lda bytes), sfa UE8M0 [R, sfa_ld]; B e4m3 [E, N, K] contiguous, sfb UE8M0
// [E, ceil(N/128), sfb_ld]; the scale row strides are multiples of 16 >= K/128 (arrays 16-byte aligned);
// C bf16 [R, N] (row stride ldc elements); seg int32 [E+1] with 128-aligned entries and seg[E] <= R.
// K a multiple of 128, N a multiple of 16.
XB_API int xb_grouped_gemm_mx_rows(const void* A, const void* sfa, const void* B, const void* sfb, void* C,
                                   const int* seg, int E, long long R, int N, int K, long long lda,
                                   long long ldc, int sfa_ld, int sfb_ld, void* stream) {
  using namespace xb_ggemm_mx;
  if (E <= 0 || R <= 0) return 0;
  if (E > MAX_E || (R % BM) || (lda % 16) || (K % BK) || (N % 16) || (sfa_ld % 16) || sfa_ld < K / BK ||
      (sfb_ld % 16) || sfb_ld < K / BK ||
      (reinterpret_cast<uintptr_t>(sfa) % 16) || (reinterpret_cast<uintptr_t>(sfb) % 16))
    return -1;
  if ((ldc % 8) || (reinterpret_cast<uintptr_t>(C) % 16)) return -1;
  CUtensorMap ta, tb, tc;
  if (xb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, R, K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (xb_make_tmap_2d(&tc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, ldc, BM, SLAB_COLS, CU_TENSOR_MAP_SWIZZLE_128B))
    return -4;
  if (xb_make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, E, N, K, (uint64_t)K * N, K, 1, BN, BK,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  Params p{};
  p.E = E; p.R = (int)R; p.N = N; p.K = K; p.seg = seg;
  p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.sfa_ld = sfa_ld; p.sfb_ld = sfb_ld;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc;
  p.num_m_blocks = (int)(R / BM); p.num_n_blocks = (N + BN - 1) / BN;
  p.status = xb_status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(ggemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -10;
    configured[dev & 63] = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < xb_sm_count() ? tiles : xb_sm_count();
  ggemm_mx_kernel<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, tc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// x bf16 [M, K] (row stride ldx elements) -> q e4m3 [M, K] (row stride ldq bytes) + UE8M0 scales [M, sf_ld]
// (bytes K/128 .. sf_ld - 1 of a scale row are left as they are).
XB_API int xb_quant_mx_rows_lim(const void* x, long long ldx, void* q, long long ldq, void* sf, int sf_ld,
                                long long M, int K, const int* row_limit, void* stream);

XB_API int xb_quant_mx_rows(const void* x, long long ldx, void* q, long long ldq, void* sf, int sf_ld, long long M,
                            int K, void* stream) {
  return xb_quant_mx_rows_lim(x, ldx, q, ldq, sf, sf_ld, M, K, nullptr, stream);
}

// row_limit (optional, device memory): only the first *row_limit rows are quantised.
XB_API int xb_quant_mx_rows_lim(const void* x, long long ldx, void* q, long long ldq, void* sf, int sf_ld,
                                long long M, int K, const int* row_limit, void* stream) {
  if (M <= 0) return 0;
  if ((K % 128) || (ldx % 8) || (ldq % 8) || sf_ld < K / 128 || (reinterpret_cast<uintptr_t>(x) % 16) ||
      (reinterpret_cast<uintptr_t>(q) % 8))
    return -1;
  const int KB = K / 128;
  const long long blocks = (M + 7) / 8;
  xb_ggemm_mx::quant_mx_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (uint8_t*)sf, sf_ld, M, KB, row_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// w bf16 [E, K, N] -> q_kn e4m3 [E, K, N] + sf_kn [E, K/128, ld_kn], q_nk e4m3 [E, N, K] + sf_nk [E, N/128, ld_nk]
// (ld_kn >= N/128, ld_nk >= K/128: row strides of the scale arrays, multiples of 16 for the GEMM).
XB_API int xb_quant_mx_weight(const void* w, void* q_kn, void* sf_kn, int ld_kn, void* q_nk, void* sf_nk, int ld_nk,
                              int E, int K, int N, void* stream) {
  if (E <= 0) return 0;
  if ((K % 128) || (N % 128) || ld_kn < N / 128 || ld_nk < K / 128) return -1;
  dim3 grid(N / 128, K / 128, E);
  xb_ggemm_mx::quant_mx_weight_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)w, (uint8_t*)q_kn, (uint8_t*)sf_kn, ld_kn, (uint8_t*)q_nk, (uint8_t*)sf_nk, ld_nk, K, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
