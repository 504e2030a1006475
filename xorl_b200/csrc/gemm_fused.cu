// bf16 GEMM on CTA pairs with the collective of one operand, or of the result, in the same kernel.
//
//   gather  (all-gather -> GEMM):  one operand is sharded by rows over the ranks (sequence-parallel
//           activations of a tensor-parallel column linear, or a row-sharded ZeRO-3 weight).  Four
//           extra warps per CTA pull the peers' shards into this rank's full copy with plain 16-byte
//           loads over NVLink (16 in flight per thread), one chunk of tile rows at a time and all
//           CTAs on the same chunk, and count each finished chunk in global memory.  The TMA warp
//           waits for the chunk that its next work item reads and then loads it from local memory,
//           so every remote byte crosses NVLink once and the tensor cores run on the chunks that
//           have already arrived.  Work items and chunks are walked in the same order, starting at
//           this rank's own rows.
//   scatter (GEMM -> reduce-scatter):  the rows of the result are owned by the ranks in equal
//           blocks.  Every rank writes its partial result into its own symmetric buffer with the
//           ordinary epilogue (local, coalesced by the memory system), computing the blocks in the
//           order rank+1, rank+2, ..., own block last; warps count the finished 32-row x 128-column
//           units per owner, and the warp that completes an owner's block signals that owner with a
//           release store.  Meanwhile the communication warps of the owner wait for those signals
//           in the order in which the peers finish (rank-1 first) and pull each peer's partial block
//           over NVLink into local staging, so the transfers overlap the remaining tiles.  At the
//           end all CTAs sum the own partial block and the pulled ones in fp32, in rank order
//           (+ an optional residual), into the output.
//
// This is the kernel behind tensor-parallel linears with sequence-parallel activations: the
// reference runs them as DTensor collectives followed / preceded by cuBLAS
// (src/xorl/distributed/torch_parallelize.py:222-270) and its FSDP2 parameter gather as a separate
// NCCL all-gather (src/xorl/distributed/torch_parallelize.py:333-783).
//
// Handshakes use epoch flags in each rank's symmetric flag area (st.release.sys / ld.acquire.sys),
// every wait is bounded by %globaltimer, and with null flag pointers the gather and the partial-
// result paths run on one device (all "peers" are local buffers), which is how they are tested on
// a single GPU.
#include "gemm2_core.cuh"

namespace xb_gemmf {
using namespace xb_gemm2;

constexpr int MAX_R = 16;
constexpr int COMM_THREADS = 128;                   // warps 10 to 13
constexpr int COPY_UNROLL = 16;                     // 16-byte loads in flight per communication thread
constexpr int NT = NUM_THREADS + COMM_THREADS;
constexpr int EPI_THREADS = 256;
constexpr int MAX_SUB = 16;                         // sub-blocks of an owner's rows, signalled one by one

struct Comm {
  int rank, nranks;
  int gather;                    // 0: none, 1: rows of A, 2: rows of B come from the ranks' shards
  int scatter;                   // 1: rows of the result go to their owners
  int rot_m, rot_n;              // rotation of the tile raster (own rows first / last)
  // ---- gather
  const uint4* shard[MAX_R];     // rank r's rows of the gathered operand (contiguous rows of K)
  uint4* full;                   // this rank's full copy (what the tensor map reads)
  long long shard_vec;           // 16-byte vectors per shard
  long long total_vec;           // vectors of the whole operand
  long long chunk_vec;           // vectors per chunk of tile rows
  int num_chunks, chunk0;
  unsigned long long* ready;     // [num_chunks] arrival counters (monotonic)
  unsigned long long ready_target;
  // ---- scatter
  const __nv_bfloat16* partial[MAX_R];   // rank r's partial result [M][N] (this rank's one is p.C)
  __nv_bfloat16* pulled;         // local staging [nranks][rows_per][N] for the peers' partial blocks
  int rows_per;                  // result rows owned by one rank (multiple of 32)
  __nv_bfloat16* out;            // this rank's reduced rows [rows_per][ldo]; null: partial result only
  long long ldo;
  const __nv_bfloat16* residual; // optional, added to the reduced rows
  int* counters;                 // [nranks][MAX_SUB] units, [1] epilogue CTAs, [1] copy CTAs; zero on entry/exit
  int sub_rows, num_sub;         // an owner's rows are signalled in num_sub pieces of sub_rows rows
  int units_per_sub;
  // ---- flags (null: single-device run without handshakes)
  int* flags[MAX_R];
  int ready_slot, done_slot;
  int epoch, done_needed;
  unsigned long long limit_ns;
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* addr) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_u64(unsigned long long* addr, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void named_bar(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Bounded wait for an epoch flag; returns false (after recording the status) on expiry.
__device__ __forceinline__ bool wait_flag(const int* addr, int epoch, int* status, int detail,
                                          unsigned long long limit_ns) {
  if (ld_acquire_sys(addr) >= epoch) return true;
  const uint64_t t0 = xb_globaltimer();
  for (uint32_t it = 1;; ++it) {
    __nanosleep(64);
    if (ld_acquire_sys(addr) >= epoch) return true;
    if ((it & 127u) == 0u && xb_globaltimer() - t0 > limit_ns) {
      xb_report(status, XB_ERR_FLAG_TIMEOUT, XB_K_AG_GEMM, detail);
      return false;
    }
  }
}

__device__ __forceinline__ Item decode_rot(const Params& p, const Comm& c, int w) {
  Item it = decode_item(p, w);
  if (c.rot_m) {
    const int mb = it.m0 / 512;
    it.m0 += (((mb + c.rot_m) % p.num_m_blocks) - mb) * 512;
  }
  if (c.rot_n) {
    const int nb = it.n0 / BN;
    it.n0 += (((nb + c.rot_n) % p.num_n_blocks) - nb) * BN;
  }
  return it;
}

// dst[lo, hi) = src[lo, hi) in 16-byte vectors, this thread taking every stride-th one from `first`.
// Up to COPY_UNROLL loads are in flight per thread, also in the last, partial batch (a chunk of tile
// rows is only a dozen strides of the whole grid long).
__device__ __forceinline__ void copy_span(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                          long long lo, long long hi, long long first, long long stride) {
  for (long long i = lo + first; i < hi; i += COPY_UNROLL * stride) {
    uint4 v[COPY_UNROLL];
#pragma unroll
    for (int k = 0; k < COPY_UNROLL; ++k)
      if (i + k * stride < hi) v[k] = src[i + k * stride];
#pragma unroll
    for (int k = 0; k < COPY_UNROLL; ++k)
      if (i + k * stride < hi) dst[i + k * stride] = v[k];
  }
}

// out = sum over ranks of src[r] (each a contiguous [rows_per][N] block), fp32 in rank order,
// optional residual.
struct BlockSources {
  const uint4* p[MAX_R];
};
__device__ __forceinline__ void acc8(float (&acc)[8], const uint4 v) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), d = unpack_bf16x2(v.z), e = unpack_bf16x2(v.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += d.x; acc[5] += d.y; acc[6] += e.x; acc[7] += e.y;
}
__device__ __forceinline__ void reduce_rows(const BlockSources& src, int nranks, int rows_per, int N,
                                            __nv_bfloat16* out, long long ldo, const __nv_bfloat16* residual,
                                            long long first, long long stride) {
  constexpr int U = 4;      // vectors per thread and step: U loads in flight for every rank
  const long long row_vec = N >> 3;
  const long long nvec = (long long)rows_per * row_vec;
  for (long long i0 = first; i0 < nvec; i0 += U * stride) {
    float acc[U][8];
#pragma unroll
    for (int k = 0; k < U; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
    for (int r = 0; r < nranks; ++r) {
      const uint4* sp = src.p[r];
      uint4 v[U];
#pragma unroll
      for (int k = 0; k < U; ++k)
        if (i0 + k * stride < nvec) v[k] = sp[i0 + k * stride];
#pragma unroll
      for (int k = 0; k < U; ++k)
        if (i0 + k * stride < nvec) acc8(acc[k], v[k]);
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const long long i = i0 + k * stride;
      if (i >= nvec) break;
      const long long row = i / row_vec;
      const long long col = (i - row * row_vec) << 3;
      if (residual != nullptr) acc8(acc[k], *reinterpret_cast<const uint4*>(residual + row * ldo + col));
      uint4 o;
      o.x = pack_bf16x2(acc[k][0], acc[k][1]);
      o.y = pack_bf16x2(acc[k][2], acc[k][3]);
      o.z = pack_bf16x2(acc[k][4], acc[k][5]);
      o.w = pack_bf16x2(acc[k][6], acc[k][7]);
      *reinterpret_cast<uint4*>(out + row * ldo + col) = o;
    }
  }
}

// Last phase of the scatter path, run by the epilogue and the communication warps of every CTA:
// wait (bounded) until this rank's own block is complete on all CTAs and all CTAs have pulled the
// peers' blocks, then sum.  `slot`: this thread's index among all reducing threads of the grid.
__device__ __forceinline__ void scatter_reduce(const Params& p, const Comm& c, int lane, long long slot) {
  if (lane == 0) {
    bool good = true;
    for (int sb = 0; sb < c.num_sub && good; ++sb)
      good = wait_flag(c.flags[c.rank] + c.ready_slot + c.rank * MAX_SUB + sb, c.epoch, p.status, 3000, c.limit_ns);
    if (good && ld_acquire_gpu_u64(c.ready) < c.ready_target) {
      const uint64_t t0 = xb_globaltimer();
      for (uint32_t spin = 1;; ++spin) {
        __nanosleep(100);
        if (ld_acquire_gpu_u64(c.ready) >= c.ready_target) break;
        if ((spin & 63u) == 0u && xb_globaltimer() - t0 > c.limit_ns) {
          xb_report(p.status, XB_ERR_FLAG_TIMEOUT, XB_K_AG_GEMM, 3001);
          break;
        }
      }
    }
  }
  __syncwarp();
  const long long blk = (long long)c.rows_per * p.N;
  BlockSources src;
  for (int r = 0; r < c.nranks; ++r)
    src.p[r] = reinterpret_cast<const uint4*>(r == c.rank ? c.partial[r] + (long long)c.rank * blk
                                                           : c.pulled + (long long)r * blk);
  reduce_rows(src, c.nranks, c.rows_per, p.N, c.out, c.ldo, c.residual, slot,
              (long long)gridDim.x * (EPI_THREADS + COMM_THREADS));
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NT, 1)
gemm_fused_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_b64, const Params p, const Comm c) {
  constexpr bool A_MN = false;
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
  const int num_kb = (p.K + BK - 1) / BK;
  const bool linked = c.flags[0] != nullptr;       // real peers (handshakes) or one device

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
        const Item item = decode_rot(p, c, w);
        const int m0 = item.m0 + (int)cta * BM;              // sub-tile u adds 256 * u
        const int bcols = item.ncols / 2;                     // B columns loaded by this CTA
        const int n0 = item.n0 + (int)cta * bcols;
        const uint32_t stage_tx = 2u * (uint32_t)(item.nsub * A_BYTES + bcols * BK * 2);
        if (c.gather) {
          // the rows this item reads must have arrived in the local full copy
          const int ch = c.gather == 1 ? item.m0 / 512 : item.n0 / BN;
          const unsigned long long* flag = c.ready + ch;
          if (ld_acquire_gpu_u64(flag) < c.ready_target) {
            const uint64_t t0 = xb_globaltimer();
            for (uint32_t spin = 1;; ++spin) {
              __nanosleep(100);
              if (ld_acquire_gpu_u64(flag) >= c.ready_target) break;
              if ((spin & 63u) == 0u) {
                if (*abort_flag) { ok = false; break; }
                if (xb_globaltimer() - t0 > c.limit_ns) {
                  *abort_flag = 1;
                  xb_report(p.status, XB_ERR_FLAG_TIMEOUT, XB_K_AG_GEMM, 1000 + ch);
                  ok = false;
                  break;
                }
              }
            }
            if (!ok) break;
          }
          fence_proxy_async();   // the copy warps wrote with ordinary stores, TMA reads them
        }
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
            tma_load_2d_pair(sa + u * A_BYTES, &tmap_a, full_leader, k0, m0 + 256 * u);
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
        // no bulk copy may still be in flight into shared memory when the CTAs exit
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
      constexpr uint64_t a_base = xb_smem_desc_base_sw128(16, 1024);
      constexpr uint64_t b_base = B_MN ? xb_smem_desc_base_sw128(BK * 128, 1024)
                                       : xb_smem_desc_base_sw128(16, 1024);
      constexpr uint32_t a_kstep = UMMA_K * 2;
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      const uint32_t bars_local = xb_smem_u32(bars);
      const uint32_t off0 = mapa_u32(bars_local, 0) - bars_local;
      const uint32_t off1 = mapa_u32(bars_local, 1) - bars_local;
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      for (int w = pair; w < p.num_items && ok; w += num_pairs, ++tcount) {
        const Item item = decode_rot(p, c, w);
        constexpr uint32_t idesc256 = xb_idesc(1, 1, 256, 256, 0, B_MN ? 1 : 0);
        constexpr uint32_t idesc128 = xb_idesc(1, 1, 256, 128, 0, B_MN ? 1 : 0);
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
  } else if (warp < 10) {
    // --------------- epilogue (both CTAs; warps 2-5 sub-tile 0, warps 6-9 sub-tile 1) ----------
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int u = (warp - 2) >> 2;          // sub-tile drained by this warp
    const int etid = threadIdx.x - 64;      // 0..255
    uint32_t tcount = 0;
    bool ok = true;
    const bool vec_ok = p.out_fp32
                            ? ((p.ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0)
                            : ((p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) % 16) == 0);
    if (c.scatter) {
      // the owners must have finished pulling what an earlier call left in this partial buffer
      if (linked && etid < c.nranks && etid != c.rank && c.done_needed > 0)
        wait_flag(c.flags[c.rank] + c.done_slot + etid, c.done_needed, p.status, 2000 + etid, c.limit_ns);
      named_bar(2, EPI_THREADS);
    }
    for (int w = pair; w < p.num_items && ok; w += num_pairs, ++tcount) {
      const Item item = decode_rot(p, c, w);
      if (!mbar_wait_warp(&bars->tmem_full, tcount & 1, abort_flag, p.status, 400 + u)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t empty_leader = mapa_u32(xb_smem_u32(&bars->tmem_empty[u]), 0);
      const int row = item.m0 + 256 * u + (int)cta * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + u * BN + ((uint32_t)(q * 32) << 16);
      const int nchunks = u < item.nsub ? item.ncols / 32 : 0;
      __nv_bfloat16* crow_bf = nullptr;
      float* crow_f = nullptr;
      if (row < p.M) {
        if (p.out_fp32) crow_f = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc;
        else crow_bf = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc;
      }
#pragma unroll 1
      for (int ch = 0; ch < nchunks; ++ch) {
        const int col0 = item.n0 + ch * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + ch * 32, r);
        tc_wait_ld();
        if (row < p.M) {
          if (crow_f != nullptr) {
            float* dst = crow_f + col0;
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
            __nv_bfloat16* dst = crow_bf + col0;
            const bool acc = p.accumulate != 0;
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * v + j]);
                if (acc) {
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
                  if (acc) o += __bfloat162float(dst[j]);
                  dst[j] = __float2bfloat16(o);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(empty_leader);
      if (c.scatter) {
        // count the finished 32-row x 128-column units per owner, warp by warp (no CTA-wide
        // barrier inside the loop: warps may leave it at different items after an abort); the
        // warp that completes an owner's block tells that owner that it may pull the block
        __threadfence_system();
        __syncwarp();
        const int row0 = item.m0 + 256 * u + (int)cta * BM + q * 32;
        if (lane == 0 && nchunks > 0 && row0 < p.M) {
          const int o = row0 / c.rows_per;
          const int sb = (row0 - o * c.rows_per) / c.sub_rows;
          const int units = item.ncols / 128;
          if (atomicAdd(c.counters + o * MAX_SUB + sb, units) + units == c.units_per_sub) {
            __threadfence_system();
            if (linked) st_release_sys(c.flags[o] + c.ready_slot + c.rank * MAX_SUB + sb, c.epoch);
          }
        }
      }
    }
    if (c.scatter && c.out != nullptr) {
      scatter_reduce(p, c, lane, blockIdx.x * (EPI_THREADS + COMM_THREADS) + etid);
    }
    if (c.scatter) {
      // the last CTA to get here clears the unit counters for the next call
      __threadfence();
      named_bar(2, EPI_THREADS);
      if (etid == 0) {
        int* cta_count = c.counters + c.nranks * MAX_SUB;
        if (atomicAdd(cta_count, 1) == (int)gridDim.x - 1) {
          __threadfence();
          for (int i = 0; i <= c.nranks * MAX_SUB; ++i) c.counters[i] = 0;
        }
      }
    }
  } else {
    // ------------------------------- communication warps --------------------------------
    const int ctid = threadIdx.x - NUM_THREADS;     // 0..127
    const long long stride = (long long)gridDim.x * COMM_THREADS;
    const long long first = (long long)blockIdx.x * COMM_THREADS + ctid;
    bool copied = false;
    if (c.gather) {
      // ---- all-gather of the sharded operand, chunk by chunk
      if (linked && blockIdx.x == 0 && ctid < c.nranks && ctid != c.rank) {
        // everything earlier in this stream (the kernel that produced the shard) is complete
        __threadfence_system();
        st_release_sys(c.flags[ctid] + c.ready_slot + c.rank, c.epoch);
      }
      uint32_t seen = linked ? (1u << c.rank) : 0xffffffffu;
      for (int j = 0; j < c.num_chunks; ++j) {
        const int ch = (c.chunk0 + j) % c.num_chunks;
        const long long lo = (long long)ch * c.chunk_vec;
        const long long hi = lo + c.chunk_vec < c.total_vec ? lo + c.chunk_vec : c.total_vec;
        int r = (int)(lo / c.shard_vec);
        for (long long s0 = lo; s0 < hi; ++r) {
          const long long end_r = (long long)(r + 1) * c.shard_vec;
          const long long s1 = hi < end_r ? hi : end_r;
          if (!((seen >> r) & 1u)) {
            if (lane == 0)
              wait_flag(c.flags[c.rank] + c.ready_slot + r, c.epoch, p.status, 4000 + r, c.limit_ns);
            __syncwarp();
            seen |= 1u << r;
          }
          // source indexed by the vector's position in the whole operand
          copy_span(c.full, c.shard[r] - (long long)r * c.shard_vec, s0, s1, first, stride);
          s0 = s1;
        }
        fence_proxy_async();    // these ordinary stores are read through TMA by other CTAs
        __threadfence();
        named_bar(1, COMM_THREADS);
        if (ctid == 0) red_release_gpu_u64(c.ready + ch, 1ull);
      }
      copied = true;
    } else if (c.scatter && c.out != nullptr) {
      // ---- pull the peers' partial blocks of this rank's rows, in the order in which they finish
      const long long blk_vec = ((long long)c.rows_per * p.N) >> 3;
      const long long sub_vec = ((long long)c.sub_rows * p.N) >> 3;
      for (int k = 1; k < c.nranks; ++k) {
        const int r = (c.rank - k + c.nranks) % c.nranks;
        for (int sb = 0; sb < c.num_sub; ++sb) {      // the peer finishes them in this order
          if (lane == 0)
            wait_flag(c.flags[c.rank] + c.ready_slot + r * MAX_SUB + sb, c.epoch, p.status, 5000 + r, c.limit_ns);
          __syncwarp();
          copy_span(reinterpret_cast<uint4*>(c.pulled) + (long long)r * blk_vec,
                    reinterpret_cast<const uint4*>(c.partial[r]) + (long long)c.rank * blk_vec,
                    sb * sub_vec, (sb + 1) * sub_vec, first, stride);
        }
      }
      __threadfence();
      named_bar(1, COMM_THREADS);
      if (ctid == 0) red_release_gpu_u64(c.ready, 1ull);
      copied = true;
      scatter_reduce(p, c, lane, blockIdx.x * (EPI_THREADS + COMM_THREADS) + EPI_THREADS + ctid);
    }
    if (copied && linked) {
      // the last CTA to finish copying tells the peers that their buffers are no longer read
      __threadfence();
      named_bar(1, COMM_THREADS);
      if (ctid == 0) {
        int* cta_count = c.counters + (c.scatter ? c.nranks * MAX_SUB + 1 : 0);
        if (atomicAdd(cta_count, 1) == (int)gridDim.x - 1) {
          *cta_count = 0;
          for (int r = 0; r < c.nranks; ++r)
            if (r != c.rank) st_release_sys(c.flags[r] + c.done_slot + c.rank, c.epoch);
        }
      }
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

__global__ void __launch_bounds__(256)
rs_reduce_kernel(const BlockSources src, int nranks, int rows_per, int N, __nv_bfloat16* out, long long ldo,
                 const __nv_bfloat16* residual) {
  reduce_rows(src, nranks, rows_per, N, out, ldo, residual, (long long)blockIdx.x * blockDim.x + threadIdx.x,
              (long long)gridDim.x * blockDim.x);
}

template <bool B_MN>
static int resident_pairs() {
  int dev = 0;
  cudaGetDevice(&dev);
  static bool configured[64] = {false};
  static int cache[64] = {0};
  auto kern = gemm_fused_kernel<B_MN>;
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -1;
    configured[dev & 63] = true;
  }
  if (!cache[dev & 63]) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (xb_sm_count() / 2));
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = xb_sm_count() / 2;
    }
    if (clusters > xb_sm_count() / 2) clusters = xb_sm_count() / 2;
    cache[dev & 63] = clusters;
  }
  return cache[dev & 63];
}

}  // namespace xb_gemmf

// Argument block of xb_gemm_fused (plain C layout, filled from Python through ctypes).
struct XbFusedArgs {
  const void* A;                 // [M, K] row-major (the local full copy when A is gathered)
  const void* B;                 // b_mn = 0: [N, K] row-major; b_mn = 1: [K, N] row-major
  void* C;                       // result; with scatter: this rank's partial buffer [M][N] (= partial_ptrs[rank])
  int M, N, K;
  long long lda, ldb, ldc;
  int b_mn, out_fp32, accumulate;
  int rank, nranks;
  int gather;                    // 0 / 1 (A) / 2 (B)
  int scatter;
  unsigned long long shard_ptrs[16];   // gather: every rank's shard of the gathered operand
  long long rows_per_rank;             // gather: rows per shard; scatter: result rows per owner
  unsigned long long ready_counters;   // gather: device u64[num_chunks], monotonic
  unsigned long long ready_target;     // gather: value every chunk counter reaches in this call is
                                       //         ready_base + CTAs; pass ready_base here
  unsigned long long partial_ptrs[16]; // scatter: every rank's partial-result buffer [M][N] (symmetric)
  void* pulled;                        // scatter: local staging [nranks][rows_per_rank][N]
  void* out;                           // scatter: reduced rows of this rank (null: partial result only)
  long long ldo;
  const void* residual;
  unsigned long long counters;         // device int[...] zeroed once by the caller
  unsigned long long flag_ptrs[16];    // every rank's flag area (0: single-device run)
  int ready_slot, done_slot, epoch, done_needed;
  int wait_ms;
  int ctas_out;                        // written: CTAs launched (the caller advances ready_base by it)
};

XB_API int xb_gemm_fused(XbFusedArgs* a, void* stream) {
  using namespace xb_gemm2;
  using namespace xb_gemmf;
  const int M = a->M, N = a->N, K = a->K;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (a->nranks < 1 || a->nranks > MAX_R || (a->gather && a->scatter)) return -1;
  if ((a->lda % 8) || (a->ldb % 8) || (reinterpret_cast<uintptr_t>(a->A) % 16) ||
      (reinterpret_cast<uintptr_t>(a->B) % 16))
    return -1;
  if (a->gather == 1 && (a->lda != K || (K % 8) || a->rows_per_rank * a->nranks < M)) return -4;   // contiguous chunks
  if (a->gather == 2 && (a->b_mn || a->ldb != K || (K % 8) || a->rows_per_rank * a->nranks < N)) return -4;
  if (a->scatter && ((a->rows_per_rank % 32) || (N % 8) || a->ldc != N || a->out_fp32 || a->accumulate ||
                     a->rows_per_rank * a->nranks != M))
    return -5;
  if (a->scatter && a->out != nullptr && (a->flag_ptrs[0] == 0 || a->pulled == nullptr || a->ready_counters == 0))
    return -7;       // pulling needs real peers; on one device only the partial result is produced
  CUtensorMap ta, tb, tb64;
  int rc = xb_make_tmap_2d(&ta, a->A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, a->lda, BM, BK,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -2;
  if (!a->b_mn) {
    rc = xb_make_tmap_2d(&tb, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, a->ldb, BNH, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc)
      rc = xb_make_tmap_2d(&tb64, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, a->ldb, 64, BK,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    rc = xb_make_tmap_2d(&tb, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, a->ldb, BK, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
    tb64 = tb;
  }
  if (rc) return -3;
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.C = a->C; p.ldc = a->ldc;
  p.out_fp32 = a->out_fp32; p.accumulate = a->accumulate;
  p.num_m_blocks = (M + 511) / 512;
  p.num_n_blocks = (N + BN - 1) / BN;
  p.status = xb_status_ptr();
  Comm c = {};
  c.rank = a->rank; c.nranks = a->nranks;
  c.gather = a->gather; c.scatter = a->scatter;
  c.limit_ns = (unsigned long long)(a->wait_ms > 0 ? a->wait_ms : 2000) * 1000000ull;
  for (int r = 0; r < MAX_R; ++r) {
    c.shard[r] = reinterpret_cast<const uint4*>(a->shard_ptrs[r]);
    c.partial[r] = reinterpret_cast<const __nv_bfloat16*>(a->partial_ptrs[r]);
    c.flags[r] = reinterpret_cast<int*>(a->flag_ptrs[r]);
  }
  c.ready_slot = a->ready_slot; c.done_slot = a->done_slot;
  c.epoch = a->epoch; c.done_needed = a->done_needed;
  c.counters = reinterpret_cast<int*>(a->counters);
  // raster: walk the blocks of the gathered / scattered dimension in rank order, this rank's own
  // rows first (gather) or last (scatter); the other dimension runs fastest
  p.group_m = 4;
  const long long row_vec = K / 8;
  if (a->gather == 1) {
    p.group_m = 1;
    c.rot_m = (int)((a->rank * a->rows_per_rank) / 512) % p.num_m_blocks;
    c.full = reinterpret_cast<uint4*>(const_cast<void*>(a->A));
    c.shard_vec = a->rows_per_rank * row_vec;
    c.total_vec = (long long)M * row_vec;
    c.chunk_vec = 512 * row_vec;
    c.num_chunks = p.num_m_blocks;
    c.chunk0 = c.rot_m;
  } else if (a->gather == 2) {
    p.group_m = p.num_m_blocks;
    c.rot_n = (int)((a->rank * a->rows_per_rank) / BN) % p.num_n_blocks;
    c.full = reinterpret_cast<uint4*>(const_cast<void*>(a->B));
    c.shard_vec = a->rows_per_rank * row_vec;
    c.total_vec = (long long)N * row_vec;
    c.chunk_vec = (long long)BN * row_vec;
    c.num_chunks = p.num_n_blocks;
    c.chunk0 = c.rot_n;
  }
  if (a->gather) {
    if (a->rows_per_rank <= 0 || a->ready_counters == 0 || (c.flags[0] && !c.counters)) return -6;
    c.ready = reinterpret_cast<unsigned long long*>(a->ready_counters);
  }
  if (a->scatter) {
    if (!c.counters) return -6;
    p.group_m = 1;
    c.rows_per = (int)a->rows_per_rank;
    // an owner's rows are announced in up to MAX_SUB pieces of at least 512 rows, so that the owner
    // starts pulling long before its whole block is complete
    c.num_sub = 1;
    for (int n = MAX_SUB; n > 1; n >>= 1)
      if (c.rows_per % (n * 32) == 0 && c.rows_per / n >= 512) { c.num_sub = n; break; }
    c.sub_rows = c.rows_per / c.num_sub;
    c.units_per_sub = (c.sub_rows / 32) * 2 * p.num_n_blocks;     // warps x column halves of every tile
    c.rot_m = (int)(((a->rank + 1) * a->rows_per_rank) / 512) % p.num_m_blocks;
    c.pulled = reinterpret_cast<__nv_bfloat16*>(a->pulled);
    c.ready = reinterpret_cast<unsigned long long*>(a->ready_counters);
    c.out = reinterpret_cast<__nv_bfloat16*>(a->out);
    c.ldo = a->ldo;
    c.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
    if (c.out && ((a->ldo % 8) || (reinterpret_cast<uintptr_t>(a->out) % 16))) return -5;
  }
  const int pairs_max = a->b_mn ? resident_pairs<true>() : resident_pairs<false>();
  if (pairs_max <= 0) return -10;
  plan_items(p, pairs_max, true);
  const int pairs = p.num_items < pairs_max ? p.num_items : pairs_max;
  a->ctas_out = 2 * pairs;
  c.ready_target = a->ready_target + (unsigned long long)(2 * pairs);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->b_mn)
    gemm_fused_kernel<true><<<2 * pairs, NT, SMEM_BYTES, st>>>(ta, tb, tb64, p, c);
  else
    gemm_fused_kernel<false><<<2 * pairs, NT, SMEM_BYTES, st>>>(ta, tb, tb64, p, c);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// out = sum over r of block_ptrs[r] (contiguous [rows_per][N] bf16 blocks) in fp32 (+ residual): the
// reduction phase of the scatter path as a kernel of its own (partials produced by separate
// launches on one device).
XB_API int xb_rs_reduce(const unsigned long long* block_ptrs, int nranks, int rows_per, int N, void* out,
                        long long ldo, const void* residual, void* stream) {
  using namespace xb_gemmf;
  if ((N % 8) || (ldo % 8) || nranks < 1 || nranks > MAX_R) return -1;
  BlockSources src = {};
  for (int r = 0; r < nranks; ++r) src.p[r] = reinterpret_cast<const uint4*>(block_ptrs[r]);
  rs_reduce_kernel<<<2 * xb_sm_count(), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      src, nranks, rows_per, N, reinterpret_cast<__nv_bfloat16*>(out), ldo,
      reinterpret_cast<const __nv_bfloat16*>(residual));
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
