// Expert-parallel dispatch / combine over NVLink peer memory (no NCCL, no host synchronisation).
//
//   xb_ep_exchange_counts  every rank writes its per-expert slot counts into row [rank] of every
//                          peer's count table, then waits (bounded) until all rows have arrived
//   xb_ep_prepare_recv     marks rows of the receive buffer that no token will occupy (alignment
//                          padding inside expert segments, everything past the last segment) with
//                          meta = -1 and zeroes padding rows so that grouped GEMMs may read them
//   xb_ep_push_rows        copies rows to arbitrary rows of arbitrary peers' buffers (one warp per
//                          row, 16-byte peer stores) and optionally tags them; the last CTA to
//                          finish signals every peer.  Used for dispatch (token slot -> expert row
//                          on the owner), for returning expert outputs (expert row -> slot on the
//                          source) and for both of their backward passes.
// The consumer waits for all peers' signals with xb_symm_wait (csrc/comm.cu).
// Replaces DeepEP's dispatch / combine (src/xorl/distributed/moe/deepep.py:454-791) and the
// all_to_all_single path (src/xorl/distributed/moe/alltoall.py:86-233) of the reference.
#include "common.cuh"

namespace {

constexpr int MAX_RANKS = 16;
struct PeerPtrs { void* p[MAX_RANKS]; };

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

PeerPtrs make_ptrs(const unsigned long long* ptrs, int n) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < n ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}

// tables.p[r]: int32 [n][E] on rank r.  flags.p[r]: int32 flag area of rank r.
__global__ void __launch_bounds__(256)
ep_exchange_counts_kernel(const int* __restrict__ counts, PeerPtrs tables, PeerPtrs flags, int slot,
                          int rank, int n, int E, int epoch, int* status, uint64_t limit_ns) {
  for (int r = 0; r < n; ++r) {
    int* dst = reinterpret_cast<int*>(tables.p[r]) + (size_t)rank * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < n && (int)threadIdx.x != rank)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot + rank, epoch);
  if ((int)threadIdx.x < n && (int)threadIdx.x != rank) {
    const int* f = reinterpret_cast<const int*>(flags.p[rank]) + slot + threadIdx.x;
    const uint64_t t0 = xb_globaltimer();
    uint32_t it = 0;
    while (ld_acquire_sys(f) < epoch) {
      __nanosleep(64);
      if ((++it & 255u) == 0u && xb_globaltimer() - t0 > limit_ns) {
        xb_report(status, XB_ERR_FLAG_TIMEOUT, XB_K_EP_DISPATCH, (int)threadIdx.x);
        break;
      }
    }
  }
}

// seg: int32 [El+1] aligned segment starts; tot: int32 [El] real rows per local expert.
__global__ void __launch_bounds__(256)
ep_prepare_recv_kernel(uint4* __restrict__ x, int* __restrict__ meta, const int* __restrict__ seg,
                       const int* __restrict__ tot, int El, int cap_rows, int row_vec) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int end = seg[El];
  for (int r = warp; r < cap_rows; r += nwarps) {
    if (r >= end) {
      if (lane == 0) meta[r] = -1;
      continue;
    }
    int e = 0;
    while (e + 1 < El && r >= seg[e + 1]) ++e;
    if (r - seg[e] >= tot[e]) {  // alignment padding inside the segment
      if (lane == 0) meta[r] = -1;
      uint4* row = x + (size_t)r * row_vec;
      for (int v = lane; v < row_vec; v += 32) row[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Item i: copy src row (src_row[i] or i) to row dest_row[i] of rank dest_rank[i] (skip if < 0),
// and, when metas is given, store tag[i] (or i) into that rank's meta[dest_row[i]].
__global__ void __launch_bounds__(256, 2)
ep_push_rows_kernel(const uint4* __restrict__ src, long long src_ld_vec, const int* __restrict__ src_row,
                    const int* __restrict__ dest_rank, const int* __restrict__ dest_row,
                    const int* __restrict__ tag, int tag_rank_shift, int n_items, int row_vec,
                    PeerPtrs dsts, long long dst_ld_vec, PeerPtrs metas, PeerPtrs flags, int slot,
                    int* counter, int rank, int n, int epoch) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int i = warp; i < n_items; i += nwarps) {
    const int dr = dest_rank[i];
    if (dr < 0) continue;
    const int row = dest_row[i];
    const uint4* s = src + (size_t)(src_row ? src_row[i] : i) * src_ld_vec;
    uint4* d = reinterpret_cast<uint4*>(dsts.p[dr]) + (size_t)row * dst_ld_vec;
    // four 16-byte loads in flight per lane before the (posted) peer stores
    int v = lane;
    for (; v + 96 < row_vec; v += 128) {
      const uint4 a = s[v], b = s[v + 32], c = s[v + 64], e = s[v + 96];
      d[v] = a; d[v + 32] = b; d[v + 64] = c; d[v + 96] = e;
    }
    for (; v < row_vec; v += 32) d[v] = s[v];
    if (metas.p[0] != nullptr && lane == 0) {
      const int t = tag ? tag[i] : i;
      reinterpret_cast<int*>(metas.p[dr])[row] = t | (rank << tag_rank_shift);
    }
  }
  // last CTA: make the stores visible system-wide, then tell every peer
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) *counter = 0;
    __threadfence_system();
    if ((int)threadIdx.x < n && (int)threadIdx.x != rank)
      st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot + rank, epoch);
  }
}

// Destination of every token slot, one block per global expert.  Slots of an expert keep their
// slot order (a block scans the slots in order and ranks its matches with a ballot prefix), so the
// layout is the same every run.  table: int32 [n][E], counts of every source rank (already
// exchanged).  Row of a slot on the owner = aligned start of the expert's segment on its owner
// + rows that lower ranks send to this expert + rank of the slot among this rank's slots of the
// expert.  Blocks of this rank's own experts also write seg / tot for the grouped GEMMs.
__global__ void __launch_bounds__(256)
ep_plan_kernel(const long long* __restrict__ indices, int S, const int* __restrict__ table, int rank, int n,
               int E, int El, int cap, int* __restrict__ dest_rank, int* __restrict__ dest_row,
               int* __restrict__ seg, int* __restrict__ tot, int* __restrict__ overflow) {
  const int e = blockIdx.x;
  const int owner = e / El, first = owner * El;
  __shared__ int s_base, s_total, s_start;
  __shared__ int s_warp[8];
  __shared__ int s_running;
  if (threadIdx.x < 32) {
    // aligned start of expert e inside its owner's buffer: sum of padded totals of the owner's earlier experts
    int start = 0;
    for (int e2 = first + (int)threadIdx.x; e2 < e; e2 += 32) {
      int t = 0;
      for (int r = 0; r < n; ++r) t += table[r * E + e2];
      start += (t + 127) / 128 * 128;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) start += __shfl_xor_sync(0xffffffffu, start, o);
    int mine = 0, before = 0;
    for (int r = (int)threadIdx.x; r < n; r += 32) {
      const int c = table[r * E + e];
      mine += c;
      if (r < rank) before += c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mine += __shfl_xor_sync(0xffffffffu, mine, o);
      before += __shfl_xor_sync(0xffffffffu, before, o);
    }
    if (threadIdx.x == 0) {
      s_start = start;
      s_base = start + before;
      s_total = mine;
      s_running = 0;
    }
  }
  __syncthreads();
  const int lim = cap / 128 * 128;
  if (owner == rank && threadIdx.x == 0) {
    const int le = e - first;
    seg[le] = min(s_start, lim);
    tot[le] = s_total;
    if (le == El - 1) seg[El] = min(s_start + (s_total + 127) / 128 * 128, lim);
  }
  const int base = s_base;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c0 = 0; c0 < S; c0 += 256) {
    const int slot = c0 + (int)threadIdx.x;
    const bool hit = slot < S && indices[slot] == (long long)e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) s_warp[warp] = __popc(m);
    __syncthreads();
    int before_w = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = s_warp[w];
      if (w < warp) before_w += c;
      total += c;
    }
    const int running = s_running;
    if (hit) {
      const int row = base + running + before_w + __popc(m & ((1u << lane) - 1u));
      if (row >= cap) {
        dest_rank[slot] = -1;
        dest_row[slot] = 0;
        *overflow = 1;
      } else {
        dest_rank[slot] = owner;
        dest_row[slot] = row;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) s_running = running + total;
    __syncthreads();
  }
}

// counts[e] = number of slots routed to expert e (shared-memory histogram, integer atomics)
__global__ void __launch_bounds__(256)
moe_histogram_kernel(const long long* __restrict__ idx, int S, int* __restrict__ counts, int E) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < S; i += gridDim.x * blockDim.x) {
    const long long e = idx[i];
    if (e >= 0 && e < E) atomicAdd(&sh[(int)e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    if (sh[e]) atomicAdd(&counts[e], sh[e]);
}

// meta (tag | rank << 24, or -1 for rows nobody owns) -> (rank or -1, slot)
__global__ void __launch_bounds__(256)
ep_meta_targets_kernel(const int* __restrict__ meta, int n, int* __restrict__ rank, int* __restrict__ slot) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int m = meta[i];
  rank[i] = m >= 0 ? (m >> 24) : -1;
  slot[i] = m >= 0 ? (m & 0xFFFFFF) : 0;
}

}  // namespace

XB_API int xb_moe_histogram(const long long* idx, int S, int* counts, int E, void* stream) {
  if (E <= 0 || E > 8192) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int), st) != cudaSuccess) return -2;
  if (S <= 0) return 0;
  int blocks = (S + 256 * 8 - 1) / (256 * 8);
  if (blocks > 64) blocks = 64;
  moe_histogram_kernel<<<blocks, 256, (size_t)E * sizeof(int), st>>>(idx, S, counts, E);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_ep_meta_targets(const int* meta, int n, int* rank, int* slot, void* stream) {
  if (n <= 0) return 0;
  ep_meta_targets_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(meta, n, rank, slot);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_ep_plan(const long long* indices, int S, const int* table, int rank, int n, int E, int El, int cap,
                      int* dest_rank, int* dest_row, int* seg, int* tot, int* overflow, void* stream) {
  if (E <= 0 || El <= 0 || E % El || n > MAX_RANKS) return -1;
  ep_plan_kernel<<<E, 256, 0, (cudaStream_t)stream>>>(indices, S, table, rank, n, E, El, cap, dest_rank,
                                                      dest_row, seg, tot, overflow);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_ep_exchange_counts(const int* counts, const unsigned long long* table_ptrs,
                                 const unsigned long long* flag_ptrs, int slot, int rank, int n, int E,
                                 int epoch, int wait_ms, void* stream) {
  if (n > MAX_RANKS) return -1;
  ep_exchange_counts_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(
      counts, make_ptrs(table_ptrs, n), make_ptrs(flag_ptrs, n), slot, rank, n, E, epoch,
      xb_status_ptr(), (uint64_t)wait_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_ep_prepare_recv(void* x, int* meta, const int* seg, const int* tot, int El, int cap_rows,
                              int row_bytes, void* stream) {
  if (row_bytes % 16) return -1;
  const int grid = xb_sm_count() * 2;
  ep_prepare_recv_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((uint4*)x, meta, seg, tot, El,
                                                                 cap_rows, row_bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// src: local rows (row stride src_ld_bytes); dst_ptrs[n]: every rank's destination buffer (row stride
// dst_ld_bytes); meta_ptrs may be null.  Tags are stored as tag | (rank << tag_rank_shift).
XB_API int xb_ep_push_rows(const void* src, long long src_ld_bytes, const int* src_row,
                           const int* dest_rank, const int* dest_row, const int* tag,
                           int tag_rank_shift, int n_items, int row_bytes,
                           const unsigned long long* dst_ptrs, long long dst_ld_bytes,
                           const unsigned long long* meta_ptrs, const unsigned long long* flag_ptrs,
                           int slot, int counter_slot, int rank, int n, int epoch, void* stream) {
  if (n > MAX_RANKS || (row_bytes % 16) || (src_ld_bytes % 16) || (dst_ld_bytes % 16)) return -1;
  PeerPtrs fl = make_ptrs(flag_ptrs, n);
  PeerPtrs mt;
  for (int i = 0; i < MAX_RANKS; ++i) mt.p[i] = nullptr;
  if (meta_ptrs) mt = make_ptrs(meta_ptrs, n);
  int* counter = reinterpret_cast<int*>(fl.p[rank]) + counter_slot;
  // nothing else runs while a layer waits for its rows: use every SM (two CTAs each)
  int grid = xb_sm_count() * 2;
  if (grid > (n_items + 7) / 8) grid = (n_items + 7) / 8;
  if (grid < 1) grid = 1;
  ep_push_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, src_ld_bytes / 16, src_row, dest_rank, dest_row, tag, tag_rank_shift, n_items,
      row_bytes / 16, make_ptrs(dst_ptrs, n), dst_ld_bytes / 16, mt, fl, slot, counter, rank, n, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
