// Collectives over NVLink peer memory, written as plain kernels on symmetric buffers.
//
// Every rank maps every peer's buffer (see xorl_b200/parallel/symm_transport.py), so a kernel can
// load from or store to another GPU with ordinary ld/st, or reduce through the NVSwitch with
// multimem.ld_reduce on the multicast mapping.  Synchronisation between ranks uses monotonically
// increasing 32-bit epochs in a small flag area of each rank's buffer: a writer stores its epoch
// into slot [its rank] of every peer with st.release.sys, a waiter spins with ld.acquire.sys on
// its own slots until all are >= the epoch.  Every spin is bounded by %globaltimer; on expiry
// the kernel records XB_ERR_FLAG_TIMEOUT and carries on without hanging the GPU.
//
//   xb_symm_barrier            all ranks reach a point (after the optimizer step, before peers read
//                              the freshly written parameter shards)
//   xb_symm_allgather          pull every peer's parameter shard into the local full buffer
//   xb_symm_reduce_scatter     wait until all peers' gradients for this buffer are final, sum the
//                              slice this rank owns over all peers in fp32 (fixed rank order), add
//                              it to the fp32 accumulator, emit sum-of-squares partials, tell the
//                              peers the buffer may be reused  (ZeRO gradient reduce-scatter +
//                              cast/scale + accumulate in one pass, with bf16 on the wire)
//   xb_symm_allgather_dma      the same gather as one cudaMemcpyAsync per peer shard: the copy engines
//                              move the bytes over NVLink and no SM is taken from the GEMMs that run
//                              beside the prefetch
//   xb_symm_gather_slices_dma  copy engines bring this rank's slice of every peer's gradient buffer
//                              into local staging; xb_symm_reduce_scatter then runs on local pointers
//                              (fp32 sum in rank order + accumulate + norm partials at HBM speed)
//   xb_symm_wait               block a stream until peers have released a buffer
//   xb_peer_copy               bulk copy between two mapped buffers (weight sync)
//   xb_peer_copy_2d            strided block copy by the copy engines (Ulysses head / sequence exchange)
// These replace the NCCL all-gather / reduce-scatter issued by FSDP2 in the reference
// (src/xorl/distributed/torch_parallelize.py:333-783) and its custom bf16 all-to-all reduce
// (src/xorl/distributed/fsdp2/bf16_a2a_reduce.py:64-114).
#include "common.cuh"

namespace {

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Waits until flags[i] >= epoch for all i < n (skipping `self`).  One thread spins per flag.
// Returns false (after recording the status) when the time limit expired.
__device__ __forceinline__ bool wait_flags(const int* flags, int n, int self, int epoch, int* status,
                                           int kernel_id, uint64_t limit_ns) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if ((int)threadIdx.x < n && (int)threadIdx.x != self) {
    const uint64_t t0 = xb_globaltimer();
    uint32_t it = 0;
    while (ld_acquire_sys(flags + threadIdx.x) < epoch) {
      __nanosleep(64);
      if ((++it & 255u) == 0u && xb_globaltimer() - t0 > limit_ns) {
        xb_report(status, XB_ERR_FLAG_TIMEOUT, kernel_id, (int)threadIdx.x);
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  return failed == 0;
}

__global__ void __launch_bounds__(32)
symm_barrier_kernel(PeerPtrs flags, int slot, int rank, int n, int epoch, int* status,
                    uint64_t limit_ns) {
  __threadfence_system();
  if ((int)threadIdx.x < n && (int)threadIdx.x != rank)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot + rank, epoch);
  wait_flags(reinterpret_cast<const int*>(flags.p[rank]) + slot, n, rank, epoch, status,
             XB_K_FLAG_WAIT_TEST, limit_ns);
}

__global__ void __launch_bounds__(32)
symm_wait_kernel(const int* flags, int n, int self, int epoch, int* status, uint64_t limit_ns) {
  wait_flags(flags, n, self, epoch, status, XB_K_FLAG_WAIT_TEST, limit_ns);
}

// dst[r * shard_vec + i] = src_r[i]   (16-byte vectors).  U independent 16-byte peer loads are in
// flight per thread: bytes in flight = CTAs x 512 x 16 x U, which has to cover the NVLink round trip
// at link bandwidth (about 2 MB).
template <int U>
__global__ void __launch_bounds__(512, 2)
symm_allgather_kernel(uint4* __restrict__ dst, PeerPtrs src, long long shard_vec, int rank, int n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int k = 0; k < n; ++k) {
    const int r = (rank + k) % n;  // start with the local shard, then walk the peers
    const uint4* s = reinterpret_cast<const uint4*>(src.p[r]);
    uint4* d = dst + (long long)r * shard_vec;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (U - 1) * stride < shard_vec; i += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = s[i + u * stride];
#pragma unroll
      for (int u = 0; u < U; ++u) d[i + u * stride] = v[u];
    }
    for (; i < shard_vec; i += stride) d[i] = s[i];
  }
}

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4 v) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z),
               d = unpack_bf16x2(v.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

// In-switch reduction of 8 bf16 values over all ranks bound to the multicast address.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_addr)
      : "memory");
  return v;
}

// grads.p[r]: base of rank r's bf16 gradient buffer; this rank owns elements
// [slice_off, slice_off + n_elem).  out (fp32 [n_elem]) (+)= sum_r grads_r[slice].
// flags.p[r]: rank r's flag area; ready slots at `ready_slot`, done slots at `done_slot`.
template <int NR>
__global__ void __launch_bounds__(512, 2)
symm_reduce_scatter_kernel(float* __restrict__ out, PeerPtrs grads, const void* mc_base,
                           long long slice_off, long long n_elem, int accumulate, float scale,
                           float* __restrict__ sumsq_partial, PeerPtrs flags, int ready_slot,
                           int done_slot, int* counter, int rank, int n, int epoch, int* status,
                           uint64_t limit_ns) {
  // 1. announce that this rank's gradients are final, then wait for everybody else's
  if (blockIdx.x == 0 && (int)threadIdx.x < n && (int)threadIdx.x != rank) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + ready_slot + rank, epoch);
  }
  const bool ok = wait_flags(reinterpret_cast<const int*>(flags.p[rank]) + ready_slot, n, rank,
                             epoch, status, XB_K_RS_ADAMW, limit_ns);
  // 2. reduce (also after a timeout: the result is then reported as invalid through the status
  //    words, but the kernel still terminates normally)
  (void)ok;
  const long long nvec = n_elem >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float ss = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (mc_base != nullptr) {
      const uint4 v = multimem_ld_reduce_bf16x8(reinterpret_cast<const __nv_bfloat16*>(mc_base) +
                                                slice_off + i * 8);
      acc_bf16x8(acc, v);
    } else {
      // NR loads in flight, summed in rank order (deterministic)
      for (int r0 = 0; r0 < n; r0 += NR) {
        uint4 v[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (r0 + r < n)
            v[r] = reinterpret_cast<const uint4*>(
                reinterpret_cast<const __nv_bfloat16*>(grads.p[r0 + r]) + slice_off)[i];
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (r0 + r < n) acc_bf16x8(acc, v[r]);
      }
    }
    float4* o = reinterpret_cast<float4*>(out + i * 8);
    float4 lo = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
    float4 hi = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
    if (accumulate) {
      const float4 a = o[0], b = o[1];
      lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
      hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
    }
    o[0] = lo; o[1] = hi;
    ss += lo.x * lo.x + lo.y * lo.y + lo.z * lo.z + lo.w * lo.w + hi.x * hi.x + hi.y * hi.y +
          hi.z * hi.z + hi.w * hi.w;
  }
  if (sumsq_partial != nullptr) {
    __shared__ float red[16];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
      sumsq_partial[blockIdx.x] = t;
    }
  }
  // 3. the last CTA to finish tells the peers that this rank no longer reads their buffers
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) {
    __threadfence();
    last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) *counter = 0;
    if ((int)threadIdx.x < n && (int)threadIdx.x != rank)
      st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + done_slot + rank, epoch);
  }
}

__global__ void __launch_bounds__(512, 2)
peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < nvec; i += stride) dst[i] = src[i];
}

PeerPtrs make_ptrs(const unsigned long long* ptrs, int n) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < n ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}

}  // namespace

// flag_ptrs[n]: device addresses of every rank's flag area (int32 array).  wait_ms bounds the spin.
XB_API int xb_symm_barrier(const unsigned long long* flag_ptrs, int slot, int rank, int n, int epoch,
                           int wait_ms, void* stream) {
  if (n > MAX_RANKS) return -1;
  symm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_ptrs(flag_ptrs, n), slot, rank, n,
                                                          epoch, xb_status_ptr(),
                                                          (uint64_t)wait_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Blocks the stream until local flags[0..n) (except `self`, pass -1 to wait for all) are >= epoch.
XB_API int xb_symm_wait(const void* flags, int n, int self, int epoch, int wait_ms, void* stream) {
  if (n > 32) return -1;
  symm_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const int*)flags, n, self, epoch,
                                                       xb_status_ptr(),
                                                       (uint64_t)wait_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// src_ptrs[n]: every rank's shard (shard_bytes each, multiple of 16); dst: local full buffer.
XB_API int xb_symm_allgather(void* dst, const unsigned long long* src_ptrs, long long shard_bytes,
                             int rank, int n, int num_ctas, void* stream) {
  if (n > MAX_RANKS || shard_bytes % 16) return -1;
  // num_ctas: low 16 bits = CTAs, bits 16.. = loads in flight per thread (4 or 8; default 4)
  const int unroll = (num_ctas >> 16) == 8 ? 8 : 4;
  num_ctas &= 0xffff;
  if (num_ctas <= 0) num_ctas = 64;
  if (unroll == 8)
    symm_allgather_kernel<8><<<num_ctas, 512, 0, (cudaStream_t)stream>>>(
        (uint4*)dst, make_ptrs(src_ptrs, n), shard_bytes / 16, rank, n);
  else
    symm_allgather_kernel<4><<<num_ctas, 512, 0, (cudaStream_t)stream>>>(
        (uint4*)dst, make_ptrs(src_ptrs, n), shard_bytes / 16, rank, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// One asynchronous device-to-device copy per rank, starting with the local shard and then walking
// the peers in ring order (rank + 1, rank + 2, ...), so that at any time every source serves one reader.
XB_API int xb_symm_allgather_dma(void* dst, const unsigned long long* src_ptrs, long long shard_bytes, int rank,
                                 int n, void* stream) {
  if (n > MAX_RANKS || shard_bytes <= 0) return -1;
  for (int k = 0; k < n; ++k) {
    const int r = (rank + k) % n;
    if (cudaMemcpyAsync(static_cast<char*>(dst) + (long long)r * shard_bytes, reinterpret_cast<const void*>(src_ptrs[r]),
                        (size_t)shard_bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream) != cudaSuccess)
      return -12;
  }
  return 0;
}

// staging: [n][slice_bytes] local; slot r receives bytes [slice_off_bytes, + slice_bytes) of rank r's
// buffer (the local rank's slot is skipped: its slice is read in place).
XB_API int xb_symm_gather_slices_dma(void* staging, const unsigned long long* buf_ptrs, long long slice_off_bytes,
                                     long long slice_bytes, int rank, int n, void* stream) {
  if (n > MAX_RANKS || slice_bytes <= 0) return -1;
  for (int k = 1; k < n; ++k) {
    const int r = (rank + k) % n;
    if (cudaMemcpyAsync(static_cast<char*>(staging) + (long long)r * slice_bytes,
                        reinterpret_cast<const char*>(buf_ptrs[r]) + slice_off_bytes, (size_t)slice_bytes,
                        cudaMemcpyDeviceToDevice, (cudaStream_t)stream) != cudaSuccess)
      return -12;
  }
  return 0;
}

// See symm_reduce_scatter_kernel.  mc_base = 0 selects peer loads, otherwise the multicast
// address of the same gradient buffer (NVLS in-switch reduction).  sumsq_partial may be null,
// else it receives num_ctas partial sums of squares of the updated accumulator slice.
XB_API int xb_symm_reduce_scatter(float* out, const unsigned long long* grad_ptrs,
                                  unsigned long long mc_base, long long slice_off, long long n_elem,
                                  int accumulate, float scale, float* sumsq_partial,
                                  const unsigned long long* flag_ptrs, int ready_slot,
                                  int done_slot, int counter_slot, int rank, int n, int epoch,
                                  int wait_ms, int num_ctas, void* stream) {
  if (n > MAX_RANKS || (n_elem % 8) || (slice_off % 8)) return -1;
  if (num_ctas <= 0) num_ctas = 48;
  PeerPtrs fl = make_ptrs(flag_ptrs, n);
  int* counter = reinterpret_cast<int*>(fl.p[rank]) + counter_slot;
#define XB_RS_ARGS out, make_ptrs(grad_ptrs, n), reinterpret_cast<const void*>(mc_base), slice_off, \
      n_elem, accumulate, scale, sumsq_partial, fl, ready_slot, done_slot, counter, rank, n, epoch, \
      xb_status_ptr(), (uint64_t)wait_ms * 1000000ull
  if (n <= 2)
    symm_reduce_scatter_kernel<2><<<num_ctas, 512, 0, (cudaStream_t)stream>>>(XB_RS_ARGS);
  else
    symm_reduce_scatter_kernel<4><<<num_ctas, 512, 0, (cudaStream_t)stream>>>(XB_RS_ARGS);
#undef XB_RS_ARGS
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_peer_copy(void* dst, const void* src, long long bytes, int num_ctas, void* stream) {
  if (bytes % 16) return -1;
  if (bytes == 0) return 0;
  if (num_ctas <= 0) num_ctas = 64;
  peer_copy_kernel<<<num_ctas, 512, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src,
                                                               bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Strided block copy by the copy engines (no SM): `height` rows of `width` bytes from src (row pitch
// spitch) to dst (row pitch dpitch); either side may be a peer's mapped memory.  The Ulysses head /
// sequence exchange is U such copies per rank: every rank writes its slice for rank u straight into
// u's receive buffer.
XB_API int xb_peer_copy_2d(void* dst, long long dpitch, const void* src, long long spitch, long long width,
                           long long height, void* stream) {
  if (width <= 0 || height <= 0) return 0;
  if (dpitch < width || spitch < width) return -1;
  return cudaMemcpy2DAsync(dst, (size_t)dpitch, src, (size_t)spitch, (size_t)width, (size_t)height,
                           cudaMemcpyDeviceToDevice, (cudaStream_t)stream) == cudaSuccess
             ? 0
             : -11;
}
