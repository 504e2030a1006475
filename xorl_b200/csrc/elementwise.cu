// SwiGLU forward/backward, embedding gather / scatter-add, dtype casts and small utilities.
// Reference behaviour: src/xorl/ops/fused_silu_and_mul.py:23-359 (silu(gate)*up with the
// silu result rounded to bf16 before the multiply — "two-round" rounding).
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16(x));
}

// gu: [T, 2I] (gate = [:, :I], up = [:, I:]) -> out [T, I]
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                  long long T, int I, int two_round, const int* __restrict__ row_limit) {
  const int vec_per_row = I >> 3;
  // row_limit (optional, device memory): only the first *row_limit rows hold data
  if (row_limit != nullptr) T = min(T, (long long)*row_limit);
  const long long total = T * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vec_per_row;
    const int v = (int)(idx % vec_per_row);
    const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * I)[v];
    const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * I + I)[v];
    const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gg[j]), b = unpack_bf16x2(uu[j]);
      float s0 = silu_f(a.x), s1 = silu_f(a.y);
      if (two_round) { s0 = round_bf16(s0); s1 = round_bf16(s1); }
      o[j] = pack_bf16x2(s0 * b.x, s1 * b.y);
    }
    reinterpret_cast<uint4*>(out + t * I)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dgu[:, :I] = dout * up * dsilu(gate);  dgu[:, I:] = dout * silu(gate)
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                  __nv_bfloat16* __restrict__ dgu, long long T, int I, const int* __restrict__ row_limit) {
  const int vec_per_row = I >> 3;
  if (row_limit != nullptr) T = min(T, (long long)*row_limit);
  const long long total = T * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vec_per_row;
    const int v = (int)(idx % vec_per_row);
    const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * I)[v];
    const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * I + I)[v];
    const uint4 d = reinterpret_cast<const uint4*>(dout + t * I)[v];
    const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w},
                   dd[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gg[j]), b = unpack_bf16x2(uu[j]), c = unpack_bf16x2(dd[j]);
      const float sg0 = sigmoid_f(a.x), sg1 = sigmoid_f(a.y);
      const float ds0 = sg0 * (1.f + a.x * (1.f - sg0)), ds1 = sg1 * (1.f + a.y * (1.f - sg1));
      og[j] = pack_bf16x2(c.x * b.x * ds0, c.y * b.y * ds1);
      ou[j] = pack_bf16x2(c.x * a.x * sg0, c.y * a.y * sg1);
    }
    reinterpret_cast<uint4*>(dgu + t * 2 * I)[v] = make_uint4(og[0], og[1], og[2], og[3]);
    reinterpret_cast<uint4*>(dgu + t * 2 * I + I)[v] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// out[t, :] = table[ids[t], :]   (ids outside [0, V) produce zeros and set a status word)
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* __restrict__ out, int T, int H, long long V, int* status) {
  const int vec_per_row = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) xb_report(status, XB_ERR_BOUNDS, 0, t);
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      uint4 val = make_uint4(0, 0, 0, 0);
      if (ok) val = reinterpret_cast<const uint4*>(table + (size_t)id * H)[v];
      reinterpret_cast<uint4*>(out + (size_t)t * H)[v] = val;
    }
  }
}

// dtable[ids[t], :] += dout[t, :]   (fp32 accumulation buffer, atomics)
__global__ void __launch_bounds__(256)
embedding_bwd_f32_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                         float* __restrict__ dtable, int T, int H, long long V) {
  const int pairs = H >> 1;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = ids[t];
    if (id < 0 || id >= V) continue;
    for (int v = threadIdx.x; v < pairs; v += blockDim.x) {
      const float2 d = unpack_bf16x2(reinterpret_cast<const uint32_t*>(dout + (size_t)t * H)[v]);
      atomicAdd(dtable + (size_t)id * H + 2 * v, d.x);
      atomicAdd(dtable + (size_t)id * H + 2 * v + 1, d.y);
    }
  }
}

// bf16x2 atomics straight into a bf16 gradient table
__global__ void __launch_bounds__(256)
embedding_bwd_bf16_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                          __nv_bfloat16* __restrict__ dtable, int T, int H, long long V) {
  const int pairs = H >> 1;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = ids[t];
    if (id < 0 || id >= V) continue;
    for (int v = threadIdx.x; v < pairs; v += blockDim.x) {
      const __nv_bfloat162 d = reinterpret_cast<const __nv_bfloat162*>(dout + (size_t)t * H)[v];
      atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + (size_t)id * H) + v, d);
    }
  }
}

__global__ void __launch_bounds__(256)
add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 x = reinterpret_cast<const uint4*>(a)[i], y = reinterpret_cast<const uint4*>(b)[i];
    const uint32_t xx[4] = {x.x, x.y, x.z, x.w}, yy[4] = {y.x, y.y, y.z, y.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p = unpack_bf16x2(xx[j]), q = unpack_bf16x2(yy[j]);
      o[j] = pack_bf16x2(p.x + q.x, p.y + q.y);
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

static inline int grid_for(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = (long long)xb_sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

XB_API int xb_swiglu_fwd(const void* gu, void* out, long long T, int I, int two_round,
                         void* stream) {
  if (I % 8) return -1;
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I, two_round, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Variants for buffers sized for the worst case: only the first *row_limit rows (an int in device
// memory, e.g. the end of the last expert segment) are processed; the grid is sized for T rows.
XB_API int xb_swiglu_fwd_rows(const void* gu, void* out, long long T, int I, int two_round, const int* row_limit,
                              void* stream) {
  if (I % 8) return -1;
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I, two_round, row_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_swiglu_bwd_rows(const void* dout, const void* gu, void* dgu, long long T, int I, const int* row_limit,
                              void* stream) {
  if (I % 8) return -1;
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, I, row_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int I,
                         void* stream) {
  if (I % 8) return -1;
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, I, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_embedding_fwd(const long long* ids, const void* table, void* out, int T, int H,
                            long long V, void* stream) {
  if (H % 8) return -1;
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<T < 4096 ? T : 4096, 256, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, V, xb_status_ptr());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_embedding_bwd(const long long* ids, const void* dout, void* dtable, int table_fp32,
                            int T, int H, long long V, void* stream) {
  if (H % 2) return -1;
  if (T <= 0) return 0;
  const int grid = T < 4096 ? T : 4096;
  if (table_fp32)
    embedding_bwd_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        ids, (const __nv_bfloat16*)dout, (float*)dtable, T, H, V);
  else
    embedding_bwd_bf16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        ids, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dtable, T, H, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n % 8) return -1;
  if (n <= 0) return 0;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
