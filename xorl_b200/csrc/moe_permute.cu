// Row movement of the MoE block without atomics and without intermediate copies: every kernel is a
// gather (one warp per output row, 16-byte vectors), so the backward of a scatter is written as the
// matching gather over an inverse index.  Replaces the Triton index / scatter / gather kernels of
// src/xorl/ops/group_gemm/kernel/moe.py:45-433 and the weighted scatter-add of
// src/xorl/ops/ep_kernels/deepep_scatter_gather.py.
//
//   xb_moe_gather_rows   out[r] = scale[r] * in[src[r]]   (src[r] < 0 -> zero row)
//                        forward permutation into expert-sorted, segment-aligned rows; backward of
//                        the weighted combine
//   xb_moe_gather_sum    out[t] = sum_j w[t,j] * in[idx[t,j]]   (fp32 accumulation)
//                        weighted combine of the k expert outputs of a token; backward of the
//                        permutation (w = null)
//   xb_moe_slot_dots     dw[t,j] = <dout[t], y[idx[t,j]]>        gradient of the routing weights
#include "common.cuh"

namespace {

__device__ __forceinline__ void fma8(float (&acc)[8], const uint4 v, float w) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  acc[0] = fmaf(w, a.x, acc[0]); acc[1] = fmaf(w, a.y, acc[1]);
  acc[2] = fmaf(w, b.x, acc[2]); acc[3] = fmaf(w, b.y, acc[3]);
  acc[4] = fmaf(w, c.x, acc[4]); acc[5] = fmaf(w, c.y, acc[5]);
  acc[6] = fmaf(w, d.x, acc[6]); acc[7] = fmaf(w, d.y, acc[7]);
}
__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  return make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                    pack_bf16x2(a[6], a[7]));
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(uint4* __restrict__ out, long long ld_out, const uint4* __restrict__ in, long long ld_in,
                   const int* __restrict__ src, const float* __restrict__ scale, int rows, int vecs) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int r = warp; r < rows; r += nwarps) {
    const int s = src[r];
    uint4* o = out + (long long)r * ld_out;
    if (s < 0) {
      for (int v = lane; v < vecs; v += 32) o[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* i = in + (long long)s * ld_in;
    if (scale == nullptr) {
      for (int v = lane; v < vecs; v += 32) o[v] = i[v];
    } else {
      const float w = scale[r];
      for (int v = lane; v < vecs; v += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        fma8(acc, i[v], w);
        o[v] = pack8(acc);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
gather_sum_kernel(uint4* __restrict__ out, long long ld_out, const uint4* __restrict__ in, long long ld_in,
                  const long long* __restrict__ idx, const float* __restrict__ w, int T, int k, int vecs) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nwarps) {
    for (int v = lane; v < vecs; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const long long r = idx[(long long)t * k + j];
        fma8(acc, in[r * ld_in + v], w ? w[(long long)t * k + j] : 1.f);
      }
      out[(long long)t * ld_out + v] = pack8(acc);
    }
  }
}

__global__ void __launch_bounds__(256)
slot_dots_kernel(float* __restrict__ dw, const uint4* __restrict__ dout, long long ld_do,
                 const uint4* __restrict__ y, long long ld_y, const long long* __restrict__ idx, int T, int k,
                 int vecs) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)T * k) return;
  const long long t = warp / k;
  const uint4* a = dout + t * ld_do;
  const uint4* b = y + idx[warp] * ld_y;
  float s = 0.f;
  for (int v = lane; v < vecs; v += 32) {
    const uint4 x = a[v], z = b[v];
    const float2 x0 = unpack_bf16x2(x.x), x1 = unpack_bf16x2(x.y), x2 = unpack_bf16x2(x.z), x3 = unpack_bf16x2(x.w);
    const float2 z0 = unpack_bf16x2(z.x), z1 = unpack_bf16x2(z.y), z2 = unpack_bf16x2(z.z), z3 = unpack_bf16x2(z.w);
    s += x0.x * z0.x + x0.y * z0.y + x1.x * z1.x + x1.y * z1.y + x2.x * z2.x + x2.y * z2.y + x3.x * z3.x +
         x3.y * z3.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dw[warp] = s;
}

inline int grid_for(long long warps) {
  long long blocks = (warps + 7) / 8;
  const long long cap = 148ll * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

// bf16 rows of `width` elements (multiple of 8); ld_* in elements (multiples of 8); 16-byte aligned.
XB_API int xb_moe_gather_rows(void* out, long long ld_out, const void* in, long long ld_in, const int* src,
                              const float* scale, int rows, int width, void* stream) {
  if (rows <= 0) return 0;
  if (width % 8 || ld_out % 8 || ld_in % 8) return -1;
  gather_rows_kernel<<<grid_for(rows), 256, 0, (cudaStream_t)stream>>>((uint4*)out, ld_out / 8, (const uint4*)in,
                                                                        ld_in / 8, src, scale, rows, width / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_moe_gather_sum(void* out, long long ld_out, const void* in, long long ld_in, const long long* idx,
                             const float* w, int T, int k, int width, void* stream) {
  if (T <= 0) return 0;
  if (width % 8 || ld_out % 8 || ld_in % 8) return -1;
  gather_sum_kernel<<<grid_for(T), 256, 0, (cudaStream_t)stream>>>((uint4*)out, ld_out / 8, (const uint4*)in,
                                                                    ld_in / 8, idx, w, T, k, width / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_moe_slot_dots(float* dw, const void* dout, long long ld_do, const void* y, long long ld_y,
                            const long long* idx, int T, int k, int width, void* stream) {
  if (T <= 0) return 0;
  if (width % 8 || ld_do % 8 || ld_y % 8) return -1;
  const long long warps = (long long)T * k;
  slot_dots_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      dw, (const uint4*)dout, ld_do / 8, (const uint4*)y, ld_y / 8, idx, T, k, width / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
