// RMSNorm forward/backward (optional fused residual add) and the fused per-head
// qk-RMSNorm + rotary embedding used by Qwen3-style attention.
//
// Memory-bound kernels: every tensor is read once with 16-byte vectors, statistics stay in
// registers, weight gradients are reduced through a per-CTA partial buffer (fixed order, so the
// result is run-to-run deterministic).
// Reference behaviour: src/xorl/models/layers/normalization.py:628-799 (RMSNorm with fused
// residual), src/xorl/models/layers/rope.py:646-676 (rotate-half RoPE),
// src/xorl/models/layers/attention/multi_head_attention.py:68-117 (norm then RoPE on q and k).
#include "common.cuh"

namespace {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 8;  // per thread: up to 8 vectors of 8 bf16 -> rows up to 16384 wide

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// y = rmsnorm(x + residual) * w ; residual_out = x + residual (when residual != nullptr).
// zero_centered: weight is stored as (w - 1).
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ residual_out, float* __restrict__ rstd_out, int T,
                   int H, float eps, int zero_centered) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + (size_t)row * H) : nullptr;
    float vals[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        uint4 a = xr[v];
        const uint32_t au[4] = {a.x, a.y, a.z, a.w};
        uint32_t ru[4] = {0, 0, 0, 0};
        if (rr) {
          uint4 b = rr[v];
          ru[0] = b.x; ru[1] = b.y; ru[2] = b.z; ru[3] = b.w;
        }
        uint32_t ho[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(au[j]);
          if (rr) {
            float2 g = unpack_bf16x2(ru[j]);
            // the sum is rounded to bf16 because the stored residual is what later layers see
            ho[j] = pack_bf16x2(f.x + g.x, f.y + g.y);
            f = unpack_bf16x2(ho[j]);
          }
          vals[i][2 * j] = f.x;
          vals[i][2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
        if (rr && residual_out) {
          reinterpret_cast<uint4*>(residual_out + (size_t)row * H)[v] =
              make_uint4(ho[0], ho[1], ho[2], ho[3]);
        }
      }
    }
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        uint4 wv = reinterpret_cast<const uint4*>(w)[v];
        const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 wf = unpack_bf16x2(wu[j]);
          if (zero_centered) { wf.x += 1.f; wf.y += 1.f; }
          o[j] = pack_bf16x2(vals[i][2 * j] * rstd * wf.x, vals[i][2 * j + 1] * rstd * wf.y);
        }
        reinterpret_cast<uint4*>(y + (size_t)row * H)[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres) ; dw partial[blockIdx][H] += dy * xhat
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H, int zero_centered) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dwacc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;

  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float g[NV][8];   // dy * w
    float xh[NV][8];  // x * rstd
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        uint4 a = reinterpret_cast<const uint4*>(dy + (size_t)row * H)[v];
        uint4 b = reinterpret_cast<const uint4*>(x + (size_t)row * H)[v];
        uint4 c = reinterpret_cast<const uint4*>(w)[v];
        const uint32_t au[4] = {a.x, a.y, a.z, a.w};
        const uint32_t bu[4] = {b.x, b.y, b.z, b.w};
        const uint32_t cu[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 d = unpack_bf16x2(au[j]);
          const float2 xx = unpack_bf16x2(bu[j]);
          float2 ww = unpack_bf16x2(cu[j]);
          if (zero_centered) { ww.x += 1.f; ww.y += 1.f; }
          xh[i][2 * j] = xx.x * rstd;
          xh[i][2 * j + 1] = xx.y * rstd;
          g[i][2 * j] = d.x * ww.x;
          g[i][2 * j + 1] = d.y * ww.y;
          dwacc[i][2 * j] += d.x * xh[i][2 * j];
          dwacc[i][2 * j + 1] += d.y * xh[i][2 * j + 1];
          dot += g[i][2 * j] * xh[i][2 * j] + g[i][2 * j + 1] * xh[i][2 * j + 1];
        }
      }
    }
    const float mean = block_sum(dot, red) / (float)H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        uint32_t ru[4] = {0, 0, 0, 0};
        if (dres) {
          uint4 r = reinterpret_cast<const uint4*>(dres + (size_t)row * H)[v];
          ru[0] = r.x; ru[1] = r.y; ru[2] = r.z; ru[3] = r.w;
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a0 = rstd * (g[i][2 * j] - xh[i][2 * j] * mean);
          float a1 = rstd * (g[i][2 * j + 1] - xh[i][2 * j + 1] * mean);
          if (dres) {
            const float2 r = unpack_bf16x2(ru[j]);
            a0 += r.x; a1 += r.y;
          }
          o[j] = pack_bf16x2(a0, a1);
        }
        reinterpret_cast<uint4*>(dx + (size_t)row * H)[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  float* out = dw_partial + (size_t)blockIdx.x * H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float4* o4 = reinterpret_cast<float4*>(out + v * 8);
      o4[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      o4[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// out[h] (+)= sum_p partial[p][h], fixed summation order.
__global__ void reduce_partials_kernel(const float* __restrict__ partial, int P, int H,
                                       __nv_bfloat16* __restrict__ out_bf16,
                                       float* __restrict__ out_f32, int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(size_t)p * H + h];
  if (out_f32) out_f32[h] = accumulate ? out_f32[h] + s : s;
  if (out_bf16)
    out_bf16[h] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[h]) + s : s);
}

// ---------------------------------------------------------------------------------------
// Fused per-head RMSNorm + RoPE on the q and k slices of a packed qkv activation.
// One warp per (token, head); head_dim must be 64, 128 or 256 (each lane owns D/32 contiguous
// elements of the first half pairing with the same offsets of the second half).
// qkv: [T, (Hq + 2*Hkv) * D];  out: [T, (Hq + Hkv) * D]  (q heads then k heads).
// cos/sin: [T, D/2] fp32 (already gathered by position).
// ---------------------------------------------------------------------------------------
// One warp takes QKR_HPW heads of one token: the token's cos / sin values are read once and the loads
// of all its heads are issued before the first is used (32-bit loads of bf16 pairs, 2 * QKR_HPW in
// flight per lane).
constexpr int QKR_HPW = 4;

template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_in,
                        const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                        const float* __restrict__ cosb, const float* __restrict__ sinb,
                        __nv_bfloat16* __restrict__ out, long long ld_out,
                        float* __restrict__ rstd_out, int T, int Hq, int Hkv, float eps,
                        int do_norm) {
  constexpr int HALF = D / 2;
  constexpr int PER = HALF / 32;  // elements per lane in each half (2, 1 or 4): even for D >= 128
  const int heads = Hq + Hkv;
  const int groups = (heads + QKR_HPW - 1) / QKR_HPW;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)T * groups) return;
  const int t = (int)(wid / groups);
  const int h0 = (int)(wid % groups) * QKR_HPW;
  const int lane = threadIdx.x & 31;
  float a[QKR_HPW][PER], b[QKR_HPW][PER];
#pragma unroll
  for (int g = 0; g < QKR_HPW; ++g) {
    const int h = h0 + g;
    if (h < heads) {
      const __nv_bfloat16* src = qkv + (size_t)t * ld_in + (size_t)h * D;
      if constexpr (PER % 2 == 0) {
#pragma unroll
        for (int i = 0; i < PER; i += 2) {
          const float2 va = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + lane * PER + i));
          const float2 vb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + HALF + lane * PER + i));
          a[g][i] = va.x; a[g][i + 1] = va.y;
          b[g][i] = vb.x; b[g][i + 1] = vb.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          a[g][i] = __bfloat162float(src[lane * PER + i]);
          b[g][i] = __bfloat162float(src[HALF + lane * PER + i]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) a[g][i] = b[g][i] = 0.f;
    }
  }
  float c[PER], sn[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    c[i] = __ldg(cosb + (size_t)t * HALF + lane * PER + i);
    sn[i] = __ldg(sinb + (size_t)t * HALF + lane * PER + i);
  }
#pragma unroll
  for (int g = 0; g < QKR_HPW; ++g) {
    const int h = h0 + g;
    if (h >= heads) break;                       // warp-uniform
    float rstd = 1.f;
    if (do_norm) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) ss += a[g][i] * a[g][i] + b[g][i] * b[g][i];
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / (float)D + eps);
      if (lane == 0 && rstd_out) rstd_out[(size_t)t * heads + h] = rstd;
    }
    const __nv_bfloat16* w = (h < Hq) ? wq : wk;
    __nv_bfloat16* dst = out + (size_t)t * ld_out + (size_t)h * D;
    __nv_bfloat16 o1[PER], o2[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane * PER + i;
      float x1 = a[g][i], x2 = b[g][i];
      if (do_norm) {
        // normalised value is rounded to bf16 before the rotation, as separate modules would do
        x1 = __bfloat162float(__float2bfloat16(x1 * rstd * __bfloat162float(w[e])));
        x2 = __bfloat162float(__float2bfloat16(x2 * rstd * __bfloat162float(w[HALF + e])));
      }
      o1[i] = __float2bfloat16(x1 * c[i] - x2 * sn[i]);
      o2[i] = __float2bfloat16(x2 * c[i] + x1 * sn[i]);
    }
    if constexpr (PER % 2 == 0) {
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        *reinterpret_cast<__nv_bfloat162*>(dst + lane * PER + i) = __halves2bfloat162(o1[i], o1[i + 1]);
        *reinterpret_cast<__nv_bfloat162*>(dst + HALF + lane * PER + i) = __halves2bfloat162(o2[i], o2[i + 1]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        dst[lane * PER + i] = o1[i];
        dst[HALF + lane * PER + i] = o2[i];
      }
    }
  }
}

// Backward of the above.  dout: [T, (Hq+Hkv)*D] (bf16, or fp32 when dout_f32 != nullptr, which is
// how the attention backward hands over its atomically accumulated dq).  Writes the q and k
// slices of dqkv and accumulates dw partials [gridDim.x][2][D].
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout_bf16,
                        const float* __restrict__ dout_f32_q, const float* __restrict__ dout_f32_k,
                        long long ld_dout, const __nv_bfloat16* __restrict__ qkv, long long ld_in,
                        const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                        const float* __restrict__ cosb, const float* __restrict__ sinb,
                        const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dqkv,
                        long long ld_dqkv, float* __restrict__ dw_partial, int T, int Hq, int Hkv,
                        int do_norm) {
  constexpr int HALF = D / 2;
  constexpr int PER = HALF / 32;
  const int heads = Hq + Hkv;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  float dwq_a[PER], dwq_b[PER], dwk_a[PER], dwk_b[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) dwq_a[i] = dwq_b[i] = dwk_a[i] = dwk_b[i] = 0.f;

  const long long total = (long long)T * heads;
  for (long long wid = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); wid < total;
       wid += (long long)gridDim.x * warps_per_block) {
    const int t = (int)(wid / heads);
    const int h = (int)(wid % heads);
    float g1[PER], g2[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane * PER + i;
      float d1, d2;
      if (dout_f32_q != nullptr) {
        const float* s = (h < Hq) ? dout_f32_q + ((size_t)t * Hq + h) * D
                                  : dout_f32_k + ((size_t)t * Hkv + (h - Hq)) * D;
        d1 = s[e];
        d2 = s[HALF + e];
      } else {
        const __nv_bfloat16* s = dout_bf16 + (size_t)t * ld_dout + (size_t)h * D;
        d1 = __bfloat162float(s[e]);
        d2 = __bfloat162float(s[HALF + e]);
      }
      const float c = cosb[(size_t)t * HALF + e], sn = sinb[(size_t)t * HALF + e];
      // transpose of the rotation
      g1[i] = d1 * c + d2 * sn;
      g2[i] = d2 * c - d1 * sn;
    }
    __nv_bfloat16* dst = dqkv + (size_t)t * ld_dqkv + (size_t)h * D;
    if (!do_norm) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        dst[lane * PER + i] = __float2bfloat16(g1[i]);
        dst[HALF + lane * PER + i] = __float2bfloat16(g2[i]);
      }
      continue;
    }
    const __nv_bfloat16* src = qkv + (size_t)t * ld_in + (size_t)h * D;
    const __nv_bfloat16* w = (h < Hq) ? wq : wk;
    const float rstd = rstd_in[(size_t)t * heads + h];
    float xh1[PER], xh2[PER], gw1[PER], gw2[PER];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane * PER + i;
      xh1[i] = __bfloat162float(src[e]) * rstd;
      xh2[i] = __bfloat162float(src[HALF + e]) * rstd;
      gw1[i] = g1[i] * __bfloat162float(w[e]);
      gw2[i] = g2[i] * __bfloat162float(w[HALF + e]);
      dot += gw1[i] * xh1[i] + gw2[i] * xh2[i];
      if (h < Hq) {
        dwq_a[i] += g1[i] * xh1[i];
        dwq_b[i] += g2[i] * xh2[i];
      } else {
        dwk_a[i] += g1[i] * xh1[i];
        dwk_b[i] += g2[i] * xh2[i];
      }
    }
    const float mean = warp_sum(dot) / (float)D;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      dst[lane * PER + i] = __float2bfloat16(rstd * (gw1[i] - xh1[i] * mean));
      dst[HALF + lane * PER + i] = __float2bfloat16(rstd * (gw2[i] - xh2[i] * mean));
    }
  }
  if (!do_norm || dw_partial == nullptr) return;
  // reduce the per-warp sums inside the block (fixed order), one partial row per block
  __shared__ float sh[8][2][D];
  const int wib = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    sh[wib][0][lane * PER + i] = dwq_a[i];
    sh[wib][0][HALF + lane * PER + i] = dwq_b[i];
    sh[wib][1][lane * PER + i] = dwk_a[i];
    sh[wib][1][HALF + lane * PER + i] = dwk_b[i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 2 * D; idx += blockDim.x) {
    float s = 0.f;
    for (int wv = 0; wv < warps_per_block; ++wv) s += sh[wv][idx / D][idx % D];
    dw_partial[(size_t)blockIdx.x * 2 * D + idx] = s;
  }
}

}  // namespace

XB_API int xb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y,
                          void* residual_out, float* rstd, int T, int H, float eps,
                          int zero_centered, void* stream) {
  if (H % 8 || H > NORM_THREADS * NORM_MAX_VEC * 8) return -1;
  if (T <= 0) return 0;
  const int grid = T < 148 * 8 ? T : 148 * 8;
#define XB_ARGS (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, \
      (__nv_bfloat16*)y, (__nv_bfloat16*)residual_out, rstd, T, H, eps, zero_centered
  cudaStream_t st = (cudaStream_t)stream;
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
  if (nv <= 2) rmsnorm_fwd_kernel<2><<<grid, NORM_THREADS, 0, st>>>(XB_ARGS);
  else if (nv <= 4) rmsnorm_fwd_kernel<4><<<grid, NORM_THREADS, 0, st>>>(XB_ARGS);
  else rmsnorm_fwd_kernel<8><<<grid, NORM_THREADS, 0, st>>>(XB_ARGS);
#undef XB_ARGS
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Number of partial rows the backward writes; the caller provides partial[rows * H] fp32.
XB_API int xb_rmsnorm_bwd_partial_rows(int T) {
  const int cap = xb_sm_count() * 2;
  return T < cap ? T : cap;
}

// dw (bf16 or fp32, one of them may be null) receives (accumulate ? old : 0) + sum over rows.
XB_API int xb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                          const void* dres, void* dx, float* partial, void* dw_bf16, float* dw_f32,
                          int accumulate, int T, int H, int zero_centered, void* stream) {
  if (H % 8 || H > NORM_THREADS * NORM_MAX_VEC * 8) return -1;
  if (T <= 0) return 0;
  const int rows = xb_rmsnorm_bwd_partial_rows(T);
  cudaStream_t st = (cudaStream_t)stream;
#define XB_ARGS (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, partial, T, H, zero_centered
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
  if (nv <= 2) rmsnorm_bwd_kernel<2><<<rows, NORM_THREADS, 0, st>>>(XB_ARGS);
  else if (nv <= 4) rmsnorm_bwd_kernel<4><<<rows, NORM_THREADS, 0, st>>>(XB_ARGS);
  else rmsnorm_bwd_kernel<8><<<rows, NORM_THREADS, 0, st>>>(XB_ARGS);
#undef XB_ARGS
  reduce_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(partial, rows, H,
                                                          (__nv_bfloat16*)dw_bf16, dw_f32,
                                                          accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_qk_norm_rope_fwd(const void* qkv, long long ld_in, const void* wq, const void* wk,
                               const float* cosb, const float* sinb, void* out, long long ld_out,
                               float* rstd, int T, int Hq, int Hkv, int D, float eps, int do_norm,
                               void* stream) {
  if (T <= 0) return 0;
  const long long warps = (long long)T * ((Hq + Hkv + QKR_HPW - 1) / QKR_HPW);
  const int grid = (int)((warps + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
#define XB_LAUNCH(DD)                                                                          \
  qk_norm_rope_fwd_kernel<DD><<<grid, 256, 0, st>>>(                                           \
      (const __nv_bfloat16*)qkv, ld_in, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk,    \
      cosb, sinb, (__nv_bfloat16*)out, ld_out, rstd, T, Hq, Hkv, eps, do_norm)
  if (D == 128) XB_LAUNCH(128);
  else if (D == 64) XB_LAUNCH(64);
  else if (D == 256) XB_LAUNCH(256);
  else return -1;
#undef XB_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_qk_norm_rope_bwd_partial_rows() { return xb_sm_count() * 4; }

// dout is either bf16 [T, (Hq+Hkv)*D] or two fp32 buffers [T,Hq,D] / [T,Hkv,D].
// partial: fp32 [xb_qk_norm_rope_bwd_partial_rows() * 2 * D]; dwq/dwk (bf16) accumulate flag.
XB_API int xb_qk_norm_rope_bwd(const void* dout_bf16, const float* dq_f32, const float* dk_f32,
                               long long ld_dout, const void* qkv, long long ld_in, const void* wq,
                               const void* wk, const float* cosb, const float* sinb,
                               const float* rstd, void* dqkv, long long ld_dqkv, float* partial,
                               void* dwq, void* dwk, int accumulate, int T, int Hq, int Hkv, int D,
                               int do_norm, void* stream) {
  if (T <= 0) return 0;
  const int grid = xb_qk_norm_rope_bwd_partial_rows();
  cudaStream_t st = (cudaStream_t)stream;
#define XB_LAUNCH(DD)                                                                           \
  qk_norm_rope_bwd_kernel<DD><<<grid, 256, 0, st>>>(                                            \
      (const __nv_bfloat16*)dout_bf16, dq_f32, dk_f32, ld_dout, (const __nv_bfloat16*)qkv,      \
      ld_in, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb, rstd,              \
      (__nv_bfloat16*)dqkv, ld_dqkv, partial, T, Hq, Hkv, do_norm)
  if (D == 128) XB_LAUNCH(128);
  else if (D == 64) XB_LAUNCH(64);
  else if (D == 256) XB_LAUNCH(256);
  else return -1;
#undef XB_LAUNCH
  if (do_norm && partial) {
    // partial rows are [2][D]: reduce q weights then k weights
    reduce_partials_kernel<<<(2 * D + 255) / 256, 256, 0, st>>>(partial, grid, 2 * D, nullptr,
                                                                partial, 0);
    // partial[0 .. 2D) now holds the totals; add them into the bf16 weight grads
    reduce_partials_kernel<<<1, 256, 0, st>>>(partial, 1, D, (__nv_bfloat16*)dwq, nullptr,
                                              accumulate);
    reduce_partials_kernel<<<1, 256, 0, st>>>(partial + D, 1, D, (__nv_bfloat16*)dwk, nullptr,
                                              accumulate);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward without any allocation (declared in noalloc.h).
//
// xb_rmsnorm_bwd needs a scratch buffer for the per-CTA partial sums of the weight gradient and
// leaves it to the caller to allocate.  Callers that are not allowed to allocate device memory
// (a real-time loop, a plugin that was handed all of its buffers up front, a process whose
// memory pool is owned by somebody else) use this entry point
// instead: its scratch is a fixed array that is part of the loaded library image.
//
//  * The array costs XB_NOALLOC_PARTIAL_ROWS * XB_NOALLOC_MAX_H * 4 bytes = 8 MiB on every GPU
//    that loads this library, for the life of the process.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress with
//    that device current).  Make that first call before starting any stream capture.
//  * All calls share the one array and it keeps whatever the previous call left in it.  Every
//    partial row that is read is written first by the same call, so nothing has to be cleared,
//    but two calls that run on the GPU at the same time (different streams) race on it.
//  * H above XB_NOALLOC_MAX_H or not a multiple of 8 is rejected with a negative return code and
//    a message on stderr; nothing is launched in that case.  T <= 0 returns 0 without launching.
// ---------------------------------------------------------------------------------------
#define XB_NOALLOC_MAX_H 8192
#define XB_NOALLOC_PARTIAL_ROWS 256

static __device__ __align__(256) float xb_noalloc_partial[XB_NOALLOC_PARTIAL_ROWS * XB_NOALLOC_MAX_H];

namespace {
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[64] = {nullptr};

// Device address of the scratch array on the current device, or nullptr on failure.
float* noalloc_scratch() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, xb_noalloc_partial);
    if (e != cudaSuccess) {
      fprintf(stderr, "xb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      return nullptr;
    }
    g_noalloc_ptr[dev] = p;
  }
  return g_noalloc_ptr[dev];
}
}  // namespace

XB_API int xb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                  const void* dres, void* dx, void* dw_bf16, float* dw_f32,
                                  int accumulate, int T, int H, int zero_centered, void* stream) {
  if (H <= 0 || H % 8 != 0 || H > XB_NOALLOC_MAX_H) {
    fprintf(stderr,
            "xb_rmsnorm_bwd_noalloc: H=%d is not supported (multiple of 8, at most %d); use "
            "xb_rmsnorm_bwd with a caller-provided scratch buffer for wider rows\n",
            H, XB_NOALLOC_MAX_H);
    return -1;
  }
  if (T <= 0) return 0;
  float* partial = noalloc_scratch();
  if (partial == nullptr) return -2;
  int rows = xb_sm_count() * 2;
  if (rows > XB_NOALLOC_PARTIAL_ROWS) rows = XB_NOALLOC_PARTIAL_ROWS;
  if (rows > T) rows = T;
  cudaStream_t st = (cudaStream_t)stream;
#define XB_ARGS (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, partial, T, H, zero_centered
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
  if (nv <= 2) rmsnorm_bwd_kernel<2><<<rows, NORM_THREADS, 0, st>>>(XB_ARGS);
  else rmsnorm_bwd_kernel<4><<<rows, NORM_THREADS, 0, st>>>(XB_ARGS);
#undef XB_ARGS
  // every one of the `rows` partial rows was just written by the kernel above
  reduce_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(partial, rows, H,
                                                          (__nv_bfloat16*)dw_bf16, dw_f32,
                                                          accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
