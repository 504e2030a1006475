// Optimizer kernels on flat fp32 shards: fused AdamW (master weight, both moments, bf16 copy of
// the weight written in the same pass), sum-of-squares partials for the global gradient norm,
// the device-side clip coefficient, SignSGD, and stochastic rounding fp32 -> bf16.
// Reference behaviour: torch fused AdamW as configured in src/xorl/optim/optimizer.py:114-242
// (betas 0.9/0.95, eps 1e-8, decoupled weight decay), gradient clipping in
// src/xorl/distributed/fsdp2/clip_grad_norm.py:16-57, src/xorl/optim/stochastic_round.py:22.
#include "common.cuh"

namespace {

// p, m, v, g: fp32 [n].  bf16_out (optional): the new weight rounded to bf16.
// clip_coef (optional device scalar) multiplies the gradient; grad_scale is a host scalar.
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
             const float* __restrict__ g, __nv_bfloat16* __restrict__ bf16_out, long long n,
             float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2_sqrt,
             float grad_scale, const float* __restrict__ clip_coef) {
  const float gs = grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long nvec = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float* pa = reinterpret_cast<float*>(&pp);
    float* ma = reinterpret_cast<float*>(&mm);
    float* va = reinterpret_cast<float*>(&vv);
    const float* ga = reinterpret_cast<const float*>(&gg);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = ga[j] * gs;
      pa[j] *= (1.f - lr * wd);
      ma[j] = beta1 * ma[j] + (1.f - beta1) * gr;
      va[j] = beta2 * va[j] + (1.f - beta2) * gr * gr;
      const float denom = sqrtf(va[j]) / bc2_sqrt + eps;
      pa[j] -= (lr / bc1) * (ma[j] / denom);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (bf16_out) {
      uint2 o;
      o.x = pack_bf16x2(pa[0], pa[1]);
      o.y = pack_bf16x2(pa[2], pa[3]);
      reinterpret_cast<uint2*>(bf16_out)[i] = o;
    }
  }
  // tail (n % 4)
  const long long base = nvec << 2;
  const long long i = base + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float gr = g[i] * gs;
    float pv = p[i] * (1.f - lr * wd);
    const float mv = beta1 * m[i] + (1.f - beta1) * gr;
    const float vv = beta2 * v[i] + (1.f - beta2) * gr * gr;
    pv -= (lr / bc1) * (mv / (sqrtf(vv) / bc2_sqrt + eps));
    p[i] = pv; m[i] = mv; v[i] = vv;
    if (bf16_out) bf16_out[i] = __float2bfloat16(pv);
  }
}

// partial[blockIdx] = sum of squares of this block's slice (fixed order inside the block)
__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[8];
  float acc = 0.f;
  const long long nvec = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 x = reinterpret_cast<const float4*>(g)[i];
    acc += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  if (blockIdx.x == 0) {
    for (long long i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) acc += g[i] * g[i];
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

// total[0] (+)= sum(partial[0..P))
__global__ void sum_partials_kernel(const float* __restrict__ partial, int P,
                                    float* __restrict__ total, int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    total[0] = accumulate ? total[0] + t : t;
  }
}

// norm_out = sqrt(sumsq); coef_out = min(1, max_norm / (norm + 1e-6))
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm,
                                 float* __restrict__ norm_out, float* __restrict__ coef_out) {
  const float norm = sqrtf(sumsq[0]);
  norm_out[0] = norm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  coef_out[0] = c;
}

// p -= lr * sign(g) (+ decoupled weight decay)
__global__ void __launch_bounds__(256)
signsgd_kernel(float* __restrict__ p, const float* __restrict__ g,
               __nv_bfloat16* __restrict__ bf16_out, long long n, float lr, float wd) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gr = g[i];
    float pv = p[i] * (1.f - lr * wd);
    pv -= lr * (gr > 0.f ? 1.f : (gr < 0.f ? -1.f : 0.f));
    p[i] = pv;
    if (bf16_out) bf16_out[i] = __float2bfloat16(pv);
  }
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

// Stochastic rounding: add 16 random bits below the bf16 mantissa, then truncate.
__global__ void __launch_bounds__(256)
stochastic_round_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n,
                        uint32_t seed) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    uint32_t bits = __float_as_uint(x[i]);
    const uint32_t r = hash_u32((uint32_t)i * 0x9e3779b9u + seed) & 0xffffu;
    if ((bits & 0x7f800000u) != 0x7f800000u) bits += r;
    reinterpret_cast<uint16_t*>(out)[i] = (uint16_t)(bits >> 16);
  }
}

__global__ void __launch_bounds__(256)
cast_accum_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n,
                  float scale, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(src[i]) * scale;
    dst[i] = accumulate ? dst[i] + v : v;
  }
}

}  // namespace

static inline int grid_for(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = (long long)xb_sm_count() * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// step >= 1.  Bias corrections are computed on the host.
XB_API int xb_adamw(float* p, float* m, float* v, const float* g, void* bf16_out, long long n,
                    float lr, float beta1, float beta2, float eps, float wd, int step,
                    float grad_scale, const float* clip_coef, void* stream) {
  if (n <= 0) return 0;
  const double bc1 = 1.0 - pow((double)beta1, (double)step);
  const double bc2 = 1.0 - pow((double)beta2, (double)step);
  // the tail path indexes with blockIdx*blockDim, so the grid must cover at least 3 elements
  adamw_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(
      p, m, v, g, (__nv_bfloat16*)bf16_out, n, lr, beta1, beta2, eps, wd, (float)bc1,
      (float)sqrt(bc2), grad_scale, clip_coef);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_sumsq_partial_count() { return xb_sm_count() * 4; }

// total[0] (+)= ||g||^2 ; partial must hold xb_sumsq_partial_count() floats.
XB_API int xb_sumsq(const float* g, long long n, float* partial, float* total, int accumulate,
                    void* stream) {
  const int P = xb_sumsq_partial_count();
  cudaStream_t st = (cudaStream_t)stream;
  sumsq_kernel<<<P, 256, 0, st>>>(g, n, partial);
  sum_partials_kernel<<<1, 256, 0, st>>>(partial, P, total, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_clip_coef(const float* sumsq, float max_norm, float* norm_out, float* coef_out,
                        void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sumsq, max_norm, norm_out, coef_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_signsgd(float* p, const float* g, void* bf16_out, long long n, float lr, float wd,
                      void* stream) {
  if (n <= 0) return 0;
  signsgd_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(p, g, (__nv_bfloat16*)bf16_out,
                                                                     n, lr, wd);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_stochastic_round(const float* x, void* out, long long n, unsigned seed,
                               void* stream) {
  if (n <= 0) return 0;
  stochastic_round_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
      x, (__nv_bfloat16*)out, n, seed);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dst (fp32) (+)= src (bf16) * scale
XB_API int xb_cast_accum(const void* src, float* dst, long long n, float scale, int accumulate,
                         void* stream) {
  if (n <= 0) return 0;
  cast_accum_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, dst, n, scale, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
