// Cross-entropy over a chunk of logits: online-softmax forward that also writes the gradient
// in place, so a [tokens, vocab] tensor is only ever materialised one token-chunk at a time and
// only in bf16.  Also the vocab-parallel form (per-shard max / sum-exp / target logit).
// Reference behaviour: src/xorl/ops/loss/causallm_loss.py:445-864 (chunked lm-head loss, sum
// reduction, ignore_index = -100) and src/xorl/ops/loss/vocab_parallel_cross_entropy.py:34-165.
#include "common.cuh"

namespace {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void ms_combine(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  const float e1 = (m == -INFINITY) ? 0.f : __expf(m - mn);
  const float e2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
  s = s * e1 + s2 * e2;
  m = mn;
}

// combine (max, sumexp) pairs: first inside the warp, then across warps
__device__ __forceinline__ void block_reduce_max_sum(float& m, float& s, float* sm, float* ss) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    ms_combine(m, s, m2, s2);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sm[w] = m; ss[w] = s; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    float mm = l < nw ? sm[l] : -INFINITY, s3 = l < nw ? ss[l] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s3, o);
      ms_combine(mm, s3, m2, s2);
    }
    if (l == 0) { sm[0] = mm; ss[0] = s3; }
  }
  __syncthreads();
  m = sm[0];
  s = ss[0];
}

// One CTA per row.  logits [rows, ld] bf16 (vocab V, columns >= V ignored).
// mode 0: full CE.  Writes loss[row] = lse - logit[target] (0 when target == ignore_index),
//         lse[row], and if write_grad: logits <- (softmax - onehot) * grad_scale (0 for ignored).
// mode 1: statistics only (vocab-parallel): stats[row] = {max, sumexp, target_logit or 0}
//         for the local vocab range [vocab_start, vocab_start + V).
__global__ void __launch_bounds__(CE_THREADS)
ce_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
          float* __restrict__ loss, float* __restrict__ lse_out, float* __restrict__ stats, int V,
          long long ignore_index, float grad_scale, int write_grad, int mode,
          long long vocab_start, float z_loss_coef, const float* __restrict__ row_scale) {
  __shared__ float sm[32], ss[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    const uint4 a = reinterpret_cast<const uint4*>(lr)[v];
    const uint32_t au[4] = {a.x, a.y, a.z, a.w};
    float f[8];
    float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p = unpack_bf16x2(au[j]);
      f[2 * j] = p.x; f[2 * j + 1] = p.y;
      lm = fmaxf(lm, fmaxf(p.x, p.y));
    }
    const float mn = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - mn);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + acc;
    m = mn;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    const float x = __bfloat162float(lr[c]);
    ms_combine(m, s, x, 1.f);
  }
  if (m == -INFINITY) s = 0.f;
  block_reduce_max_sum(m, s, sm, ss);

  const long long tgt = targets[row];
  if (mode == 1) {
    if (threadIdx.x == 0) {
      const long long lt = tgt - vocab_start;
      const bool mine = tgt != ignore_index && lt >= 0 && lt < V;
      stats[row * 3 + 0] = m;
      stats[row * 3 + 1] = s;
      stats[row * 3 + 2] = mine ? __bfloat162float(lr[lt]) : 0.f;
    }
    return;
  }
  const float lse = m + __logf(s);
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignored) l = lse - __bfloat162float(lr[tgt]) + z_loss_coef * lse * lse;
    loss[row] = l;
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // the target logit has been read
  const float gs = ignored ? 0.f : grad_scale * (row_scale ? row_scale[row] : 1.f);
  const float zfac = 1.f + 2.f * z_loss_coef * lse;  // d(lse + z*lse^2)/d(lse)
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    const uint4 a = reinterpret_cast<const uint4*>(lr)[v];
    const uint32_t au[4] = {a.x, a.y, a.z, a.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p = unpack_bf16x2(au[j]);
      const int c0 = v * 8 + 2 * j;
      float g0 = __expf(p.x - lse) * zfac, g1 = __expf(p.y - lse) * zfac;
      if (c0 == tgt) g0 -= 1.f;
      if (c0 + 1 == tgt) g1 -= 1.f;
      o[j] = pack_bf16x2(g0 * gs, g1 * gs);
    }
    reinterpret_cast<uint4*>(lr)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[c]) - lse) * zfac;
    if (c == tgt) g -= 1.f;
    lr[c] = __float2bfloat16(g * gs);
  }
}

// Vocab-parallel backward: logits <- (exp(logit - lse_global) - onehot_local) * grad_scale
__global__ void __launch_bounds__(CE_THREADS)
ce_vp_grad_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                  const long long* __restrict__ targets, const float* __restrict__ lse, int V,
                  long long ignore_index, float grad_scale, long long vocab_start) {
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long tgt = targets[row];
  const float gs = (tgt == ignore_index) ? 0.f : grad_scale;
  const long long lt = tgt - vocab_start;
  const float l = lse[row];
  for (int c = threadIdx.x; c < V; c += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[c]) - l);
    if (c == lt) g -= 1.f;
    lr[c] = __float2bfloat16(g * gs);
  }
}

}  // namespace

// logits: [rows, ld] bf16, rewritten with the gradient when write_grad != 0.
XB_API int xb_cross_entropy(void* logits, long long ld, const long long* targets, float* loss,
                            float* lse, int rows, int V, long long ignore_index, float grad_scale,
                            int write_grad, float z_loss_coef, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) % 16)) return -1;
  ce_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, ld, targets, loss, lse, nullptr, V, ignore_index, grad_scale,
      write_grad, 0, 0, z_loss_coef, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// stats: [rows, 3] fp32 = (local max, local sum-exp relative to that max, local target logit)
XB_API int xb_cross_entropy_vp_stats(void* logits, long long ld, const long long* targets,
                                     float* stats, int rows, int V_local, long long vocab_start,
                                     long long ignore_index, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) % 16)) return -1;
  ce_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, ld, targets, nullptr, nullptr, stats, V_local, ignore_index, 0.f, 0,
      1, vocab_start, 0.f, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

XB_API int xb_cross_entropy_vp_grad(void* logits, long long ld, const long long* targets,
                                    const float* lse, int rows, int V_local, long long vocab_start,
                                    long long ignore_index, float grad_scale, void* stream) {
  if (rows <= 0) return 0;
  ce_vp_grad_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, ld, targets, lse, V_local, ignore_index, grad_scale, vocab_start);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// As xb_cross_entropy with a per-row gradient weight: the gradient of row r is multiplied by
// grad_scale * row_scale[r].  Used for losses that are functions of per-token log-probabilities.
XB_API int xb_cross_entropy_rows(void* logits, long long ld, const long long* targets, float* loss,
                                 float* lse, const float* row_scale, int rows, int V,
                                 long long ignore_index, float grad_scale, int write_grad,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) % 16)) return -1;
  ce_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, ld, targets, loss, lse, nullptr, V, ignore_index, grad_scale,
      write_grad, 0, 0, 0.f, row_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
