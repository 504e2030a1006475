// Fused MoE routing: scores -> top-k -> (re)normalised weights -> per-expert counts, one warp per
// token, no sort.  Replaces the softmax / topk / gather / bincount chain of
// src/xorl/models/layers/moe/router.py:232-259 and the Triton index kernels of
// src/xorl/ops/group_gemm/kernel/moe.py:45-433 for the routing step.
//
//   scoring 0: softmax over all experts, then top-k          (Qwen3-MoE, Mixtral)
//   scoring 1: sigmoid scores, then top-k                    (DeepSeek-V3, GLM-4.5; optional selection bias)
//   scoring 2: top-k on the logits, softmax over the k       (gpt-oss)
// The selection uses score + bias when a bias is given; the weights never include the bias.
// Ties go to the lower expert index (as torch.topk does on CPU; on CUDA torch leaves ties unordered).
#include "common.cuh"

namespace {

constexpr int MAX_PER_LANE = 16;   // up to 512 experts

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256)
route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias,
             float* __restrict__ weights, long long* __restrict__ indices, float* __restrict__ probs,
             int* __restrict__ counts, int T, int E, int k, int scoring, int renorm, float scale) {
  const int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (token >= T) return;
  const float* row = logits + (long long)token * ld;
  float x[MAX_PER_LANE], sc[MAX_PER_LANE];
  const int per = (E + 31) / 32;
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    x[j] = (j < per && e < E) ? row[e] : -INFINITY;
    m = fmaxf(m, x[j]);
  }
  m = warp_max(m);
  // scores used for the weights (p) and for the selection (sc = p + bias)
  float p[MAX_PER_LANE];
  float denom = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    const bool ok = j < per && e < E;
    float v;
    if (scoring == 1) v = ok ? 1.f / (1.f + __expf(-x[j])) : 0.f;
    else v = ok ? __expf(x[j] - m) : 0.f;
    p[j] = v;
    denom += v;
  }
  if (scoring != 1) {
    denom = warp_sum_f(denom);
    const float inv = 1.f / denom;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) p[j] *= inv;       // softmax probabilities
  }
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    const bool ok = j < per && e < E;
    if (probs && ok) probs[(long long)token * E + e] = p[j];
    // scoring 2 selects on the raw logits; the others on the (biased) score
    sc[j] = !ok ? -INFINITY : (scoring == 2 ? x[j] : p[j] + (bias ? bias[e] : 0.f));
  }
  // k rounds of warp arg-max
  float wsel = 0.f;          // lane i < k keeps the weight of the i-th choice
  int isel = 0;
  float wsum = 0.f, top_logit_max = 0.f;
  for (int i = 0; i < k; ++i) {
    float best = -INFINITY;
    int bidx = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      if (sc[j] > best) { best = sc[j]; bidx = e; }           // ascending e within a lane: first max wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; }
    }
    // the owner lane reports the unbiased score (or logit) of the chosen expert and retires it
    float val = 0.f;
    const int owner = bidx & 31, slot = bidx >> 5;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      if (j == slot && lane == owner) {
        val = scoring == 2 ? x[j] : p[j];
        sc[j] = -INFINITY;
      }
    }
    val = __shfl_sync(0xffffffffu, val, owner);
    if (i == 0) top_logit_max = val;
    if (scoring == 2) val = __expf(val - top_logit_max);      // softmax over the k selected logits
    wsum += val;
    if (lane == i) { wsel = val; isel = bidx; }
  }
  if (lane < k) {
    float w = wsel;
    if (scoring == 2 || renorm) w = w / fmaxf(wsum, 1e-20f);
    w *= scale;
    weights[(long long)token * k + lane] = w;
    indices[(long long)token * k + lane] = isel;
    if (counts) atomicAdd(counts + isel, 1);
  }
}

}  // namespace

// logits fp32 [T, E] (row stride ld); bias fp32 [E] or null; weights fp32 [T, k]; indices int64
// [T, k]; probs fp32 [T, E] or null; counts int32 [E] or null (must be zeroed by the caller).
XB_API int xb_moe_route(const float* logits, long long ld, const float* bias, float* weights,
                        long long* indices, float* probs, int* counts, int T, int E, int k, int scoring,
                        int renorm, float scale, void* stream) {
  if (T <= 0) return 0;
  if (E > 32 * MAX_PER_LANE || k > 32 || k > E || scoring < 0 || scoring > 2) return -1;
  const int warps_per_block = 8;
  const int blocks = (T + warps_per_block - 1) / warps_per_block;
  route_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(logits, ld, bias, weights, indices, probs, counts, T, E,
                                                         k, scoring, renorm, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
