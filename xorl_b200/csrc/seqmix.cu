// Small memory-bound kernels of the sequence mixers and of the 4-bit weight codecs.
//
// 1. Causal depthwise convolution over a packed batch (GatedDeltaNet q/k/v branches, Mamba2 x/B/C
//    branch): y[t, c] = act(bias[c] + sum_j w[c, j] * x[t - (K-1) + j, c]), taps that would reach
//    before the start of token t's document read zero.  Forward, and a backward in three passes
//    without atomics: dpre = dy * act'(pre) (pre recomputed), dx from dpre with the taps mirrored,
//    and per-chunk partial sums of dw / dbias that the caller adds up in a fixed order.
//    Reference behaviour: src/xorl/ops/linear_attention/ops/causal_conv1d_triton.py:24 and
//    src/xorl/ops/ssm/conv.py (conv followed by SiLU, state reset per document).
// 2. Dequantisation of 4-bit packed weights (two codes per byte, low nibble first) to bf16:
//    NF4 and INT4 with fp32 group scales, NVFP4 (e2m1 codes, e4m3 scale per group, fp32 global
//    scale), MXFP4 (e2m1 codes, e8m0 scale per group).
//    Reference behaviour: src/xorl/ops/quantize/{nf4,int4,nvfp4,mxfp4}_quantize.py.
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(w[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

// pre-activation of 8 channels of token t
__device__ __forceinline__ void conv_pre(const __nv_bfloat16* __restrict__ x, long long ldx,
                                         const __nv_bfloat16* __restrict__ w,
                                         const __nv_bfloat16* __restrict__ bias, int t, int start,
                                         int c0, int K, float (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = bias ? __bfloat162float(bias[c0 + i]) : 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = t - (K - 1) + j;
    if (src < start) continue;
    float xv[8];
    load8(x + (long long)src * ldx + c0, xv);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(w[(c0 + i) * K + j]) * xv[i];
  }
}

// mode 0: y = act(pre);  mode 1: y = dy * act'(pre)  (dy read from `aux`)
template <int MODE>
__global__ void __launch_bounds__(256)
conv1d_point_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                    const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                    const int* __restrict__ doc_start, const __nv_bfloat16* __restrict__ aux,
                    long long ldaux, __nv_bfloat16* __restrict__ out, long long ldo, int T, int C,
                    int K, int silu) {
  const int vec_per_row = C >> 3;
  const long long total = (long long)T * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / vec_per_row);
    const int c0 = (int)(idx % vec_per_row) * 8;
    float acc[8];
    conv_pre(x, ldx, w, bias, t, doc_start[t], c0, K, acc);
    float o[8];
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = silu ? acc[i] * sigmoid_f(acc[i]) : acc[i];
    } else {
      float d[8];
      load8(aux + (long long)t * ldaux + c0, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float s = sigmoid_f(acc[i]);
        o[i] = silu ? d[i] * s * (1.f + acc[i] * (1.f - s)) : d[i];
      }
    }
    store8(out + (long long)t * ldo + c0, o);
  }
}

// dx[t, c] = sum_j w[c, j] * dpre[t + (K-1) - j, c] over the tokens of the same document
__global__ void __launch_bounds__(256)
conv1d_dx_kernel(const __nv_bfloat16* __restrict__ dpre, long long ldd,
                 const __nv_bfloat16* __restrict__ w, const int* __restrict__ doc_start,
                 __nv_bfloat16* __restrict__ dx, long long ldx, int T, int C, int K) {
  const int vec_per_row = C >> 3;
  const long long total = (long long)T * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / vec_per_row);
    const int c0 = (int)(idx % vec_per_row) * 8;
    const int start = doc_start[t];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < K; ++j) {
      const int dst = t + (K - 1) - j;                 // the output token that read x[t] with tap j
      if (dst >= T || doc_start[dst] != start) continue;
      float dv[8];
      load8(dpre + (long long)dst * ldd + c0, dv);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(w[(c0 + i) * K + j]) * dv[i];
    }
    store8(dx + (long long)t * ldx + c0, acc);
  }
}

// ---- streaming forms for K = 4 (the tap count of both mixers) ---------------------------------
// One thread owns 8 channels and walks a chunk of tokens: weights and the last three input rows
// stay in registers (packed bf16, unpacked at use, which keeps the kernel near 64 registers and
// the SM well occupied), so every row of x is read once, and four rows are requested before the
// first is used.
constexpr int STREAM_THREADS = 128;
constexpr int STREAM_CHUNK = 128;

__device__ __forceinline__ uint32_t lane32(const uint4& v, int j) {
  return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

template <int MODE>
__global__ void __launch_bounds__(STREAM_THREADS, 5)
conv1d_stream4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                      const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                      const int* __restrict__ doc_start, const __nv_bfloat16* __restrict__ aux,
                      long long ldaux, __nv_bfloat16* __restrict__ out, long long ldo, int T, int C,
                      int silu) {
  const int c0 = (blockIdx.x * STREAM_THREADS + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * STREAM_CHUNK;
  const int t1 = min(T, t0 + STREAM_CHUNK);
  uint2 wq[8];                                        // the four taps of channel c0 + i
#pragma unroll
  for (int i = 0; i < 8; ++i) wq[i] = *reinterpret_cast<const uint2*>(w + (long long)(c0 + i) * 4);
  uint4 bq = make_uint4(0u, 0u, 0u, 0u);
  if (bias) bq = *reinterpret_cast<const uint4*>(bias + c0);
  uint4 h0 = make_uint4(0u, 0u, 0u, 0u), h1 = h0, h2 = h0;     // x[t-3], x[t-2], x[t-1]
  if (t0 - 3 >= 0) h0 = *reinterpret_cast<const uint4*>(x + (long long)(t0 - 3) * ldx + c0);
  if (t0 - 2 >= 0) h1 = *reinterpret_cast<const uint4*>(x + (long long)(t0 - 2) * ldx + c0);
  if (t0 - 1 >= 0) h2 = *reinterpret_cast<const uint4*>(x + (long long)(t0 - 1) * ldx + c0);
  for (int tb = t0; tb < t1; tb += 4) {
    uint4 xr[4], dr[4];
    int st[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = min(tb + u, t1 - 1);
      xr[u] = *reinterpret_cast<const uint4*>(x + (long long)t * ldx + c0);
      if (MODE == 1) dr[u] = *reinterpret_cast<const uint4*>(aux + (long long)t * ldaux + c0);
      st[u] = doc_start[t];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = tb + u;
      if (t < t1) {
        const bool m1 = t - 1 >= st[u], m2 = t - 2 >= st[u], m3 = t - 3 >= st[u];
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xc = unpack_bf16x2(lane32(xr[u], j));
          const float2 a1 = unpack_bf16x2(m1 ? lane32(h2, j) : 0u);
          const float2 a2 = unpack_bf16x2(m2 ? lane32(h1, j) : 0u);
          const float2 a3 = unpack_bf16x2(m3 ? lane32(h0, j) : 0u);
          const float2 b = unpack_bf16x2(lane32(bq, j));
          const float2 w01a = unpack_bf16x2(wq[2 * j].x), w23a = unpack_bf16x2(wq[2 * j].y);
          const float2 w01b = unpack_bf16x2(wq[2 * j + 1].x), w23b = unpack_bf16x2(wq[2 * j + 1].y);
          const float pa = b.x + w23a.y * xc.x + w23a.x * a1.x + w01a.y * a2.x + w01a.x * a3.x;
          const float pb = b.y + w23b.y * xc.y + w23b.x * a1.y + w01b.y * a2.y + w01b.x * a3.y;
          float ra, rb;
          if (MODE == 0) {
            ra = silu ? pa * sigmoid_f(pa) : pa;
            rb = silu ? pb * sigmoid_f(pb) : pb;
          } else {
            const float2 d = unpack_bf16x2(lane32(dr[u], j));
            const float sa = sigmoid_f(pa), sb = sigmoid_f(pb);
            ra = silu ? d.x * sa * (1.f + pa * (1.f - sa)) : d.x;
            rb = silu ? d.y * sb * (1.f + pb * (1.f - sb)) : d.y;
          }
          o[j] = pack_bf16x2(ra, rb);
        }
        h0 = h1; h1 = h2; h2 = xr[u];
        *reinterpret_cast<uint4*>(out + (long long)t * ldo + c0) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// dx[t] = sum_m w[., 3 - m] * dpre[t + m] over m = 0..3 with t + m in the same document
__global__ void __launch_bounds__(STREAM_THREADS, 5)
conv1d_dx_stream4_kernel(const __nv_bfloat16* __restrict__ dpre, long long ldd,
                         const __nv_bfloat16* __restrict__ w, const int* __restrict__ doc_start,
                         __nv_bfloat16* __restrict__ dx, long long ldx, int T, int C) {
  const int c0 = (blockIdx.x * STREAM_THREADS + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * STREAM_CHUNK;
  const int t1 = min(T, t0 + STREAM_CHUNK);
  uint2 wq[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) wq[i] = *reinterpret_cast<const uint2*>(w + (long long)(c0 + i) * 4);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 d0 = zero, d1 = zero, d2 = zero;              // dpre[t], dpre[t+1], dpre[t+2]
  int s0 = -1, s1 = -1, s2 = -1;                      // their document starts (-1 past the end)
  if (t0 < T) { d0 = *reinterpret_cast<const uint4*>(dpre + (long long)t0 * ldd + c0); s0 = doc_start[t0]; }
  if (t0 + 1 < T) { d1 = *reinterpret_cast<const uint4*>(dpre + (long long)(t0 + 1) * ldd + c0); s1 = doc_start[t0 + 1]; }
  if (t0 + 2 < T) { d2 = *reinterpret_cast<const uint4*>(dpre + (long long)(t0 + 2) * ldd + c0); s2 = doc_start[t0 + 2]; }
  for (int tb = t0; tb < t1; tb += 4) {
    uint4 nr[4];
    int ns[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int src = tb + u + 3;
      nr[u] = zero;
      ns[u] = -1;
      if (src < T) {
        nr[u] = *reinterpret_cast<const uint4*>(dpre + (long long)src * ldd + c0);
        ns[u] = doc_start[src];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = tb + u;
      if (t < t1) {
        const bool m1 = s1 == s0, m2 = s2 == s0, m3 = ns[u] == s0;
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 c = unpack_bf16x2(lane32(d0, j));
          const float2 a1 = unpack_bf16x2(m1 ? lane32(d1, j) : 0u);
          const float2 a2 = unpack_bf16x2(m2 ? lane32(d2, j) : 0u);
          const float2 a3 = unpack_bf16x2(m3 ? lane32(nr[u], j) : 0u);
          const float2 w01a = unpack_bf16x2(wq[2 * j].x), w23a = unpack_bf16x2(wq[2 * j].y);
          const float2 w01b = unpack_bf16x2(wq[2 * j + 1].x), w23b = unpack_bf16x2(wq[2 * j + 1].y);
          o[j] = pack_bf16x2(w23a.y * c.x + w23a.x * a1.x + w01a.y * a2.x + w01a.x * a3.x,
                             w23b.y * c.y + w23b.x * a1.y + w01b.y * a2.y + w01b.x * a3.y);
        }
        d0 = d1; d1 = d2; d2 = nr[u];
        s0 = s1; s1 = s2; s2 = ns[u];
        *reinterpret_cast<uint4*>(dx + (long long)t * ldx + c0) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// Streaming form of the weight / bias gradient for K = 4: one thread owns 8 channels of one token
// chunk (uint4 rows, four rows in flight) and writes its 8 x 5 partial sums once.
__global__ void __launch_bounds__(STREAM_THREADS, 4)
conv1d_dw_stream4_kernel(const __nv_bfloat16* __restrict__ dpre, long long ldd,
                         const __nv_bfloat16* __restrict__ x, long long ldx,
                         const int* __restrict__ doc_start, float* __restrict__ partial, int T, int C,
                         int chunk_len) {
  const int c0 = (blockIdx.x * STREAM_THREADS + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * chunk_len;
  const int t1 = min(T, t0 + chunk_len);
  float acc[8][5];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < 5; ++j) acc[i][j] = 0.f;
  }
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 h0 = zero, h1 = zero, h2 = zero;              // x[t-3], x[t-2], x[t-1]
  if (t0 < t1) {
    if (t0 - 3 >= 0) h0 = *reinterpret_cast<const uint4*>(x + (long long)(t0 - 3) * ldx + c0);
    if (t0 - 2 >= 0) h1 = *reinterpret_cast<const uint4*>(x + (long long)(t0 - 2) * ldx + c0);
    if (t0 - 1 >= 0) h2 = *reinterpret_cast<const uint4*>(x + (long long)(t0 - 1) * ldx + c0);
  }
  for (int tb = t0; tb < t1; tb += 4) {
    uint4 xr[4], dr[4];
    int st[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = min(tb + u, t1 - 1);
      xr[u] = *reinterpret_cast<const uint4*>(x + (long long)t * ldx + c0);
      dr[u] = *reinterpret_cast<const uint4*>(dpre + (long long)t * ldd + c0);
      st[u] = doc_start[t];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = tb + u;
      if (t < t1) {
        const bool m1 = t - 1 >= st[u], m2 = t - 2 >= st[u], m3 = t - 3 >= st[u];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xc = unpack_bf16x2(lane32(xr[u], j));
          const float2 a1 = unpack_bf16x2(m1 ? lane32(h2, j) : 0u);
          const float2 a2 = unpack_bf16x2(m2 ? lane32(h1, j) : 0u);
          const float2 a3 = unpack_bf16x2(m3 ? lane32(h0, j) : 0u);
          const float2 d = unpack_bf16x2(lane32(dr[u], j));
          acc[2 * j][3] += d.x * xc.x; acc[2 * j][2] += d.x * a1.x;
          acc[2 * j][1] += d.x * a2.x; acc[2 * j][0] += d.x * a3.x; acc[2 * j][4] += d.x;
          acc[2 * j + 1][3] += d.y * xc.y; acc[2 * j + 1][2] += d.y * a1.y;
          acc[2 * j + 1][1] += d.y * a2.y; acc[2 * j + 1][0] += d.y * a3.y; acc[2 * j + 1][4] += d.y;
        }
        h0 = h1; h1 = h2; h2 = xr[u];
      }
    }
  }
  float* p = partial + ((long long)blockIdx.y * C + c0) * 5;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < 5; ++j) p[i * 5 + j] = acc[i][j];
  }
}

// partial[chunk, c, 0..K-1] = sum_t dpre[t, c] * x[t - (K-1) + j, c];  partial[chunk, c, K] = sum_t dpre[t, c]
// One thread owns two adjacent channels and walks the tokens of its chunk with a register window of
// the last K inputs.
__global__ void __launch_bounds__(128)
conv1d_dw_kernel(const __nv_bfloat16* __restrict__ dpre, long long ldd,
                 const __nv_bfloat16* __restrict__ x, long long ldx,
                 const int* __restrict__ doc_start, float* __restrict__ partial, int T, int C, int K,
                 int chunk_len) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const int t0 = blockIdx.y * chunk_len;
  const int t1 = min(T, t0 + chunk_len);
  float win0[MAX_TAPS], win1[MAX_TAPS], a0[MAX_TAPS + 1], a1[MAX_TAPS + 1];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) { win0[j] = win1[j] = 0.f; }
#pragma unroll
  for (int j = 0; j <= MAX_TAPS; ++j) { a0[j] = a1[j] = 0.f; }
  // window slot j holds x[t - (K-1) + j]; preload the K-1 tokens before the chunk
  for (int j = 1; j < K; ++j) {
    const int src = t0 - K + j;
    if (src >= 0) {
      const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + (long long)src * ldx + c));
      win0[j] = f.x;
      win1[j] = f.y;
    }
  }
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j) {
      if (j < K - 1) { win0[j] = win0[j + 1]; win1[j] = win1[j + 1]; }
    }
    const float2 xc = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + (long long)t * ldx + c));
    const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dpre + (long long)t * ldd + c));
    const int start = doc_start[t];
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
      if (j == K - 1) { win0[j] = xc.x; win1[j] = xc.y; }
      if (j < K && t - (K - 1) + j >= start) {
        a0[j] += d.x * win0[j];
        a1[j] += d.y * win1[j];
      }
    }
    a0[MAX_TAPS] += d.x;
    a1[MAX_TAPS] += d.y;
  }
  float* p0 = partial + ((long long)blockIdx.y * C + c) * (K + 1);
  float* p1 = p0 + (K + 1);
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j < K) { p0[j] = a0[j]; p1[j] = a1[j]; }
  }
  p0[K] = a0[MAX_TAPS];
  p1[K] = a1[MAX_TAPS];
}

// ---------------------------------------------------------------------------------------------
__constant__ float NF4_TABLE[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
__constant__ float E2M1_TABLE[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                     -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

enum { FMT_NF4 = 0, FMT_INT4 = 1, FMT_NVFP4 = 2, FMT_MXFP4 = 3 };

// One thread decodes 8 consecutive elements (4 packed bytes); group sizes are multiples of 8, so the
// eight share one scale.
template <int FMT>
__global__ void __launch_bounds__(256)
dequant4_kernel(const uint32_t* __restrict__ packed, const void* __restrict__ scale,
                const float* __restrict__ global_scale, __nv_bfloat16* __restrict__ out,
                long long n_vec, int group) {
  const float gs = (FMT == FMT_NVFP4) ? *global_scale : 1.f;
  // code -> value table in shared memory: 16 entries in 16 banks, so lanes with different codes
  // do not serialise (a __constant__ table would, one access per distinct code)
  __shared__ float tab[16];
  if (threadIdx.x < 16)
    tab[threadIdx.x] = (FMT == FMT_NF4) ? NF4_TABLE[threadIdx.x] : E2M1_TABLE[threadIdx.x];
  __syncthreads();
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec;
       v += (long long)gridDim.x * blockDim.x) {
    const uint32_t bits = packed[v];
    const long long g = (v * 8) / group;
    float s;
    if (FMT == FMT_NF4 || FMT == FMT_INT4) {
      s = reinterpret_cast<const float*>(scale)[g];
    } else if (FMT == FMT_NVFP4) {
      const __nv_fp8_storage_t b = reinterpret_cast<const __nv_fp8_storage_t*>(scale)[g];
      s = __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
    } else {
      s = exp2f((float)reinterpret_cast<const uint8_t*>(scale)[g] - 127.f);
    }
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t code = (bits >> (4 * i)) & 0xF;
      float val;
      if (FMT == FMT_INT4) val = (float)code - 8.f;
      else val = tab[code];
      o[i] = (FMT == FMT_NVFP4) ? (val * s) * gs : val * s;
    }
    store8(out + v * 8, o);
  }
}

// Quantiser for the same four formats: one thread encodes 8 consecutive elements, the group/8 lanes
// that share a group (2, 4, 8 or 16: aligned inside a warp) agree on its absolute maximum by shuffles.
// The arithmetic follows the tensor-op definitions step by step (fp32, IEEE division, nearest table
// entry with the lower index on ties), so the codes are the ones those definitions give.
template <typename T> __device__ __forceinline__ void load8f(const T* p, float* v);
template <> __device__ __forceinline__ void load8f<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void load8f<float>(const float* p, float* v) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <int N> __device__ __forceinline__ uint32_t nearest_code(float x, const float* tab) {
  uint32_t best = 0;
  float bd = fabsf(x - tab[0]);
#pragma unroll
  for (int i = 1; i < N; ++i) {
    const float d = fabsf(x - tab[i]);
    if (d < bd) { bd = d; best = i; }
  }
  return best;
}

template <int FMT, typename T>
__global__ void __launch_bounds__(256)
quant4_kernel(const T* __restrict__ w, const float* __restrict__ gmax, uint32_t* __restrict__ packed,
              void* __restrict__ scale, float* __restrict__ global_scale_out, long long n_vec, int group) {
  __shared__ float tab[16];
  if (threadIdx.x < 16)
    tab[threadIdx.x] = (FMT == FMT_NF4) ? NF4_TABLE[threadIdx.x] : E2M1_TABLE[threadIdx.x];
  __syncthreads();
  float gs = 1.f;
  if (FMT == FMT_NVFP4) {
    gs = fmaxf(*gmax, 1e-12f) / (6.0f * 448.0f);
    if (blockIdx.x == 0 && threadIdx.x == 0) *global_scale_out = gs;
  }
  const int lanes = group >> 3;                        // lanes that share a group
  const long long stride = (long long)gridDim.x * blockDim.x;
  // the loop bound is warp-uniform (rounded up to a warp) so that the shuffles below are convergent
  const long long n_round = (n_vec + 31) / 32 * 32;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_round; v += stride) {
    float x[8];
    const bool live = v < n_vec;
    if (live) load8f<T>(w + v * 8, x);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    for (int o = 1; o < lanes; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) continue;
    const long long g = (v * 8) / group;
    const bool writer = ((v * 8) % group) == 0;
    uint32_t bits = 0;
    if (FMT == FMT_NF4) {
      const float s = fmaxf(amax, 1e-12f);
      if (writer) reinterpret_cast<float*>(scale)[g] = s;
#pragma unroll
      for (int i = 0; i < 8; ++i) bits |= nearest_code<16>(x[i] / s, tab) << (4 * i);
    } else if (FMT == FMT_INT4) {
      const float s = fmaxf(amax, 1e-12f) / 7.0f;
      if (writer) reinterpret_cast<float*>(scale)[g] = s;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float q = fminf(fmaxf(rintf(x[i] / s), -8.f), 7.f) + 8.f;
        bits |= (uint32_t)q << (4 * i);
      }
    } else {
      float denom;
      if (FMT == FMT_NVFP4) {
        const float bs = fminf(fmaxf(amax / 6.0f / gs, 1e-12f), 448.0f);
        const __nv_fp8_storage_t b8 = __nv_cvt_float_to_fp8(bs, __NV_SATFINITE, __NV_E4M3);
        if (writer) reinterpret_cast<__nv_fp8_storage_t*>(scale)[g] = b8;
        denom = fmaxf(__half2float(__half(__nv_cvt_fp8_to_halfraw(b8, __NV_E4M3))) * gs, 1e-30f);
      } else {
        const float a = fmaxf(amax, 1.17549435e-38f);                       // 2^-126
        const float e = fminf(fmaxf(ceilf(log2f(a / 6.0f)), -127.f), 127.f);
        if (writer) reinterpret_cast<uint8_t*>(scale)[g] = (uint8_t)(e + 127.f);
        denom = exp2f(e);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float q = x[i] / denom;
        bits |= (nearest_code<8>(fabsf(q), tab) | (q < 0.f ? 8u : 0u)) << (4 * i);
      }
    }
    packed[v] = bits;
  }
}

inline int grid_for(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = (long long)xb_sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

inline dim3 stream_grid(int T, int C) {
  return dim3((C / 8 + STREAM_THREADS - 1) / STREAM_THREADS, (T + STREAM_CHUNK - 1) / STREAM_CHUNK);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// x [T, C] (row stride ldx), w [C, K], bias [C] or null, doc_start [T] (index of the first token of
// each token's document) -> y [T, C].  C % 8 == 0, row strides % 8 == 0, K <= 8.
XB_API int xb_causal_conv1d_fwd(const void* x, long long ldx, const void* w, const void* bias,
                                const int* doc_start, void* y, long long ldy, int T, int C, int K,
                                int silu, void* stream) {
  if (C % 8 || ldx % 8 || ldy % 8 || K < 1 || K > MAX_TAPS || !aligned16(x) || !aligned16(y))
    return -1;
  if (T <= 0) return 0;
  if (K == 4) {
    conv1d_stream4_kernel<0><<<stream_grid(T, C), STREAM_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias,
        doc_start, nullptr, 0, (__nv_bfloat16*)y, ldy, T, C, silu);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  conv1d_point_kernel<0><<<grid_for((long long)T * (C / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, doc_start,
      nullptr, 0, (__nv_bfloat16*)y, ldy, T, C, K, silu);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Number of token chunks (rows of `partial`) the backward writes for T tokens.
XB_API int xb_causal_conv1d_bwd_chunks(int T) {
  const int c = (T + 255) / 256;
  return c < 1 ? 1 : (c > 128 ? 128 : c);
}

// dy, x [T, C]; dpre [T, C] bf16 workspace (may alias nothing else); dx [T, C];
// partial [chunks, C, K + 1] fp32 (taps, then the bias column).
XB_API int xb_causal_conv1d_bwd(const void* dy, long long lddy, const void* x, long long ldx,
                                const void* w, const void* bias, const int* doc_start, void* dpre,
                                void* dx, long long lddx, float* partial, int T, int C, int K,
                                int silu, void* stream) {
  if (C % 8 || ldx % 8 || lddy % 8 || lddx % 8 || K < 1 || K > MAX_TAPS || !aligned16(x) ||
      !aligned16(dy) || !aligned16(dx) || !aligned16(dpre))
    return -1;
  if (T <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for((long long)T * (C / 8), 256);
  if (K == 4) {
    conv1d_stream4_kernel<1><<<stream_grid(T, C), STREAM_THREADS, 0, st>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias,
        doc_start, (const __nv_bfloat16*)dy, lddy, (__nv_bfloat16*)dpre, C, T, C, silu);
    conv1d_dx_stream4_kernel<<<stream_grid(T, C), STREAM_THREADS, 0, st>>>(
        (const __nv_bfloat16*)dpre, C, (const __nv_bfloat16*)w, doc_start, (__nv_bfloat16*)dx,
        lddx, T, C);
  } else {
    conv1d_point_kernel<1><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias,
        doc_start, (const __nv_bfloat16*)dy, lddy, (__nv_bfloat16*)dpre, C, T, C, K, silu);
    conv1d_dx_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dpre, C, (const __nv_bfloat16*)w,
                                           doc_start, (__nv_bfloat16*)dx, lddx, T, C, K);
  }
  const int chunks = xb_causal_conv1d_bwd_chunks(T);
  const int chunk_len = (T + chunks - 1) / chunks;
  if (K == 4) {
    dim3 g((C / 8 + STREAM_THREADS - 1) / STREAM_THREADS, chunks);
    conv1d_dw_stream4_kernel<<<g, STREAM_THREADS, 0, st>>>(
        (const __nv_bfloat16*)dpre, C, (const __nv_bfloat16*)x, ldx, doc_start, partial, T, C,
        chunk_len);
  } else {
    dim3 g((C / 2 + 127) / 128, chunks);
    conv1d_dw_kernel<<<g, 128, 0, st>>>((const __nv_bfloat16*)dpre, C, (const __nv_bfloat16*)x, ldx,
                                        doc_start, partial, T, C, K, chunk_len);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// packed: n / 2 bytes; scale: n / group entries (fp32 for nf4 / int4, one byte for nvfp4 / mxfp4);
// out: n bf16.  n % 8 == 0, group % 8 == 0.
XB_API int xb_dequant4(const void* packed, const void* scale, const float* global_scale, void* out,
                       long long n, int group, int fmt, void* stream) {
  if (n % 8 || group % 8 || group <= 0 || !aligned16(out) ||
      (reinterpret_cast<uintptr_t>(packed) & 3))
    return -1;
  if (fmt == FMT_NVFP4 && !global_scale) return -1;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const long long nv = n / 8;
  const int grid = grid_for(nv, 256);
  const uint32_t* p = (const uint32_t*)packed;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  switch (fmt) {
    case FMT_NF4: dequant4_kernel<FMT_NF4><<<grid, 256, 0, st>>>(p, scale, global_scale, o, nv, group); break;
    case FMT_INT4: dequant4_kernel<FMT_INT4><<<grid, 256, 0, st>>>(p, scale, global_scale, o, nv, group); break;
    case FMT_NVFP4: dequant4_kernel<FMT_NVFP4><<<grid, 256, 0, st>>>(p, scale, global_scale, o, nv, group); break;
    case FMT_MXFP4: dequant4_kernel<FMT_MXFP4><<<grid, 256, 0, st>>>(p, scale, global_scale, o, nv, group); break;
    default: return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// w: n elements (bf16 when w_fp32 == 0, else fp32); packed: n / 2 bytes; scale: n / group entries (fp32
// for nf4 / int4, one byte for nvfp4 / mxfp4).  nvfp4 also takes gmax (device fp32: max |w| over the whole
// tensor) and writes the fp32 global scale.  n % 8 == 0; group in {16, 32, 64, 128}.
XB_API int xb_quant4(const void* w, int w_fp32, const float* gmax, void* packed, void* scale,
                     float* global_scale_out, long long n, int group, int fmt, void* stream) {
  if (n % 8 || !(group == 16 || group == 32 || group == 64 || group == 128) || n % group || !aligned16(w) ||
      (reinterpret_cast<uintptr_t>(packed) & 3))
    return -1;
  if (fmt == FMT_NVFP4 && (!gmax || !global_scale_out)) return -1;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const long long nv = n / 8;
  const int grid = grid_for(nv, 256);
  uint32_t* p = (uint32_t*)packed;
#define XB_Q4(F)                                                                                          \
  do {                                                                                                    \
    if (w_fp32) quant4_kernel<F, float><<<grid, 256, 0, st>>>((const float*)w, gmax, p, scale,            \
                                                              global_scale_out, nv, group);               \
    else quant4_kernel<F, __nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, gmax, p, scale,    \
                                                               global_scale_out, nv, group);              \
  } while (0)
  switch (fmt) {
    case FMT_NF4: XB_Q4(FMT_NF4); break;
    case FMT_INT4: XB_Q4(FMT_INT4); break;
    case FMT_NVFP4: XB_Q4(FMT_NVFP4); break;
    case FMT_MXFP4: XB_Q4(FMT_MXFP4); break;
    default: return -1;
  }
#undef XB_Q4
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
