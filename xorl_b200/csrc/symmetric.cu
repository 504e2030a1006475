// Mirror of the block-lower triangle of a square matrix into its upper part:
// C[i, j] = C[j, i] for every (i, j) whose row block (of `block` rows) lies above its column block.
// Used by the symmetric GEMM of the Muon Newton-Schulz iteration (X X^T, A A, P A P): the panels
// on and below the block diagonal are computed by the tcgen05 GEMM, the rest is copied, which is
// the contract of the reference's triangle-only GEMM (src/xorl/ops/quack/gemm_symmetric.py, used by
// src/xorl/optim/gram_newton_schulz.py).
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
mirror_lower_kernel(T* __restrict__ C, long long ld, int M, int block) {
  __shared__ T tile[32][33];
  const int tr = blockIdx.y, tc = blockIdx.x;              // destination tile (rows tr, cols tc)
  if ((tr * 32) / block >= (tc * 32) / block) return;       // on or below the block diagonal
  // A 32 x 32 tile never straddles a block border (block is a multiple of 32).
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8 threads
  for (int r = ty; r < 32; r += 8) {
    const int i = tc * 32 + r, j = tr * 32 + tx;           // source element C[i, j] (lower part)
    if (i < M && j < M) tile[r][tx] = C[(long long)i * ld + j];
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int i = tr * 32 + r, j = tc * 32 + tx;           // destination C[i, j] = source C[j, i]
    if (i < M && j < M) C[(long long)i * ld + j] = tile[tx][r];
  }
}

}  // namespace

XB_API int xb_mirror_lower(void* C, long long ld, int M, int block, int is_fp32, void* stream) {
  if (M <= 0) return 0;
  if (block <= 0 || block % 32) return -1;
  const int tiles = (M + 31) / 32;
  dim3 grid(tiles, tiles);
  if (is_fp32)
    mirror_lower_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((float*)C, ld, M, block);
  else
    mirror_lower_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)C, ld, M, block);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
