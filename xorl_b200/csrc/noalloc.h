// Entry points of libxorl_b200.so that never allocate device memory.
//
// This header has no counterpart in the reference framework: the reference is pure Python on top
// of PyTorch's caching allocator and has no notion of a caller that may not allocate.  It exists
// for users who embed these kernels where cudaMalloc (or a framework allocator) is off limits —
// in a latency-bounded loop, or in a host program that pre-partitions all GPU memory — and who
// therefore cannot provide the scratch buffer that the regular entry point asks for.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Backward of RMSNorm (same math and argument meaning as xb_rmsnorm_bwd) using a scratch area
// that lives inside the library image instead of a caller-provided buffer.
//
//   dy, x, w      bf16 inputs: upstream gradient [T, H], the layer's input before normalisation
//                 [T, H] (the kernel applies rstd itself), weight [H]
//   rstd          fp32 [T] from the forward pass
//   dres          optional bf16 [T, H] gradient of the residual stream, added into dx (may be null)
//   dx            bf16 [T, H] output
//   dw_bf16/dw_f32  weight-gradient outputs [H]; either may be null; with accumulate != 0 the
//                 result is added to what is already there
//   stream        cudaStream_t
//
// Limits: H must be a multiple of 8 and at most 8192 (the built-in scratch is 256 x 8192 floats,
// 8 MiB per GPU).  Returns 0 on success (T <= 0: nothing to do, nothing launched), -1 for an unsupported H (a message is printed), -2 when
// the scratch address could not be resolved, -11 on a launch error.
//
// The first call on each device resolves the scratch address; issue it before any stream capture.
// Calls share the scratch, so calls that overlap on the GPU race; serialise them on one stream.
int xb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                           const void* dres, void* dx, void* dw_bf16, float* dw_f32,
                           int accumulate, int T, int H, int zero_centered, void* stream);

#ifdef __cplusplus
}
#endif
