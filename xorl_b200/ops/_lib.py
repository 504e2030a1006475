"""ctypes binding to ``libxorl_b200.so`` (CUDA kernels) and ``libxorl_b200_host.so`` (C++ host
runtime).

The kernels take raw device pointers and the CUDA stream handle; tensors stay owned by PyTorch.
On a machine with a GPU the CUDA library is mandatory: ``cuda_lib()`` raises if it cannot be
loaded, so no operator can silently fall back to a PyTorch implementation there.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p
from pathlib import Path

import torch

_LIBDIR = Path(__file__).resolve().parent.parent / "lib"
_lock = threading.Lock()
_cuda_lib = None
_host_lib = None

P = c_void_p
I = c_int
L = c_longlong
F = c_float

# name -> argtypes (restype is always int unless listed in _RESTYPES)
_SIGNATURES = {
    "xb_status_read": [P, I],
    "xb_device_sm_count": [],
    "xb_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, P],
    "xb_gemm_set_batch_invariant": [I],
    "xb_gemm_bf16_pair": [P, P, P, I, I, I, L, L, L, I, I, I, I, P],
    "xb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, I, P],
    "xb_rmsnorm_bwd_partial_rows": [I],
    "xb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, I, P],
    "xb_qk_norm_rope_fwd": [P, L, P, P, P, P, P, L, P, I, I, I, I, F, I, P],
    "xb_qk_norm_rope_bwd_partial_rows": [],
    "xb_qk_norm_rope_bwd": [P, P, P, L, P, L, P, P, P, P, P, P, L, P, P, P, I, I, I, I, I, I, P],
    "xb_swiglu_fwd": [P, P, L, I, I, P],
    "xb_swiglu_bwd": [P, P, P, L, I, P],
    "xb_swiglu_fwd_rows": [P, P, L, I, I, P, P],
    "xb_swiglu_bwd_rows": [P, P, P, L, I, P, P],
    "xb_quant_mx_rows_lim": [P, L, P, L, P, I, L, I, P, P],
    "xb_embedding_fwd": [P, P, P, I, I, L, P],
    "xb_embedding_bwd": [P, P, P, I, I, I, L, P],
    "xb_add_bf16": [P, P, P, L, P],
    "xb_cross_entropy": [P, L, P, P, P, I, I, L, F, I, F, P],
    "xb_cross_entropy_rows": [P, L, P, P, P, P, I, I, L, F, I, P],
    "xb_cross_entropy_vp_stats": [P, L, P, P, I, I, L, L, P],
    "xb_cross_entropy_vp_grad": [P, L, P, P, I, I, L, L, F, P],
    "xb_adamw": [P, P, P, P, P, L, F, F, F, F, F, I, F, P, P],
    "xb_sumsq_partial_count": [],
    "xb_sumsq": [P, L, P, P, I, P],
    "xb_clip_coef": [P, F, P, P, P],
    "xb_signsgd": [P, P, P, L, F, F, P],
    "xb_stochastic_round": [P, P, L, c_uint, P],
    "xb_cast_accum": [P, P, L, F, I, P],
    "xb_symm_barrier": [P, I, I, I, I, I, P],
    "xb_symm_wait": [P, I, I, I, I, P],
    "xb_symm_allgather": [P, P, L, I, I, I, P],
    "xb_symm_allgather_dma": [P, P, L, I, I, P],
    "xb_symm_gather_slices_dma": [P, P, L, L, I, I, P],
    "xb_symm_reduce_scatter": [P, P, ctypes.c_ulonglong, L, L, I, F, P, P, I, I, I, I, I, I, I, I, P],
    "xb_ep_exchange_counts": [P, P, P, I, I, I, I, I, I, P],
    "xb_ep_prepare_recv": [P, P, P, P, I, I, I, P],
    "xb_ep_push_rows": [P, L, P, P, P, P, I, I, I, P, L, P, P, I, I, I, I, I, P],
    "xb_peer_copy": [P, P, L, I, P],
    "xb_peer_copy_2d": [P, L, P, L, L, L, P],
    "xb_gemm_fused": [P, P],
    "xb_rs_reduce": [P, I, I, I, P, L, P, P],
    "xb_moe_route": [P, L, P, P, P, P, P, I, I, I, I, I, F, P],
    "xb_moe_histogram": [P, I, P, I, P],
    "xb_ep_meta_targets": [P, I, P, P, P],
    "xb_ep_plan": [P, I, P, I, I, I, I, I, P, P, P, P, P, P],
    "xb_moe_gather_rows": [P, L, P, L, P, P, I, I, P],
    "xb_moe_gather_sum": [P, L, P, L, P, P, I, I, I, P],
    "xb_moe_slot_dots": [P, P, L, P, L, P, I, I, I, P],
    "xb_attn_bwd_set_split": [I],
    "xb_block_fp8_gemm": [P, P, P, P, P, I, I, I, P],
    "xb_block_fp8_gemm_ex": [P, P, P, P, P, I, I, I, L, L, L, L, L, P],
    "xb_quant_fp8_rows": [P, L, P, L, P, L, I, I, P],
    "xb_quant_fp8_blocks": [P, L, P, L, P, L, I, I, P],
    "xb_dequant_fp8_blocks": [P, L, P, L, P, L, I, I, P],
    "xb_grouped_gemm_rows": [P, P, P, P, I, L, I, I, L, L, I, P],
    "xb_grouped_gemm_wgrad": [P, P, P, P, I, L, I, I, L, L, I, I, P],
    "xb_grouped_gemm_mx_rows": [P, P, P, P, P, P, I, L, I, I, L, L, I, I, P],
    "xb_quant_mx_rows": [P, L, P, L, P, I, L, I, P],
    "xb_quant_mx_weight": [P, P, P, I, P, P, I, I, I, I, P],
    "xb_attn_fwd_sink": [P, P, P, P, P, P, P, P, L, L, L, L, I, I, I, I, I, I, I, F, I, P],
    "xb_attn_fwd_ex": [P, P, P, P, P, P, P, L, L, L, L, I, I, I, I, I, I, I, F, I, P],
    "xb_attn_bwd_ex": [P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, L, L, L, I, I, I, I, I, I, I, F, I, I, P],
    "xb_attn_fwd": [P, P, P, P, P, P, L, L, L, L, I, I, I, I, I, I, F, I, P],
    "xb_attn_bwd": [P, P, P, P, P, P, P, P, P, P, P, L, L, L, L, L, L, I, I, I, I, I, I, F, I, P],
    "xb_causal_conv1d_fwd": [P, L, P, P, P, P, L, I, I, I, I, P],
    "xb_causal_conv1d_bwd_chunks": [I],
    "xb_causal_conv1d_bwd": [P, L, P, L, P, P, P, P, P, L, P, I, I, I, I, P],
    "xb_dequant4": [P, P, P, P, L, I, I, P],
    "xb_quant4": [P, I, P, P, P, P, L, I, I, P],
    "xb_mirror_lower": [P, L, I, I, I, P],
}


class NativeLibraryMissing(RuntimeError):
    pass


def _declare(lib, table) -> None:
    for name, argtypes in table.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


def cuda_lib_path() -> Path:
    return _LIBDIR / "libxorl_b200.so"


def cuda_lib():
    """The CUDA kernel library.  Raises NativeLibraryMissing when it has not been built."""
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                path = cuda_lib_path()
                if not path.exists():
                    raise NativeLibraryMissing(
                        f"{path} not found: run `python -m xorl_b200._build` (needs nvcc) first")
                lib = ctypes.CDLL(str(path))
                _declare(lib, _SIGNATURES)
                _cuda_lib = lib
    return _cuda_lib


def have_cuda_lib() -> bool:
    return cuda_lib_path().exists()


def host_lib():
    """The C++ host runtime (packing, schedules, delta codec).  Built on demand with g++."""
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                path = _LIBDIR / "libxorl_b200_host.so"
                if not path.exists():
                    from .. import _build
                    _build.build_host()
                _host_lib = ctypes.CDLL(str(path))
    return _host_lib


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def read_status(clear: bool = True) -> list[int]:
    """Synchronises the device and returns its 8 status words (all zero when no kernel gave up
    on a bounded wait)."""
    buf = (c_int * 8)()
    check(cuda_lib().xb_status_read(buf, 1 if clear else 0), "xb_status_read")
    return list(buf)


class DeviceWaitTimeout(RuntimeError):
    """A kernel abandoned a bounded wait (mbarrier or peer flag) and returned early."""


def raise_on_status() -> None:
    st = read_status(clear=True)
    if st[0] != 0:
        raise DeviceWaitTimeout(
            f"kernel {st[1]} block {st[2]} reported status {st[0]} (detail {st[3]})")
