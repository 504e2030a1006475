"""GEMMs whose collective runs inside the same kernel (``csrc/gemm_fused.cu``).

``ag_gemm``   all-gather -> GEMM: one operand is sharded by rows over the ranks; communication warps
              of the GEMM kernel pull the peers' shards over NVLink chunk by chunk while the tensor
              cores work on the chunks that have arrived.
``gemm_rs``   GEMM -> reduce-scatter: every rank writes its partial result into its symmetric buffer,
              owners are signalled block by block, pull the peers' blocks of their rows over NVLink
              while the remaining tiles are computed, and sum all partials in fp32.

These are the building blocks of tensor-parallel linears with sequence-parallel activations
(``parallel/tp_fused.py``); the reference runs the same linears as DTensor collectives around cuBLAS
(src/xorl/distributed/torch_parallelize.py:222-270).  ``peers`` carries the symmetric-memory
addresses of every rank; with ``peers.flags is None`` all "ranks" are buffers of one device and the
kernel runs without handshakes (how the data path is tested on a single GPU).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib


class _Args(ctypes.Structure):
    _fields_ = [
        ("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("C", ctypes.c_void_p),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
        ("lda", ctypes.c_longlong), ("ldb", ctypes.c_longlong), ("ldc", ctypes.c_longlong),
        ("b_mn", ctypes.c_int), ("out_fp32", ctypes.c_int), ("accumulate", ctypes.c_int),
        ("rank", ctypes.c_int), ("nranks", ctypes.c_int),
        ("gather", ctypes.c_int), ("scatter", ctypes.c_int),
        ("shard_ptrs", ctypes.c_ulonglong * 16),
        ("rows_per_rank", ctypes.c_longlong),
        ("ready_counters", ctypes.c_ulonglong),
        ("ready_target", ctypes.c_ulonglong),
        ("partial_ptrs", ctypes.c_ulonglong * 16),
        ("pulled", ctypes.c_void_p), ("out", ctypes.c_void_p), ("ldo", ctypes.c_longlong), ("residual", ctypes.c_void_p),
        ("counters", ctypes.c_ulonglong),
        ("flag_ptrs", ctypes.c_ulonglong * 16),
        ("ready_slot", ctypes.c_int), ("done_slot", ctypes.c_int),
        ("epoch", ctypes.c_int), ("done_needed", ctypes.c_int),
        ("wait_ms", ctypes.c_int), ("ctas_out", ctypes.c_int),
    ]


@dataclass
class Peers:
    """Who takes part in a fused collective GEMM.  ``flags``: symmetric flag-area addresses of all
    ranks (int32 arrays), or None for a single-device run."""
    rank: int
    nranks: int
    flags: Optional[Sequence[int]] = None
    ready_slot: int = 0
    done_slot: int = 16
    wait_ms: int = 2000


_launches = 0
_state: Dict[Tuple, Dict] = {}      # per device: counters shared by all calls of one shape


def launch_count() -> int:
    return _launches


def _shape_state(dev: torch.device, key: Tuple, num_chunks: int) -> Dict:
    k = (dev.index, *key)
    st = _state.get(k)
    if st is None:
        st = {"ready": torch.zeros(max(num_chunks, 1), device=dev, dtype=torch.int64), "base": 0,
              "counters": torch.zeros(1024, device=dev, dtype=torch.int32)}
        _state[k] = st
    return st


def _check_bf16(*ts: torch.Tensor) -> None:
    for t in ts:
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0


def ag_gemm(full: torch.Tensor, shard_ptrs: Sequence[int], rows_per_rank: int, other: torch.Tensor,
            peers: Peers, *, gathered: str = "a", b_mn: bool = False, epoch: int = 0,
            out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """C = A @ op(B)^T where the rows of ``full`` (A if ``gathered == "a"``, else B) are pulled from
    ``shard_ptrs`` (rank r holds rows [r * rows_per_rank, (r + 1) * rows_per_rank)) by the kernel
    itself.  ``full`` is this rank's gathered copy and is valid after the call."""
    global _launches
    assert gathered in ("a", "b")
    a, b = (full, other) if gathered == "a" else (other, full)
    _check_bf16(a, b)
    M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb and full.is_contiguous() and len(shard_ptrs) == peers.nranks
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    chunk_rows = 512 if gathered == "a" else 256
    num_chunks = (full.shape[0] + chunk_rows - 1) // chunk_rows
    st = _shape_state(a.device, ("ag", gathered, M, N, K), num_chunks)
    args = _Args()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.M, args.N, args.K = M, N, K
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.b_mn, args.out_fp32, args.accumulate = int(b_mn), int(out.dtype == torch.float32), 0
    args.rank, args.nranks = peers.rank, peers.nranks
    args.gather, args.scatter = (1 if gathered == "a" else 2), 0
    for r, ptr in enumerate(shard_ptrs):
        args.shard_ptrs[r] = ptr
    args.rows_per_rank = rows_per_rank
    args.ready_counters = st["ready"].data_ptr()
    args.ready_target = st["base"]
    args.counters = st["counters"].data_ptr()
    if peers.flags is not None:
        for r, ptr in enumerate(peers.flags):
            args.flag_ptrs[r] = ptr
    args.ready_slot, args.done_slot = peers.ready_slot, peers.done_slot
    args.epoch, args.done_needed, args.wait_ms = epoch, 0, peers.wait_ms
    _lib.check(_lib.cuda_lib().xb_gemm_fused(ctypes.byref(args), _lib.stream_ptr()), "xb_gemm_fused(gather)")
    st["base"] += args.ctas_out
    _launches += 1
    return out


def gemm_rs(a: torch.Tensor, b: torch.Tensor, partial: torch.Tensor, partial_ptrs: Sequence[int],
            rows_per_rank: int, peers: Peers, *, b_mn: bool = False, epoch: int = 0, done_needed: int = 0,
            pulled: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows [rank * rows_per_rank, ...) of sum_r (A_r @ op(B_r)^T): every rank calls this with its
    partial operands.  ``partial`` [M, N] (bf16, symmetric memory) receives this rank's partial
    result and ``partial_ptrs[r]`` is rank r's buffer of the same shape.  With ``out`` (and
    ``pulled`` [nranks, rows_per_rank, N] as local staging) the kernel pulls the peers' blocks of
    this rank's rows and writes their fp32 sum (+ ``residual``); without it only ``partial`` is
    produced.  Returns ``out`` or ``partial``."""
    global _launches
    _check_bf16(a, b, partial)
    M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb and len(partial_ptrs) == peers.nranks and rows_per_rank % 32 == 0
    assert partial.shape == (M, N) and partial.is_contiguous() and M == rows_per_rank * peers.nranks
    st = _shape_state(a.device, ("rs", M, N, K), 1)
    args = _Args()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), partial.data_ptr()
    args.M, args.N, args.K = M, N, K
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), N
    args.b_mn, args.out_fp32, args.accumulate = int(b_mn), 0, 0
    args.rank, args.nranks = peers.rank, peers.nranks
    args.gather, args.scatter = 0, 1
    for r, ptr in enumerate(partial_ptrs):
        args.partial_ptrs[r] = ptr
    args.rows_per_rank = rows_per_rank
    args.ready_counters = st["ready"].data_ptr()
    args.ready_target = st["base"]
    if out is not None:
        _check_bf16(out, pulled)
        assert out.shape == (rows_per_rank, N) and pulled.numel() >= peers.nranks * rows_per_rank * N
        args.out, args.ldo, args.pulled = out.data_ptr(), out.stride(0), pulled.data_ptr()
        if residual is not None:
            _check_bf16(residual)
            assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
            args.residual = residual.data_ptr()
    args.counters = st["counters"].data_ptr()
    if peers.flags is not None:
        for r, ptr in enumerate(peers.flags):
            args.flag_ptrs[r] = ptr
    args.ready_slot, args.done_slot = peers.ready_slot, peers.done_slot
    args.epoch, args.done_needed, args.wait_ms = epoch, done_needed, peers.wait_ms
    _lib.check(_lib.cuda_lib().xb_gemm_fused(ctypes.byref(args), _lib.stream_ptr()), "xb_gemm_fused(scatter)")
    if out is not None:
        st["base"] += args.ctas_out
    _launches += 1
    return out if out is not None else partial


def rs_reduce(blocks: Sequence[torch.Tensor], out: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = sum of ``blocks`` (contiguous [rows, N] bf16 tensors, one per rank) in fp32, in order
    (+ residual): the reduction phase of ``gemm_rs`` as a kernel of its own."""
    rows, N = blocks[0].shape
    _check_bf16(out, *blocks)
    assert all(b.is_contiguous() and b.shape == (rows, N) for b in blocks)
    ptrs = (ctypes.c_ulonglong * len(blocks))(*[b.data_ptr() for b in blocks])
    _lib.check(_lib.cuda_lib().xb_rs_reduce(ptrs, len(blocks), rows, N, out.data_ptr(), out.stride(0),
                                            residual.data_ptr() if residual is not None else None,
                                            _lib.stream_ptr()), "xb_rs_reduce")
    return out
