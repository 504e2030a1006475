"""Tensor parallelism with sequence-parallel activations.

Between the tensor-parallel regions the residual stream, the norms and the dropout-free glue work
on ``T / tp`` tokens per rank.  A column-parallel linear is then ``all_gather(x_s) @ W_c^T`` and a
row-parallel linear ``reduce_scatter(h @ W_r^T)``, and so are their backward passes:

=====================  ==============================  =======================================
op                     forward                         backward (input gradient)
=====================  ==============================  =======================================
``sp_column_linear``   all-gather -> GEMM              GEMM -> reduce-scatter  (``dY @ W``)
``sp_row_linear``      GEMM -> reduce-scatter          all-gather -> GEMM      (``AG(dY_s) @ W``)
=====================  ==============================  =======================================

On CUDA each of the four is ONE kernel (``csrc/gemm_fused.cu`` through ``ops/fused_gemm.py``): the
shards and the staging buffers live in symmetric memory mapped into every peer of the group, the
all-gather runs in communication warps of the GEMM kernel, and so does the pull of the peers' partial
result blocks of the reduce-scatter, signalled block by block from the epilogue.
On CPU (gloo), for fp32, or when a shape does not fit the kernel (rows per rank not a multiple of
32 for the reduce-scatter) the same functions run the collective through ``torch.distributed``
followed / preceded by a plain GEMM, so the model code is identical everywhere.

The reference runs tensor parallelism through DTensor ``ColwiseParallel`` / ``RowwiseParallel``
with an all-reduce and no overlap of communication and compute
(src/xorl/distributed/torch_parallelize.py:222-270,
docs/src/content/docs/parallelism/tensor_parallelism.mdx:326).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as gemm_ops

# flag-area layout (int32 slots): 16 per kind, except the reduce-scatter ready flags, which are
# [rank][sub-block] (16 x 16)
_G_READY, _G_DONE, _S_DONE, _S_READY = 0, 16, 32, 256
_FLAG_INTS = 1024
_RING = 2


class SequenceParallelTP:
    """Collective GEMMs of one tensor-parallel group; owns the symmetric buffers of the fused path."""

    def __init__(self, group, rank: int, world: int):
        self.group, self.rank, self.world = group, rank, world
        self.fused = os.environ.get("XORL_B200_TP_FUSED", "1") == "1"
        self._heap = None
        self._pulled = None                       # local staging of the peers' partial blocks
        self._cap: Tuple[int, int] = (0, 0)       # (rows per rank, features) the buffers can hold
        self.g_epoch = 0
        self.s_epoch = 0
        self.fused_calls = 0
        self.fallback_calls = 0

    # ---- symmetric buffers ------------------------------------------------------------------------
    def _ensure(self, rows_per: int, feat: int, device) -> None:
        if self._heap is not None and rows_per <= self._cap[0] and feat <= self._cap[1]:
            return
        import torch.distributed._symmetric_memory as symm_mem
        rows_per = max(rows_per, self._cap[0])
        feat = max(feat, self._cap[1])
        shard_bytes = _align(rows_per * feat * 2)
        stage_bytes = _align(self.world * rows_per * feat * 2)
        total = _align(_FLAG_INTS * 4) + _RING * (shard_bytes + stage_bytes)
        if self._heap is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        heap = symm_mem.empty(total, dtype=torch.uint8, device=device)
        heap[:_FLAG_INTS * 4].zero_()
        hdl = symm_mem.rendezvous(heap, self.group)
        self._heap, self._hdl = heap, hdl
        self._base = [int(p) for p in hdl.buffer_ptrs]
        self._shard_off = [_align(_FLAG_INTS * 4) + i * shard_bytes for i in range(_RING)]
        self._stage_off = [_align(_FLAG_INTS * 4) + _RING * shard_bytes + i * stage_bytes for i in range(_RING)]
        self._cap = (rows_per, feat)
        self.g_epoch = self.s_epoch = 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _peers(self, ready: int, done: int):
        from ..ops.fused_gemm import Peers
        return Peers(self.rank, self.world, flags=self._base, ready_slot=ready, done_slot=done)

    # ---- all-gather -> GEMM --------------------------------------------------------------------------
    def all_gather_gemm(self, x_s: torch.Tensor, w: torch.Tensor, b_mn: bool = False):
        """(all_gather(x_s) @ op(w)^T, all_gather(x_s)); x_s [T / tp, K]."""
        rows_per, K = x_s.shape
        if self._fused_ok(x_s, w) and K % 8 == 0:
            from ..ops import fused_gemm
            self._ensure(rows_per, K, x_s.device)
            self.g_epoch += 1
            e = self.g_epoch
            slot = e % _RING
            if e > _RING:
                # the peers must have finished reading what this buffer held two calls ago
                flags = self._base[self.rank] + 4 * _G_DONE
                _lib.check(_lib.cuda_lib().xb_symm_wait(ctypes.c_void_p(flags), self.world, self.rank, e - _RING,
                                                        2000, _lib.stream_ptr()), "xb_symm_wait")
            off = self._shard_off[slot]
            stage = self._heap[off:off + rows_per * K * 2].view(torch.bfloat16).view(rows_per, K)
            stage.copy_(x_s)
            full = torch.empty(rows_per * self.world, K, device=x_s.device, dtype=torch.bfloat16)
            y = fused_gemm.ag_gemm(full, [b + off for b in self._base], rows_per, w,
                                   self._peers(_G_READY, _G_DONE), gathered="a", b_mn=b_mn, epoch=e)
            self.fused_calls += 1
            return y, full
        self.fallback_calls += 1
        full = torch.empty(rows_per * self.world, K, device=x_s.device, dtype=x_s.dtype)
        dist.all_gather_into_tensor(full, x_s.contiguous(), group=self.group)
        return _mm(full, w, b_mn), full

    # ---- GEMM -> reduce-scatter ----------------------------------------------------------------------
    def gemm_reduce_scatter(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False,
                            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows of this rank of sum over ranks (a_r @ op(w_r)^T) (+ residual); a [T, K_local]."""
        T = a.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        assert T % self.world == 0, f"{T} tokens not divisible by tensor-parallel size {self.world}"
        rows_per = T // self.world
        if self._fused_ok(a, w) and rows_per % 32 == 0 and N % 8 == 0 and a.shape[1] % 8 == 0:
            from ..ops import fused_gemm
            self._ensure(rows_per, N, a.device)
            self.s_epoch += 1
            e = self.s_epoch
            off = self._stage_off[e % _RING]
            partial = self._heap[off:off + T * N * 2].view(torch.bfloat16).view(T, N)
            if self._pulled is None or self._pulled.numel() < T * N:
                self._pulled = torch.empty(T * N, device=a.device, dtype=torch.bfloat16)
            out = torch.empty(rows_per, N, device=a.device, dtype=torch.bfloat16)
            fused_gemm.gemm_rs(a.contiguous(), w, partial, [b + off for b in self._base], rows_per,
                               self._peers(_S_READY, _S_DONE), b_mn=b_mn, epoch=e,
                               done_needed=max(e - _RING, 0), pulled=self._pulled, out=out,
                               residual=residual)
            self.fused_calls += 1
            return out
        self.fallback_calls += 1
        y = _mm(a, w, b_mn).contiguous()
        out = torch.empty(rows_per, N, device=a.device, dtype=y.dtype)
        dist.reduce_scatter_tensor(out, y, group=self.group)
        if residual is not None:
            out = out + residual
        return out

    def _fused_ok(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        return (self.fused and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and self.world <= 16 and w.stride(-1) == 1 and w.data_ptr() % 16 == 0)


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


def _mm(a: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
    if a.is_cuda and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        return gemm_ops.gemm(a, w, b_mn=b_mn)
    return a @ w if b_mn else a @ w.t()


_CONTEXTS: Dict[int, SequenceParallelTP] = {}


def sp_context() -> Optional[SequenceParallelTP]:
    """The context of the current tensor-parallel group (None without tensor parallelism)."""
    from .state import get_parallel_state
    ps = get_parallel_state()
    if ps.tp_size <= 1:
        return None
    g = ps.group("tp")
    c = _CONTEXTS.get(id(g))
    if c is None:
        c = _CONTEXTS[id(g)] = SequenceParallelTP(g, ps.tp_rank, ps.tp_size)
    return c


def reset_sp_contexts() -> None:
    _CONTEXTS.clear()


class _SPColumnLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_s, w, sp: SequenceParallelTP):
        y, x_full = sp.all_gather_gemm(x_s, w)
        ctx.save_for_backward(x_full)
        ctx.w, ctx.sp = w, sp
        return y

    @staticmethod
    def backward(ctx, dy):
        (x_full,) = ctx.saved_tensors
        w, sp = ctx.w, ctx.sp
        dy = dy.contiguous()
        dx_s = sp.gemm_reduce_scatter(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = gemm_ops.weight_grad(dy, x_full, w) if ctx.needs_input_grad[1] else None
        return dx_s, dw, None


class _SPRowLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, sp: SequenceParallelTP):
        h = h.contiguous()
        ctx.save_for_backward(h)
        ctx.w, ctx.sp = w, sp
        return sp.gemm_reduce_scatter(h, w)

    @staticmethod
    def backward(ctx, dy_s):
        (h,) = ctx.saved_tensors
        w, sp = ctx.w, ctx.sp
        dh, dy_full = sp.all_gather_gemm(dy_s.contiguous(), w, b_mn=True)
        dw = gemm_ops.weight_grad(dy_full, h, w) if ctx.needs_input_grad[1] else None
        return (dh if ctx.needs_input_grad[0] else None), dw, None


def sp_column_linear(x_s: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], sp: SequenceParallelTP):
    """[T / tp, K] token shard -> [T, N_local]."""
    y = _SPColumnLinear.apply(x_s, w, sp)
    return y if bias is None else y + bias


def sp_row_linear(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], sp: SequenceParallelTP):
    """[T, K_local] -> [T / tp, N] token shard (the bias, replicated, is added once per token)."""
    y = _SPRowLinear.apply(h, w, sp)
    return y if bias is None else y + bias


class _GatherTokens(torch.autograd.Function):
    """all_gather of token shards whose consumer computes the same gradient on every rank (the
    lm-head loss): backward keeps this rank's rows."""

    @staticmethod
    def forward(ctx, x_s, sp: SequenceParallelTP):
        ctx.sp = sp
        full = torch.empty(x_s.shape[0] * sp.world, *x_s.shape[1:], device=x_s.device, dtype=x_s.dtype)
        dist.all_gather_into_tensor(full, x_s.contiguous(), group=sp.group)
        return full

    @staticmethod
    def backward(ctx, g):
        sp = ctx.sp
        n = g.shape[0] // sp.world
        return g[sp.rank * n:(sp.rank + 1) * n].contiguous(), None


def gather_tokens(x_s: torch.Tensor, sp: SequenceParallelTP) -> torch.Tensor:
    return _GatherTokens.apply(x_s, sp)


def local_tokens(x: torch.Tensor, sp: SequenceParallelTP) -> torch.Tensor:
    """This rank's contiguous slice of a token-major tensor."""
    assert x.shape[0] % sp.world == 0, f"{x.shape[0]} tokens not divisible by tensor-parallel size {sp.world}"
    n = x.shape[0] // sp.world
    return x[sp.rank * n:(sp.rank + 1) * n]
