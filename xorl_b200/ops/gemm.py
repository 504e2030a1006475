"""Dense GEMM on tcgen05 (``csrc/gemm.cu``) and the ``linear`` autograd function built on it.

``gemm(a, b, a_mn, b_mn)`` computes ``op(a) @ op(b).T`` where an operand flagged ``*_mn`` is
stored transposed (reduction dimension outermost).  Forward, dgrad and wgrad of a linear layer
are the three layout combinations (K,K), (K,MN) and (MN,MN), so no transpose copy is ever made.
Replaces ``F.linear`` / cuBLAS in the reference (every nn.Linear, e.g.
src/xorl/models/transformers/qwen3/modeling_qwen3.py:40-81).
"""
from __future__ import annotations

import os

import torch

from . import _lib
from .grad_sink import current_wgrad_store, grad_target, mark_written, note_wgrad_issued, wgrad_stream

_launches = 0
# "pair": CTA-pair kernel (tcgen05 cta_group::2, 512x256 pair tiles, csrc/gemm2.cu);
# "single": one CTA per 128x256 tile (csrc/gemm.cu), also used for small M
_VARIANT = os.environ.get("XORL_B200_GEMM", "pair")


def set_variant(name: str) -> str:
    """Selects the dense GEMM kernel ("pair" or "single"); returns the previous choice."""
    global _VARIANT
    assert name in ("pair", "single")
    prev, _VARIANT = _VARIANT, name
    return prev


def launch_count() -> int:
    return _launches


_BATCH_INVARIANT = False


def set_batch_invariant(on: bool) -> bool:
    """Batch-invariant GEMMs: the value of an output row no longer depends on how many rows the
    call carries (src/xorl/ops/batch_invariant_ops.py:177-300 gives the same guarantee with a
    persistent kernel of fixed tile order).  Here every element of C is owned by one tile whose K
    loop runs in a fixed order; the mode removes the two things that vary with the problem size:
    the choice between the single-CTA and the CTA-pair kernel (always the pair kernel) and the
    cutting of the tiles of a partial last wave (always whole 512 x 256 tiles).  Returns the
    previous setting.  Also settable with ``XORL_B200_BATCH_INVARIANT=1``."""
    global _BATCH_INVARIANT
    prev = _BATCH_INVARIANT
    _BATCH_INVARIANT = bool(on)
    if _lib.have_cuda_lib() and torch.cuda.is_available():
        _lib.cuda_lib().xb_gemm_set_batch_invariant(int(_BATCH_INVARIANT))
    return prev


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
         accumulate: bool = False) -> torch.Tensor:
    """C[M,N] (+)= op(a)[M,K] @ op(b)[N,K]^T with fp32 accumulation."""
    assert a.dim() == 2 and b.dim() == 2
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    if not a.is_cuda:
        A = a.t() if a_mn else a
        B = b.t() if b_mn else b
        res = (A.float() @ B.float().t())
        dt = out.dtype if out is not None else (out_dtype or a.dtype)
        if out is not None:
            if accumulate:
                out.add_(res.to(dt))
            else:
                out.copy_(res.to(dt))
            return out
        return res.to(dt)
    global _launches
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 operands required"
    if a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
        a = a.contiguous()
    if b.stride(1) != 1 or b.stride(0) % 8 or b.data_ptr() % 16:
        b = b.contiguous()
    if a.stride(0) % 8 or b.stride(0) % 8:
        # leading dimensions must be multiples of 8 elements for TMA: pad the reduction dim
        raise ValueError("gemm operands need leading dimensions that are multiples of 8")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or torch.bfloat16)
        assert not accumulate
    assert out.shape == (M, N) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    lib = _lib.cuda_lib()
    args = (a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
            out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate))
    if _BATCH_INVARIANT or (_VARIANT == "pair" and M >= 384):
        rc = lib.xb_gemm_bf16_pair(*args, _lib.stream_ptr())
    else:
        rc = lib.xb_gemm_bf16(*args, _lib.stream_ptr())
    _lib.check(rc, "xb_gemm_bf16")
    _launches += 1
    return out


_PANEL_STREAMS: dict = {}


def _panel_streams(device, n: int):
    key = (device.index if device.index is not None else torch.cuda.current_device())
    pool = _PANEL_STREAMS.setdefault(key, [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device))
    return pool[:n]


# Below this many rows the full product is faster on a B200 than its lower half in panels
# (measured: 4096 x 12288 -> 0.84x, 8192 x 8192 -> 1.17x with 1024-row panels on four streams).
SYMMETRIC_MIN_ROWS = 8192


def gemm_symmetric(a: torch.Tensor, b: torch.Tensor | None = None, *, out_dtype: torch.dtype | None = None,
                   block: int = 1024, min_rows: int | None = None) -> torch.Tensor:
    """C = a @ b^T for a product that is known to be symmetric (``b`` omitted: a @ a^T; or two
    commuting symmetric factors).  Only the row panels on and below the block diagonal go through
    the GEMM kernel (panel r covers columns 0 .. end of block r); the blocks above are mirrored by
    ``xb_mirror_lower``.  With M / block panels the GEMM work is (1 + block / M) / 2 of the full
    product; matrices with fewer than ``min_rows`` rows take the plain GEMM, which is faster there.
    Same role as src/xorl/ops/quack/gemm_symmetric.py."""
    global _launches
    b = a if b is None else b
    M = a.shape[0]
    assert b.shape[0] == M and a.shape[1] == b.shape[1]
    min_rows = SYMMETRIC_MIN_ROWS if min_rows is None else min_rows
    if not a.is_cuda or M < max(2 * block, min_rows) or a.shape[1] % 8 or M % 8:
        return gemm(a, b, out_dtype=out_dtype)
    out = torch.empty((M, M), device=a.device, dtype=out_dtype or torch.bfloat16)
    # A panel alone has too few tiles to fill 148 SMs, so the panels run side by side on a few
    # streams (largest first); the launching stream waits for all of them before the mirror.
    main = torch.cuda.current_stream()
    ready = torch.cuda.Event()
    ready.record(main)
    panels = [(r0, min(M, r0 + block)) for r0 in range(0, M, block)][::-1]
    streams = _panel_streams(a.device, min(len(panels), 4))
    for i, (r0, r1) in enumerate(panels):
        st = streams[i % len(streams)]
        if i < len(streams):
            st.wait_event(ready)
        with torch.cuda.stream(st):
            gemm(a[r0:r1], b[:r1], out=out[r0:r1, :r1])
    for st in streams:
        done = torch.cuda.Event()
        done.record(st)
        main.wait_event(done)
    _lib.check(_lib.cuda_lib().xb_mirror_lower(out.data_ptr(), out.stride(0), M, block,
                                               int(out.dtype == torch.float32), _lib.stream_ptr()),
               "xb_mirror_lower")
    _launches += 1
    return out


def weight_grad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor):
    """dW = dy2^T @ x2 for weight ``w``: written straight into the flat gradient buffer of the ZeRO
    unit (returns None), deferred to a W slot of a zero-bubble schedule, or returned as a tensor."""
    tgt, fresh = grad_target(w)
    store = current_wgrad_store()
    if tgt is not None and store is not None:
        # zero-bubble: the buffer slice is claimed now, the GEMM runs in a later W slot
        mark_written(w)
        store.append(lambda a=dy2, b=x2, o=tgt, acc=not fresh:
                     gemm(a, b, a_mn=True, b_mn=True, out=o, accumulate=acc))
        return None
    if tgt is not None:
        side = wgrad_stream(dy2.device) if dy2.is_cuda else None
        if side is not None:
            # overlap with the input-gradient GEMM that follows on the main stream
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                gemm(dy2, x2, a_mn=True, b_mn=True, out=tgt, accumulate=not fresh)
            dy2.record_stream(side)
            x2.record_stream(side)
            note_wgrad_issued()
        else:
            gemm(dy2, x2, a_mn=True, b_mn=True, out=tgt, accumulate=not fresh)
        mark_written(w)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)


class _Linear(torch.autograd.Function):
    """y = x @ w.T.  The weight is kept on ctx as a plain attribute (not through
    save_for_backward) because ZeRO-3 re-fills the same gathered buffer before backward."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.x_shape = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2)
        ctx.w = w
        y = gemm(x2, w)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        w = ctx.w
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        # the weight gradient is issued first (on its side stream when it goes to an engine buffer), the
        # input gradient follows on the main stream: the two persistent kernels fill each other's tails
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy2, x2, w)
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.x_shape)
        return dx, dw


_LIBRARY_FALLBACKS: set = set()


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Linear layer through the tcgen05 GEMM (CUDA) or torch (CPU)."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, w, bias)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[-1] % 8 or w.shape[0] % 8:
        # the tcgen05 kernel takes bf16 operands whose row pitches are multiples of 16 bytes (TMA): the
        # reduction dim for the forward, the output dim for the gradient GEMMs; anything else runs in the
        # library, and says so once per case instead of doing it silently
        key = (x.dtype, w.dtype, x.shape[-1] % 8 != 0, w.shape[0] % 8 != 0)
        if key not in _LIBRARY_FALLBACKS:
            _LIBRARY_FALLBACKS.add(key)
            import logging
            logging.getLogger("xorl_b200").warning(
                "ops.gemm.linear: %s x %s with K=%d, N=%d runs in the library GEMM, not the tcgen05 kernel "
                "(bf16 operands, K %% 8 == 0 and N %% 8 == 0 are required)", x.dtype, w.dtype, x.shape[-1], w.shape[0])
        return torch.nn.functional.linear(x, w, bias)
    y = _Linear.apply(x, w)
    if bias is not None:
        y = y + bias
    return y


if os.environ.get("XORL_B200_BATCH_INVARIANT", "0") == "1":
    set_batch_invariant(True)
