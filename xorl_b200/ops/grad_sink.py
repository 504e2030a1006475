"""Where custom autograd functions put parameter gradients.

The ZeRO engine points every parameter of the unit that is running backward at its slice of the
unit's flat gradient buffer (``p._xb_grad_buf``).  Kernels that can accumulate in their epilogue
(the wgrad GEMM) write there directly; everything else hands its gradient to
``deliver_param_grad`` which adds it to the slice.  Without an engine (plain autograd use, unit
tests) the gradient is simply returned to autograd.
"""
from __future__ import annotations

import torch


def grad_target(p: torch.Tensor):
    """(buffer view or None, fresh) — ``fresh`` means nothing has been written yet in this
    backward pass, so the first writer may overwrite instead of accumulate."""
    buf = getattr(p, "_xb_grad_buf", None)
    if buf is None:
        return None, False
    return buf, getattr(p, "_xb_grad_fresh", False)


def mark_written(p: torch.Tensor) -> None:
    p._xb_grad_fresh = False


def deliver_param_grad(p: torch.Tensor, g: torch.Tensor):
    """Adds ``g`` to the engine's buffer and returns None, or returns ``g`` cast to the parameter
    dtype when no engine buffer is attached."""
    buf, fresh = grad_target(p)
    if buf is None:
        return g.to(p.dtype).reshape(p.shape)
    g = g.reshape(buf.shape)
    if fresh:
        buf.copy_(g)
        mark_written(p)
    else:
        buf.add_(g.to(buf.dtype))
    return None


# ---- deferred weight gradients (zero-bubble pipeline schedules) --------------------------------
_wgrad_store = None


class defer_wgrad:
    """While active, linear layers do not run their weight-gradient GEMM in backward but append a
    closure that does to the returned list; the pipeline runner calls them in a later ``W`` slot."""

    def __enter__(self):
        global _wgrad_store
        self.prev = _wgrad_store
        _wgrad_store = []
        return _wgrad_store

    def __exit__(self, *exc):
        global _wgrad_store
        _wgrad_store = self.prev
        return False


def current_wgrad_store():
    return _wgrad_store


# ---- weight gradients on a side stream --------------------------------------------------------
# A linear layer's two backward GEMMs (input gradient and weight gradient) are independent.  Both are
# persistent kernels that leave part of the GPU idle during their last, partial wave of tiles; issued
# on two streams, the CTAs of one start on the SMs the other's tail has freed.  The input gradient
# stays on the main stream (the next layer's backward waits for it); the weight gradient goes to this
# stream, and whoever consumes the gradient buffers calls ``join_wgrad_stream`` first.
import os as _os

_WGRAD_OVERLAP = _os.environ.get("XORL_B200_WGRAD_STREAM", "1") == "1"
_wgrad_stream = {}
_wgrad_pending = False


def wgrad_stream(device: torch.device):
    """The side stream for weight-gradient GEMMs on ``device`` (None when the overlap is off)."""
    if not _WGRAD_OVERLAP or device.type != "cuda":
        return None
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _wgrad_stream.get(key)
    if st is None:
        st = _wgrad_stream[key] = torch.cuda.Stream(device)
    return st


def note_wgrad_issued() -> None:
    global _wgrad_pending
    _wgrad_pending = True


def join_wgrad_stream() -> None:
    """Makes the current stream wait for every weight-gradient GEMM issued on the side stream."""
    global _wgrad_pending
    if _wgrad_pending:
        for st in _wgrad_stream.values():
            torch.cuda.current_stream().wait_stream(st)
        _wgrad_pending = False
