"""Guard words around long-lived device buffers that kernels index with computed offsets.

With ``XORL_B200_CANARIES=1`` the workspaces of the peer-memory paths (expert-dispatch scratch, the
ZeRO transport's staging) are allocated with a 256-byte pattern-filled guard on either side;
``check_all()`` -- called by the trainer after every step in this mode -- compares the guards with the
pattern in one reduction per buffer and raises naming the buffer and the side that was overwritten.
A write past the end of a capacity-sized buffer thus fails the step that made it instead of corrupting a
neighbour silently.  Off by default: the guards cost nothing when disabled and one small kernel per
buffer per step when enabled.  (The role compute-sanitizer's memcheck would play on a pool where it is
available; src/xorl has no counterpart.)
"""
from __future__ import annotations

import os
import weakref
from typing import List, Tuple

import torch

GUARD_BYTES = 256
PATTERN = 0xA5
_registry: List[Tuple[str, "weakref.ReferenceType[torch.Tensor]"]] = []


def enabled() -> bool:
    return os.environ.get("XORL_B200_CANARIES", "0") == "1"


def guarded_empty(shape, dtype, device, name: str, force: bool = False) -> torch.Tensor:
    """``torch.empty(shape)`` -- with guards around it when canaries are on (or ``force``)."""
    if not (force or enabled()):
        return torch.empty(shape, dtype=dtype, device=device)
    es = torch.empty(0, dtype=dtype).element_size()
    n = 1
    for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
        n *= int(s)
    body = (n * es + GUARD_BYTES - 1) // GUARD_BYTES * GUARD_BYTES          # keeps the body 256-byte aligned
    raw = torch.empty(body + 2 * GUARD_BYTES, dtype=torch.uint8, device=device)
    raw[:GUARD_BYTES] = PATTERN
    raw[GUARD_BYTES + n * es:] = PATTERN                                    # tail padding belongs to the guard
    view = raw[GUARD_BYTES:GUARD_BYTES + n * es].view(dtype).reshape(shape)
    view._xb_canary_raw = raw                                               # keeps the allocation alive
    view._xb_canary_body = n * es
    _registry.append((name, weakref.ref(raw), n * es))
    return view


def check_all() -> int:
    """Verifies every live guarded buffer; returns how many were checked."""
    live, bad = [], []
    for name, ref, nbytes in _registry:
        raw = ref()
        if raw is None:
            continue
        live.append((name, ref, nbytes))
        head_ok = bool((raw[:GUARD_BYTES] == PATTERN).all())
        tail_ok = bool((raw[GUARD_BYTES + nbytes:] == PATTERN).all())
        if not (head_ok and tail_ok):
            bad.append(f"{name} ({'before its start' if not head_ok else 'past its end'})")
    _registry[:] = live
    if bad:
        raise RuntimeError("guard words overwritten around: " + ", ".join(bad))
    return len(live)
