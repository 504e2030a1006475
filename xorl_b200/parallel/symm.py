"""Attachment point of the fused peer-memory transport (symmetric heap + own kernels)."""
from __future__ import annotations

from ..utils.logging import warning_rank0


def try_attach_symmetric_transport(engine, required: bool = False) -> bool:
    try:
        from .symm_transport import SymmetricTransport
        engine.symm = SymmetricTransport.create(engine)
        return engine.symm is not None
    except Exception as e:  # noqa: BLE001
        if required:
            raise
        warning_rank0(f"fused peer-memory transport unavailable ({e!r}); using NCCL collectives")
        engine.symm = None
        return False
