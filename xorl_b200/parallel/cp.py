"""Context parallelism entry point: picks the strategy object the attention layers call.

None (local attention), Ulysses, ring, or hybrid Ulysses x ring, following the selection rules of
src/xorl/distributed/sequence_parallel/strategy.py:487-544."""
from __future__ import annotations


def attach_cp_strategy(model, pstate) -> None:
    if pstate.sp_size <= 1:
        model.cp_strategy = None
        return
    from .sequence_parallel import build_cp_strategy
    model.cp_strategy = build_cp_strategy(model, pstate)
