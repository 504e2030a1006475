"""Checks at pipeline-stage borders that keep a pipelined run numerically equal to the unsplit
model: the stage plan, the identity of the layers on each stage, the dtype on the wire and the
per-micro-batch metadata a stage must receive.

Why each check exists (src/xorl/distributed/pp_byte_contract.py:1-438):

* the plan may cut only between decoder layers, cover every layer once and in order, keep the
  embedding on the first global stage and the final norm + head together on the last;
* a stage's layers keep their *global* ``layer_idx``: code that picks a kernel or a norm variant
  by layer position would otherwise change behaviour at a cut without any error;
* activations cross a border in the compute dtype: a silent up- or down-cast on one side changes
  the bytes the next stage sees;
* a packed batch without its document boundaries does not fail downstream, the attention just
  treats the pack as one document; a stage therefore refuses to run without ``position_ids`` and
  ``cu_seqlens``."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

import torch

REQUIRED_METADATA = ("position_ids", "cu_seqlens")


class PPContractError(RuntimeError):
    """A pipeline configuration or message would change the numbers of the unsplit model."""


def validate_stage_plan(stages: Sequence[Sequence[int]], num_layers: int) -> None:
    """``stages[g]`` = decoder layers of global stage g."""
    flat: List[int] = []
    for g, layers in enumerate(stages):
        layers = list(layers)
        if layers != list(range(layers[0], layers[0] + len(layers))) if layers else False:
            raise PPContractError(f"stage {g} holds non-contiguous layers {layers}")
        flat += layers
    if flat != list(range(num_layers)):
        raise PPContractError(f"stages cover layers {flat}, expected 0..{num_layers - 1} once each, in order")


def validate_layout(layout: Dict, num_layers: int) -> None:
    """A rank's own layout from ``local_stage_layout``: the embedding lives with global stage 0 and
    the head with the last stage."""
    n = layout["n_stages"]
    if layout["has_embed"] != (0 in layout["chunk_stage"]):
        raise PPContractError("embedding must live on the rank that owns global stage 0")
    if layout["has_head"] != ((n - 1) in layout["chunk_stage"]):
        raise PPContractError("final norm and head must live on the rank that owns the last stage")
    for g, layers in zip(layout["chunk_stage"], layout["chunk_layers"]):
        if any(not (0 <= l < num_layers) for l in layers):
            raise PPContractError(f"stage {g} names layers outside 0..{num_layers - 1}: {layers}")


def validate_layer_identity(named_layers: Iterable, expected: Sequence[int]) -> None:
    """``named_layers``: (global index, module) pairs of one stage."""
    seen = []
    for idx, mod in named_layers:
        seen.append(idx)
        for attr in ("layer_idx", "layer_id"):
            have = getattr(mod, attr, None)
            if have is not None and int(have) != int(idx):
                raise PPContractError(f"layer {idx} reports {attr}={have} after the split")
    if list(seen) != list(expected):
        raise PPContractError(f"stage holds layers {seen}, plan says {list(expected)}")


def assert_wire_dtype(t: torch.Tensor, expected: torch.dtype, where: str) -> None:
    if t.dtype != expected:
        raise PPContractError(f"{where}: activation crosses the stage border as {t.dtype}, expected {expected}")
    if not t.is_contiguous():
        raise PPContractError(f"{where}: non-contiguous tensor on the wire")


def validate_microbatch_metadata(mb: Dict[str, Optional[torch.Tensor]], index: int) -> None:
    missing = [k for k in REQUIRED_METADATA if mb.get(k) is None]
    if missing:
        raise PPContractError(f"micro-batch {index} reaches a pipeline stage without {missing}: the pack would be "
                              "treated as one document")
    cu = mb["cu_seqlens"]
    n = int(mb["position_ids"].numel())
    if int(cu[0]) != 0 or int(cu[-1]) > n or bool((cu[1:] < cu[:-1]).any()):
        raise PPContractError(f"micro-batch {index}: cu_seqlens {cu.tolist()} do not delimit {n} tokens")
