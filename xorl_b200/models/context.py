"""Per-micro-batch metadata passed to every layer (packed-sequence form)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch


@dataclass
class StepContext:
    """All activations are packed ``[T, ...]``; ``cu_seqlens`` delimits the documents."""
    cu_seqlens: torch.Tensor                 # int32 [B+1]
    position_ids: torch.Tensor               # int64 [T]
    cos: Optional[torch.Tensor] = None       # fp32 [T, rot/2]
    sin: Optional[torch.Tensor] = None
    max_seqlen: int = 0
    causal: bool = True
    cp: Any = None                            # context-parallel strategy (None = local attention)
    aux: Dict[str, Any] = field(default_factory=dict)   # router statistics, replay records, ...
    training: bool = True

    @property
    def num_tokens(self) -> int:
        return int(self.position_ids.numel())


def packed_metadata_from_padded(batch: int, seqlen: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    cu = torch.arange(0, (batch + 1) * seqlen, seqlen, device=device, dtype=torch.int32)
    pos = torch.arange(seqlen, device=device).repeat(batch)
    return cu, pos


def cu_seqlens_from_position_ids(position_ids: torch.Tensor) -> torch.Tensor:
    """Document boundaries are where the position resets to 0."""
    flat = position_ids.reshape(-1)
    starts = torch.nonzero(flat == 0, as_tuple=False).reshape(-1)
    if starts.numel() == 0 or starts[0] != 0:
        starts = torch.cat([starts.new_zeros(1), starts])
    end = torch.tensor([flat.numel()], device=flat.device, dtype=starts.dtype)
    return torch.cat([starts, end]).to(torch.int32)
