"""Collator chain: shift tokens -> pack documents into one row with position ids and cu_seqlens ->
pad to a multiple -> (optionally) shard the sequence for context parallelism with zigzag order.

Counterparts in the reference: ShiftTokensCollator (src/xorl/data/collators/shift_tokens_collator.py),
PackingConcatCollator (src/xorl/data/collators/packing_concat_collator.py:12-42),
TextSequenceShardCollator with zigzag reordering (src/xorl/data/collators/sequence_shard_collator.py:90-157,191-)."""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import numpy as np
import torch

IGNORE_INDEX = -100


def shift_sample(sample: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """input_ids[:-1] predicts labels[1:]; the last target of a document is dropped."""
    ids = np.asarray(sample["input_ids"])
    labels = np.asarray(sample.get("labels", ids))
    return {"input_ids": ids[:-1], "labels": labels[1:]}


class PackingCollator:
    """A list of samples (one bin) -> one packed row.

    Output tensors (1-D, length T padded to ``pad_to_multiple_of``): ``input_ids``, ``labels``,
    ``position_ids`` (restart at each document) and ``cu_seqlens`` (int32; padding forms a final
    pseudo-document whose labels are all ignored)."""

    def __init__(self, pad_to_multiple_of: int = 128, shift: bool = True, pad_token_id: int = 0,
                 pad_to_length: int = 0):
        self.mult = max(1, int(pad_to_multiple_of or 1))
        self.shift = shift
        self.pad_id = pad_token_id
        self.pad_to_length = pad_to_length

    def __call__(self, samples: Sequence[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        ids, labels, pos, cu = [], [], [], [0]
        for s in samples:
            s = shift_sample(s) if self.shift else s
            n = len(s["input_ids"])
            if n == 0:
                continue
            ids.append(np.asarray(s["input_ids"], dtype=np.int64))
            labels.append(np.asarray(s["labels"], dtype=np.int64))
            pos.append(np.arange(n, dtype=np.int64))
            cu.append(cu[-1] + n)
        T = cu[-1]
        target = max(self.pad_to_length, (T + self.mult - 1) // self.mult * self.mult)
        pad = target - T
        if pad > 0:
            ids.append(np.full(pad, self.pad_id, dtype=np.int64))
            labels.append(np.full(pad, IGNORE_INDEX, dtype=np.int64))
            pos.append(np.arange(pad, dtype=np.int64))
            cu.append(cu[-1] + pad)
        lab = np.concatenate(labels)
        return {
            "num_valid_tokens": int((lab != IGNORE_INDEX).sum()),
            "input_ids": torch.from_numpy(np.concatenate(ids)),
            "labels": torch.from_numpy(lab),
            "position_ids": torch.from_numpy(np.concatenate(pos)),
            "cu_seqlens": torch.tensor(cu, dtype=torch.int32),
        }


def zigzag_indices(length: int, cp: int, rank: int) -> np.ndarray:
    """Token indices of one document that ring-attention rank ``rank`` of ``cp`` owns: chunks
    ``rank`` and ``2*cp-1-rank`` out of 2*cp equal chunks (length must divide by 2*cp)."""
    chunk = length // (2 * cp)
    a = np.arange(rank * chunk, (rank + 1) * chunk)
    b = np.arange((2 * cp - 1 - rank) * chunk, (2 * cp - rank) * chunk)
    return np.concatenate([a, b])


class SequenceShardCollator:
    """Splits a packed row across sequence-parallel ranks.

    ``ring`` ranks take zigzag chunks of every document (balanced causal work); inside a ring
    rank the ``ulysses`` ranks take contiguous slices.  Documents are padded so their length
    divides by ``2 * ring * ulysses``; the full-row ``cu_seqlens`` and ``position_ids`` of the
    local tokens are kept because attention still needs global positions."""

    def __init__(self, ring: int, ulysses: int, ring_rank: int, ulysses_rank: int, pad_token_id: int = 0):
        self.ring, self.uly, self.rr, self.ur = ring, ulysses, ring_rank, ulysses_rank
        self.pad_id = pad_token_id

    def __call__(self, row: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.ring * self.uly == 1:
            return row
        cu = row["cu_seqlens"].tolist()
        mult = 2 * self.ring * self.uly
        ids, labels, pos, new_cu = [], [], [], [0]
        for s, e in zip(cu[:-1], cu[1:]):
            n = e - s
            padded = (n + mult - 1) // mult * mult
            i = torch.full((padded,), self.pad_id, dtype=torch.long)
            l = torch.full((padded,), IGNORE_INDEX, dtype=torch.long)
            i[:n], l[:n] = row["input_ids"][s:e], row["labels"][s:e]
            ids.append(i); labels.append(l); pos.append(torch.arange(padded)); new_cu.append(new_cu[-1] + padded)
        full_ids, full_labels, full_pos = torch.cat(ids), torch.cat(labels), torch.cat(pos)
        sel = []
        for s, e in zip(new_cu[:-1], new_cu[1:]):
            zz = zigzag_indices(e - s, self.ring, self.rr) if self.ring > 1 else np.arange(e - s)
            per = len(zz) // self.uly
            sel.append(torch.from_numpy(zz[self.ur * per:(self.ur + 1) * per] + s))
        sel = torch.cat(sel)
        local_cu = [0]
        for s, e in zip(new_cu[:-1], new_cu[1:]):
            local_cu.append(local_cu[-1] + (e - s) // (self.ring * self.uly))
        return {
            "input_ids": full_ids[sel], "labels": full_labels[sel], "position_ids": full_pos[sel],
            "cu_seqlens": torch.tensor(new_cu, dtype=torch.int32),            # global documents
            "local_cu_seqlens": torch.tensor(local_cu, dtype=torch.int32),    # this rank's slices
        }
