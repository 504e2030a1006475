"""Datum -> micro-batch packing for the server: sequential, best-fit and DP-balanced
(src/xorl/server/orchestrator/packing.py:545-903)."""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import torch

IGNORE_INDEX = -100


def pack_sequential(lengths: Sequence[int], capacity: int) -> List[List[int]]:
    bins, cur, used = [], [], 0
    for i, n in enumerate(lengths):
        if cur and used + n > capacity:
            bins.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += n
    if cur:
        bins.append(cur)
    return bins


def pack_best_fit(lengths: Sequence[int], capacity: int) -> List[List[int]]:
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[List[int]] = []
    space: List[int] = []
    for i in order:
        n = lengths[i]
        best, best_space = -1, None
        for b, s in enumerate(space):
            if s >= n and (best_space is None or s < best_space):
                best, best_space = b, s
        if best < 0:
            bins.append([i])
            space.append(max(capacity - n, 0))
        else:
            bins[best].append(i)
            space[best] -= n
    return bins


def balance_across_dp(bins: List[List[int]], lengths: Sequence[int], dp: int) -> List[List[List[int]]]:
    """Distributes bins over ``dp`` ranks so that token counts are as even as possible; every rank
    gets the same number of micro-batches (empty ones become dummy batches)."""
    loads = [0] * dp
    per_rank: List[List[List[int]]] = [[] for _ in range(dp)]
    for b in sorted(bins, key=lambda b: -sum(lengths[i] for i in b)):
        r = min(range(dp), key=lambda k: (len(per_rank[k]), loads[k]))
        per_rank[r].append(b)
        loads[r] += sum(lengths[i] for i in b)
    n = max(len(x) for x in per_rank) if per_rank else 0
    for x in per_rank:
        while len(x) < n:
            x.append([])
    return per_rank


def datums_to_micro_batch(datums: List[Dict[str, Any]], pad_to: int = 128) -> Dict[str, Any]:
    """Packed row from datums (already shifted: ``target_tokens[i]`` is the label of ``tokens[i]``).
    Extra per-token loss inputs are concatenated the same way.  An empty list yields a dummy batch
    with every label ignored, so idle ranks still take part in the collectives."""
    ids, labels, pos, cu = [], [], [], [0]
    routed: List[torch.Tensor] = []
    extras: Dict[str, List[float]] = {}
    for d in datums:
        toks = list(d["tokens"])
        n = len(toks)
        tgt = list(d.get("target_tokens", toks[1:] + [IGNORE_INDEX]))
        w = d.get("weights")
        if w is not None:
            tgt = [t if wi > 0 else IGNORE_INDEX for t, wi in zip(tgt, w)]
        ids += toks
        labels += tgt
        pos += list(range(n))
        cu.append(cu[-1] + n)
        for k, v in d.items():
            if k == "routed_experts":
                routed.append(torch.as_tensor(v).to(torch.long))
                continue
            if k in ("tokens", "target_tokens", "weights", "datum_index"):
                continue
            extras.setdefault(k, []).extend(list(v) + [0.0] * (n - len(v)))
    T = cu[-1]
    target = max(pad_to, (T + pad_to - 1) // pad_to * pad_to)
    pad = target - T
    if pad:
        ids += [0] * pad
        labels += [IGNORE_INDEX] * pad
        pos += list(range(pad))
        cu.append(cu[-1] + pad)
        for v in extras.values():
            v.extend([0.0] * pad)
    mb = {"input_ids": torch.tensor(ids, dtype=torch.long), "labels": torch.tensor(labels, dtype=torch.long),
          "position_ids": torch.tensor(pos, dtype=torch.long), "cu_seqlens": torch.tensor(cu, dtype=torch.int32),
          "num_valid_tokens": sum(1 for t in labels if t != IGNORE_INDEX),
          "datum_spans": [(cu[i], cu[i + 1]) for i in range(len(datums))],
          "datum_index": [d.get("datum_index", i) for i, d in enumerate(datums)]}
    for k, v in extras.items():
        mb[k] = torch.tensor(v, dtype=torch.float32)
    if routed and len(routed) == len(datums):
        r = torch.cat(routed, 0)
        if pad:
            r = torch.cat([r, r.new_full((pad,) + tuple(r.shape[1:]), -1)], 0)
        mb["routed_experts"] = r
    return mb
