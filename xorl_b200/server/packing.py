"""Datum -> micro-batch packing for the server: sequential, best-fit and DP-balanced
(src/xorl/server/orchestrator/packing.py:545-903)."""
from __future__ import annotations

import heapq
import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

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


def _lpt(lengths: Sequence[int], n_bins: int, capacity: int) -> Optional[List[List[int]]]:
    """Longest-first into the currently lightest of ``n_bins`` bins; None when a bin would overflow."""
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    heap: List[Tuple[int, int]] = [(0, b) for b in range(n_bins)]
    bins: List[List[int]] = [[] for _ in range(n_bins)]
    for i in order:
        load, b = heapq.heappop(heap)
        if load + lengths[i] > capacity:
            return None
        bins[b].append(i)
        heapq.heappush(heap, (load + lengths[i], b))
    return [sorted(b) for b in bins]


def pack_balanced_dp(lengths: Sequence[int], capacity: int, dp: int) -> List[List[int]]:
    """``k * dp`` bins of near-equal token count for the smallest ``k`` that fits, so that every
    data-parallel rank gets ``k`` real micro-batches and no dummy ones
    (src/xorl/server/orchestrator/packing.py:857-928).  With fewer samples than ranks, or when no
    multiple of ``dp`` fits, the result is the best-fit packing."""
    n = len(lengths)
    if dp <= 1 or n < dp:
        return pack_best_fit(lengths, capacity)
    k_min = max(1, math.ceil(sum(lengths) / (dp * capacity)))
    for k in range(k_min, n // dp + 1):
        bins = _lpt(lengths, k * dp, capacity)
        if bins is not None:
            return bins
    return pack_best_fit(lengths, capacity)


def apply_oversized_policy(datums: List[Dict[str, Any]], capacity: int, mode: str = "error"
                           ) -> Tuple[List[Dict[str, Any]], List[int]]:
    """What happens to a datum longer than the packing length: ``error`` raises, ``skip`` drops it,
    ``truncate`` clips its tokens and every per-token field (src/xorl/server/orchestrator/packing.py:713-792).
    Returns the surviving datums and the positions (in the input list) they came from."""
    if mode not in ("error", "skip", "truncate"):
        raise ValueError(f"unknown on_oversized mode {mode!r}")
    kept, origin = [], []
    for i, d in enumerate(datums):
        n = len(d["tokens"])
        if n <= capacity:
            kept.append(d)
            origin.append(i)
            continue
        if mode == "error":
            raise ValueError(f"datum {i} has {n} tokens, more than the packing length {capacity}")
        if mode == "skip":
            continue
        c = {}
        for k, v in d.items():
            if k == "routed_experts":
                c[k] = v[:capacity]
            elif hasattr(v, "__len__") and not isinstance(v, (str, bytes, dict)) and len(v) == n:
                c[k] = v[:capacity]
            else:
                c[k] = v
        kept.append(c)
        origin.append(i)
    return kept, origin


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
