"""Sampling-filter programme for log-probabilities that have to match the serving engine.

When the rollout engine samples with top-k / top-p / min-p, the behaviour policy is the model's
distribution *restricted to the kept tokens*; an RL loss that compares against it needs the
trainer's log-probability on the same support.  One programme, applied after the temperature:

1. order every row by descending logit, ties broken by the smaller token id (a stable sort);
2. keep the first ``top_k`` tokens;
3. keep a token while the probability mass *before* it is below ``top_p`` (the token that crosses
   the threshold is kept);
4. keep a token only if its probability is at least ``min_p`` times the row's largest probability
   (probabilities of the unfiltered row);
5. renormalise on the tokens that passed all three.

Same contract as src/xorl/ops/exact_sampling_transforms.py:53-288 (validation of per-row
parameters, ``None`` for the all-identity case so the unfiltered path keeps its bytes, row chunks
to bound the sort workspace)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

TOP_K_ALL = 1 << 30
ROW_CHUNK = 32
PROGRAM_NAME = "temperature_then_stable_token_id_topk_inclusive_topp_original_max_minp_v1"

Rows = Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]


def _rows(value, rows: int, device, dtype, name: str) -> torch.Tensor:
    if isinstance(value, torch.Tensor):
        if value.dtype is not dtype:
            raise TypeError(f"per-row {name} must be {dtype}, got {value.dtype}")
        if tuple(value.shape) != (rows,):
            raise ValueError(f"per-row {name} must have shape ({rows},), got {tuple(value.shape)}")
        if value.requires_grad:
            raise ValueError(f"per-row {name} is sampling metadata and must not require grad")
        return value.to(device).contiguous()
    return torch.full((rows,), value, dtype=dtype, device=device)


def normalize_sampling_transforms(top_k=TOP_K_ALL, top_p=1.0, min_p=0.0, *, rows: int, device) -> Rows:
    """Validated per-row tensors, or ``(None, None, None)`` when nothing would be filtered."""
    scalars = not any(isinstance(v, torch.Tensor) for v in (top_k, top_p, min_p))
    if scalars and int(top_k) >= TOP_K_ALL and float(top_p) == 1.0 and float(min_p) == 0.0:
        return None, None, None
    ks = _rows(top_k, rows, device, torch.int64, "top_k")
    ps = _rows(top_p, rows, device, torch.float32, "top_p")
    ms = _rows(min_p, rows, device, torch.float32, "min_p")
    if bool((ks < 1).any()):
        raise ValueError("top_k must be >= 1")
    if bool((~torch.isfinite(ps) | (ps <= 0) | (ps > 1)).any()):
        raise ValueError("top_p must be finite and in (0, 1]")
    if bool((~torch.isfinite(ms) | (ms < 0) | (ms > 1)).any()):
        raise ValueError("min_p must be finite and in [0, 1]")
    if bool(((ks >= TOP_K_ALL) & (ps == 1.0) & (ms == 0.0)).all()):
        return None, None, None
    return ks, ps, ms


def sampling_support(logits: torch.Tensor, top_ks, top_ps, min_ps) -> torch.Tensor:
    """bool [R, V]: the tokens that survive the joint filter (never empty: the arg-max always stays)."""
    x = logits.detach().float()
    R, V = x.shape
    order = torch.sort(x, dim=-1, descending=True, stable=True)
    sorted_logits, idx = order.values, order.indices
    probs = torch.softmax(sorted_logits, dim=-1)
    rank = torch.arange(V, device=x.device).unsqueeze(0)
    keep = rank < top_ks.clamp_max(V).unsqueeze(1)
    before = probs.cumsum(-1) - probs
    keep &= before < top_ps.unsqueeze(1)
    keep &= probs >= min_ps.unsqueeze(1) * probs[:, :1]
    keep[:, 0] = True
    out = torch.zeros_like(keep)
    out.scatter_(1, idx, keep)
    return out


def selected_logprob(logits: torch.Tensor, targets: torch.Tensor, top_k=TOP_K_ALL, top_p=1.0, min_p=0.0,
                     row_chunk: int = ROW_CHUNK):
    """(log-probability of ``targets`` on the filtered support [R], in_support [R] bool).

    Differentiable in ``logits``.  A target outside its row's support has probability zero under
    the behaviour policy; its entry is ``-inf`` and ``in_support`` is False so the caller can mask
    it."""
    R, V = logits.shape
    ks, ps, ms = normalize_sampling_transforms(top_k, top_p, min_p, rows=R, device=logits.device)
    if ks is None:
        lp = torch.log_softmax(logits.float(), dim=-1).gather(1, targets.view(-1, 1)).squeeze(1)
        return lp, torch.ones(R, dtype=torch.bool, device=logits.device)
    lps, oks = [], []
    for r0 in range(0, R, row_chunk):
        sl = slice(r0, min(R, r0 + row_chunk))
        x = logits[sl].float()
        sup = sampling_support(x, ks[sl], ps[sl], ms[sl])
        masked = x.masked_fill(~sup, float("-inf"))
        lse = torch.logsumexp(masked, dim=-1)
        t = targets[sl].view(-1, 1)
        ok = sup.gather(1, t).squeeze(1)
        val = x.gather(1, t).squeeze(1) - lse
        lps.append(torch.where(ok, val, torch.full_like(val, float("-inf"))))
        oks.append(ok)
    return torch.cat(lps), torch.cat(oks)


def support_workspace_bytes(vocab_size: int, row_chunk: int = ROW_CHUNK) -> int:
    """Peak temporary bytes of one row chunk (sorted values + indices + probabilities + masks)."""
    return row_chunk * vocab_size * (4 + 8 + 4 + 4 + 2)


def filtered_token_logprobs(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, *,
                            temperature: float = 1.0, top_k=TOP_K_ALL, top_p=1.0, min_p=0.0,
                            chunk_tokens: int = 1024, ignore_index: int = -100):
    """Log-probability of every label token under the lm-head distribution restricted to the
    sampling support, chunk by chunk so only ``chunk_tokens x vocab`` logits exist at a time.

    ``hidden`` [T, H], ``weight`` [V, H], ``labels`` [T]; per-row ``top_k / top_p / min_p`` may be
    tensors of shape [T].  Returns (logprobs [T] fp32, in_support [T] bool); ignored positions get 0
    and True.  Differentiable in ``hidden`` and ``weight`` (each chunk's logits are recomputed in
    backward through activation checkpointing, so they are never all alive)."""
    from torch.utils.checkpoint import checkpoint
    T = hidden.shape[0]
    lab = labels.reshape(-1)
    valid = lab != ignore_index
    safe = torch.where(valid, lab, torch.zeros_like(lab))

    def rows(v, s, e):
        return v[s:e] if isinstance(v, torch.Tensor) else v

    def chunk_fn(h, w, tgt, k, p, m):
        logits = (h.float() @ w.float().t()) if not h.is_cuda else torch.nn.functional.linear(h, w).float()
        if temperature != 1.0:
            logits = logits / temperature
        lp, ok = selected_logprob(logits, tgt, k, p, m)
        return lp, ok

    lps, oks = [], []
    needs_grad = torch.is_grad_enabled() and (hidden.requires_grad or weight.requires_grad)
    for s in range(0, T, chunk_tokens):
        e = min(T, s + chunk_tokens)
        args = (hidden[s:e], weight, safe[s:e], rows(top_k, s, e), rows(top_p, s, e), rows(min_p, s, e))
        if needs_grad:
            lp, ok = checkpoint(chunk_fn, *args, use_reentrant=False)
        else:
            lp, ok = chunk_fn(*args)
        lps.append(lp)
        oks.append(ok)
    lp, ok = torch.cat(lps), torch.cat(oks)
    lp = torch.where(valid, lp, torch.zeros_like(lp))
    return lp, ok | ~valid
