"""Teacher-student divergences over the full vocabulary without ever holding ``[N, V]`` logits, and
the single-sample KL estimators used by policy-distillation losses.

* ``streaming_kl``: exact KL(student || teacher) ("reverse") or KL(teacher || student) ("forward")
  per token.  The vocabulary is walked in chunks twice in forward (normalisers, then the divergence)
  and once more in backward, so only per-token statistics are saved and peak memory is
  ``[N, vocab_chunk]`` (src/xorl/ops/loss/opd_streaming_kl.py:56-470).
* ``vocab_parallel_kl``: the same divergences when both lm-head weights are row-sharded over a
  process group: each rank forms its ``[N, V / world]`` logits, the normalisers and the divergence
  sums are all-reduced, the hidden-state gradient is summed over ranks and the weight gradient
  stays local (src/xorl/ops/loss/vocab_parallel_reverse_kl.py:1-385).
* ``kl_penalty``: k1 / abs / k2 / k3 estimators from sampled log-probabilities, with the ``+`` suffix
  for the straight-through form (value of the chosen estimator, gradient of k2)
  (src/xorl/ops/loss/opd_loss.py:47-96).
* ``TokenPartial`` / ``SequencePartial``: denominators under which per-rank, per-micro-batch shares
  add up to the global token mean or the mean of per-sequence means
  (src/xorl/ops/loss/reducers.py:20-66).

Matrix products go through ``ops.gemm.gemm`` (the tcgen05 kernel on a GPU, fp32 results); everything else is
element-wise fp32 math on ``[N, chunk]`` tiles.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

IGNORE_INDEX = -100
KINDS = ("forward_kl", "reverse_kl")


# ---------------------------------------------------------------------------------------------
# estimators on sampled log-probabilities
# ---------------------------------------------------------------------------------------------
def _penalty_value(lp: torch.Tensor, ref: torch.Tensor, mode: str) -> torch.Tensor:
    d = lp - ref
    if mode in ("kl", "k1"):
        return d
    if mode == "abs":
        return d.abs()
    if mode in ("mse", "k2"):
        return 0.5 * d.square()
    if mode in ("low_var_kl", "k3"):
        r = torch.clamp(-d, min=-20.0, max=20.0)
        return torch.clamp(torch.exp(r) - r - 1.0, min=-10.0, max=10.0)
    raise ValueError(f"unknown KL estimator {mode!r}")


def kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor, mode: str = "k3") -> torch.Tensor:
    """Per-token estimate of KL(policy || reference) from the log-probabilities of the sampled
    tokens.  ``mode + "+"``: the forward value of ``mode`` with the gradient of k2."""
    straight = mode.endswith("+")
    base = mode[:-1] if straight else mode
    value = _penalty_value(logprob, ref_logprob, base)
    if not straight or base in ("mse", "k2"):
        return value
    surrogate = 0.5 * (logprob - ref_logprob).square()
    return surrogate - surrogate.detach() + value.detach()


# ---------------------------------------------------------------------------------------------
# reducers
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TokenPartial:
    """Masked sum over a caller-supplied global token count."""
    scale: torch.Tensor

    def __call__(self, values: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        return (values * mask).sum() / self.scale.clamp(min=1.0)


@dataclass(frozen=True)
class SequencePartial:
    """Sum over local segments of (masked segment sum / the segment's global length), over a
    caller-supplied global sequence count.  Under context parallelism every rank holds a slice of
    each segment; dividing by the global length makes the slices add up to the segment mean."""
    scale: torch.Tensor
    cu_seqlens_local: torch.Tensor
    seq_lengths_global: torch.Tensor

    def __call__(self, values: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        flat = (values * mask).reshape(-1)
        lens = self.cu_seqlens_local.diff().to(torch.long)
        seg = torch.repeat_interleave(torch.arange(lens.numel(), device=flat.device), lens)
        sums = torch.zeros(lens.numel(), dtype=flat.dtype, device=flat.device).index_add(0, seg, flat[:seg.numel()])
        return (sums / self.seq_lengths_global.clamp(min=1.0)).sum() / self.scale.clamp(min=1.0)


# ---------------------------------------------------------------------------------------------
# shared pieces of the streaming / vocabulary-parallel divergences
# ---------------------------------------------------------------------------------------------
def _mm(a, b, a_mn=False, b_mn=False, out=None, accumulate=False) -> torch.Tensor:
    """fp32 ``op(a) @ op(b)^T`` in the convention of ``ops.gemm.gemm`` (tcgen05 kernel for bf16
    operands on a GPU, fp32 result without an intermediate rounding)."""
    from .gemm import gemm
    if a.is_cuda and (a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16):
        A = (a.t() if a_mn else a).float()
        B = (b if b_mn else b.t()).float()
        res = A @ B
        if out is None:
            return res
        return out.add_(res) if accumulate else out.copy_(res)
    return gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=torch.float32, accumulate=accumulate)


def _logits(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _mm(h, w)


def _online_lse(run_max, run_sum, logits):
    cmax = logits.max(dim=-1, keepdim=True).values
    new = torch.maximum(run_max, cmax)
    keep = torch.where(torch.isfinite(run_max), (run_max - new).exp(), torch.zeros_like(run_sum))
    return new, run_sum * keep + (logits - new).exp().sum(-1, keepdim=True)


def _all_reduce(t: torch.Tensor, group, op=dist.ReduceOp.SUM) -> torch.Tensor:
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=op, group=group)
    return t


def _normalisers(h, w, chunk, group) -> torch.Tensor:
    """log-sum-exp of ``h @ w.T`` per row, [N, 1] fp32, over vocabulary chunks and over the group."""
    N = h.shape[0]
    m = torch.full((N, 1), float("-inf"), device=h.device, dtype=torch.float32)
    s = torch.zeros((N, 1), device=h.device, dtype=torch.float32)
    for a in range(0, w.shape[0], chunk):
        m, s = _online_lse(m, s, _logits(h, w[a:a + chunk]))
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        gmax = _all_reduce(m.clone(), group, dist.ReduceOp.MAX)
        s = _all_reduce(s * (m - gmax).exp(), group)
        m = gmax
    return m + s.log()


class _FullVocabKL(torch.autograd.Function):
    """Per-token divergence between softmax(hs @ ws.T) and softmax(ht @ wt.T); the teacher side is a
    constant.  ``ws`` / ``wt`` may be this rank's vocabulary shard (``group`` given)."""

    @staticmethod
    def forward(ctx, hs, ws, ht, wt, mask, kind, chunk, group):
        with torch.no_grad():
            lz_s = _normalisers(hs, ws, chunk, group)
            lz_t = _normalisers(ht, wt, chunk, group)
            kl = torch.zeros((hs.shape[0], 1), device=hs.device, dtype=torch.float32)
            for a in range(0, ws.shape[0], chunk):
                lp_s = _logits(hs, ws[a:a + chunk]) - lz_s
                lp_t = _logits(ht, wt[a:a + chunk]) - lz_t
                if kind == "reverse_kl":
                    kl += (lp_s.exp() * (lp_s - lp_t)).sum(-1, keepdim=True)
                else:
                    kl += (lp_t.exp() * (lp_t - lp_s)).sum(-1, keepdim=True)
            _all_reduce(kl, group)
            kl = kl * mask.view(-1, 1)
        ctx.save_for_backward(hs, ws, ht, wt, mask, lz_s, lz_t, kl)
        ctx.cfg = (kind, chunk, group)
        return kl.view(-1)

    @staticmethod
    def backward(ctx, g):
        hs, ws, ht, wt, mask, lz_s, lz_t, kl = ctx.saved_tensors
        kind, chunk, group = ctx.cfg
        up = (g.float() * mask).view(-1, 1)
        dh = torch.zeros(hs.shape, device=hs.device, dtype=torch.float32)
        dw = torch.zeros(ws.shape, device=ws.device, dtype=torch.float32) if ctx.needs_input_grad[1] else None
        for a in range(0, ws.shape[0], chunk):
            wc = ws[a:a + chunk]
            lp_s = _logits(hs, wc) - lz_s
            p_s = lp_s.exp()
            if kind == "reverse_kl":
                # d KL / d s_v = p_s(v) (log p_s(v) - log p_t(v) - KL)
                lp_t = _logits(ht, wt[a:a + chunk]) - lz_t
                ds = p_s * (lp_s - lp_t - kl)
            else:
                # d KL(t || s) / d s_v = p_s(v) - p_t(v)
                ds = p_s - (_logits(ht, wt[a:a + chunk]) - lz_t).exp()
            ds = (ds * up).to(hs.dtype)
            _mm(ds, wc, b_mn=True, out=dh, accumulate=True)                 # dh += ds @ W_chunk
            if dw is not None:
                _mm(ds, hs, a_mn=True, b_mn=True, out=dw[a:a + chunk])      # dW_chunk = ds^T @ h
        _all_reduce(dh, group)
        return dh.to(hs.dtype), (dw.to(ws.dtype) if dw is not None else None), None, None, None, None, None, None


def _check(hs, ws, ht, wt, kind):
    if kind not in KINDS:
        raise ValueError(f"kind must be one of {KINDS}, got {kind!r}")
    if ws.shape[0] != wt.shape[0]:
        raise ValueError(f"teacher and student vocabularies differ: {wt.shape[0]} vs {ws.shape[0]}")


def streaming_kl(hidden_s: torch.Tensor, w_s: torch.Tensor, hidden_t: torch.Tensor, w_t: torch.Tensor,
                 labels: torch.Tensor, kind: str = "reverse_kl", vocab_chunk: int = 8192,
                 ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """Per-token divergence [N] (zero where ``labels == ignore_index``), exact over the whole
    vocabulary, with ``[N, vocab_chunk]`` peak memory."""
    _check(hidden_s, w_s, hidden_t, w_t, kind)
    hs, ht = hidden_s.reshape(-1, hidden_s.shape[-1]), hidden_t.reshape(-1, hidden_t.shape[-1])
    mask = (labels.reshape(-1) != ignore_index).float()
    chunk = w_s.shape[0] if vocab_chunk <= 0 else min(vocab_chunk, w_s.shape[0])
    return _FullVocabKL.apply(hs, w_s, ht.detach(), w_t.detach(), mask, kind, chunk, None)


def vocab_parallel_kl(hidden_s: torch.Tensor, w_s_shard: torch.Tensor, hidden_t: torch.Tensor,
                      w_t_shard: torch.Tensor, labels: torch.Tensor, group, kind: str = "reverse_kl",
                      vocab_chunk: int = 0, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """As ``streaming_kl`` with both lm-head weights sharded by rows over ``group``; every rank passes
    the same hidden states and gets the same per-token divergence."""
    _check(hidden_s, w_s_shard, hidden_t, w_t_shard, kind)
    hs, ht = hidden_s.reshape(-1, hidden_s.shape[-1]), hidden_t.reshape(-1, hidden_t.shape[-1])
    mask = (labels.reshape(-1) != ignore_index).float()
    chunk = w_s_shard.shape[0] if vocab_chunk <= 0 else min(vocab_chunk, w_s_shard.shape[0])
    return _FullVocabKL.apply(hs, w_s_shard, ht.detach(), w_t_shard.detach(), mask, kind, chunk, group)


def full_vocab_diagnostics(hidden_s, w_s, hidden_t, w_t, labels, vocab_chunk: int = 8192,
                           ignore_index: int = IGNORE_INDEX) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(mean reverse KL, mean forward KL, top-1 agreement) over supervised tokens, no gradients
    (src/xorl/ops/loss/opd_streaming_kl.py:373-443)."""
    with torch.no_grad():
        mask = (labels.reshape(-1) != ignore_index).float()
        n = mask.sum().clamp(min=1.0)
        rk = streaming_kl(hidden_s, w_s, hidden_t, w_t, labels, "reverse_kl", vocab_chunk, ignore_index).sum() / n
        fk = streaming_kl(hidden_s, w_s, hidden_t, w_t, labels, "forward_kl", vocab_chunk, ignore_index).sum() / n
        hs, ht = hidden_s.reshape(-1, hidden_s.shape[-1]), hidden_t.reshape(-1, hidden_t.shape[-1])
        best_s = torch.full((hs.shape[0],), float("-inf"), device=hs.device)
        best_t = best_s.clone()
        arg_s = torch.zeros(hs.shape[0], dtype=torch.long, device=hs.device)
        arg_t = arg_s.clone()
        for a in range(0, w_s.shape[0], vocab_chunk):
            for h, w, best, arg in ((hs, w_s, best_s, arg_s), (ht, w_t, best_t, arg_t)):
                v, i = _logits(h, w[a:a + vocab_chunk]).max(-1)
                upd = v > best
                best[upd], arg[upd] = v[upd], i[upd] + a
        agree = ((arg_s == arg_t).float() * mask).sum() / n
    return rk, fk, agree
