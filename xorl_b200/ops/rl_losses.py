"""Token-level RL / distillation losses on per-token log-probabilities, and the loss registry
(src/xorl/ops/loss/__init__.py:34-42; policy_loss.py, grpo_loss.py, cispo_loss.py,
importance_sampling_loss.py, opd_loss.py).  Every function takes new log-probs ``lp`` [T], the
inputs recorded at sampling time and a mask, and returns the **sum** over tokens (callers divide
by the global token count) plus metrics."""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch


def _masked_sum(x, mask):
    return (x * mask).sum()


def cross_entropy(lp, mask, weights=None, **_) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    w = mask if weights is None else mask * weights
    return -(lp * w).sum(), {}


def importance_sampling(lp, mask, old_logprobs, advantages, **_):
    ratio = torch.exp(lp - old_logprobs)
    loss = -_masked_sum(ratio * advantages, mask)
    return loss, {"ratio_mean": _masked_sum(ratio.detach(), mask) / mask.sum().clamp_min(1)}


def policy_loss(lp, mask, old_logprobs, advantages, clip_low: float = 0.2, clip_high: float = 0.2,
                tis_cap: float = 0.0, sampling_logprobs=None, **_):
    """PPO clipped surrogate; optional truncated importance sampling against the sampler's
    log-probs (TIS)."""
    ratio = torch.exp(lp - old_logprobs)
    clipped = torch.clamp(ratio, 1.0 - clip_low, 1.0 + clip_high)
    obj = torch.minimum(ratio * advantages, clipped * advantages)
    if tis_cap and sampling_logprobs is not None:
        obj = obj * torch.exp(old_logprobs - sampling_logprobs).clamp(max=tis_cap).detach()
    frac = _masked_sum(((ratio - clipped).abs() > 0).float(), mask) / mask.sum().clamp_min(1)
    return -_masked_sum(obj, mask), {"clip_frac": frac}


def drgrpo(lp, mask, old_logprobs, advantages, clip_low: float = 0.2, clip_high: float = 0.28,
           max_tokens: int = 0, **_):
    """Dr. GRPO: clipped surrogate normalised by a constant length instead of each sample's own."""
    loss, m = policy_loss(lp, mask, old_logprobs, advantages, clip_low, clip_high)
    if max_tokens:
        loss = loss * (mask.sum().clamp_min(1) / max_tokens)
    return loss, m


def cispo(lp, mask, old_logprobs, advantages, eps_low: float = 1.0, eps_high: float = 0.28, **_):
    """CISPO: clip the (detached) importance weight, keep every token's gradient."""
    ratio = torch.exp(lp - old_logprobs)
    w = torch.clamp(ratio, 1.0 - eps_low, 1.0 + eps_high).detach()
    return -_masked_sum(w * advantages * lp, mask), {"ratio_mean": _masked_sum(ratio.detach(), mask) / mask.sum().clamp_min(1)}


def opd_loss(lp, mask, teacher_logprobs, **_):
    """On-policy distillation: reverse KL estimate on sampled tokens, log p_student - log p_teacher
    as the per-token advantage (gradient through the score function)."""
    adv = (lp.detach() - teacher_logprobs)
    return _masked_sum(adv * lp, mask), {"reverse_kl": _masked_sum(adv, mask) / mask.sum().clamp_min(1)}


LOSS_REGISTRY: Dict[str, Callable] = {
    "causallm_loss": cross_entropy, "cross_entropy": cross_entropy,
    "importance_sampling": importance_sampling, "cispo": cispo, "policy_loss": policy_loss,
    "ppo": policy_loss, "drgrpo": drgrpo, "opd_loss": opd_loss,
}
