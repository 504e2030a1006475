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


def _mean(x, mask):
    return _masked_sum(x, mask) / mask.sum().clamp_min(1)


def kl_statistics(lp, old_logprobs, mask) -> Dict[str, torch.Tensor]:
    """Diagnostics of the drift between the policy that sampled and the policy being trained
    (src/xorl/ops/loss/policy_loss.py:262-310): the k3 estimate of their KL, the log-ratio's mean and
    extremes, the sampler's entropy estimate, the share of tokens whose ratio left [0.5, 2]."""
    with torch.no_grad():
        from .kl_losses import kl_penalty
        lr_ = (lp - old_logprobs).detach()
        valid = mask > 0
        big = torch.where(valid, lr_, torch.zeros_like(lr_))
        return {"kl_sample_train_k3": _mean(kl_penalty(old_logprobs, lp.detach(), "k3"), mask),
                "logratio_mean": _mean(lr_, mask), "abs_logratio_mean": _mean(lr_.abs(), mask),
                "logratio_max": big.max() if big.numel() else big.sum(), "logratio_min": big.min() if big.numel() else big.sum(),
                "entropy_sample": _mean(-old_logprobs, mask),
                "frac_ratio_outside_half_double": _mean((lr_.abs() > 0.6931471805599453).float(), mask),
                "ratio_mean": _mean(torch.exp(lr_), mask)}


def policy_loss(lp, mask, old_logprobs, advantages, clip_low: float = 0.2, clip_high: float = 0.2,
                tis_cap: float = 0.0, sampling_logprobs=None, ref_logprobs=None, kl_coef: float = 0.0,
                kl_estimator: str = "k3", compute_kl_stats: bool = False, **_):
    """PPO clipped surrogate; optional truncated importance sampling against the sampler's log-probs
    (TIS, policy_loss.py:81-135); optional penalty ``kl_coef * KL(policy || reference)`` estimated on
    the sampled tokens from ``ref_logprobs`` (the frozen base model's log-probabilities: the runner's
    ``forward`` with ``loss_fn_config: {reference: true}``) with any estimator of ``ops.kl_losses``."""
    ratio = torch.exp(lp - old_logprobs)
    clipped = torch.clamp(ratio, 1.0 - clip_low, 1.0 + clip_high)
    obj = torch.minimum(ratio * advantages, clipped * advantages)
    metrics = {}
    if tis_cap and sampling_logprobs is not None:
        tis = torch.exp(old_logprobs - sampling_logprobs).detach()
        obj = obj * tis.clamp(max=tis_cap)
        metrics.update(tis_mean=_mean(tis, mask), tis_clipfrac=_mean((tis > tis_cap).float(), mask))
    metrics["clip_frac"] = _mean(((ratio - clipped).abs() > 0).float(), mask)
    loss = -_masked_sum(obj, mask)
    if kl_coef and ref_logprobs is not None:
        from .kl_losses import kl_penalty
        kl = kl_penalty(lp, ref_logprobs, kl_estimator)
        loss = loss + kl_coef * _masked_sum(kl, mask)
        metrics["kl_ref"] = _mean(kl.detach(), mask)
    if compute_kl_stats:
        metrics.update(kl_statistics(lp, old_logprobs, mask))
    return loss, metrics


def grpo(lp, mask, old_logprobs, advantages, clip_low: float = 0.2, clip_high: float = 0.2, ref_logprobs=None,
         kl_coef: float = 0.04, kl_estimator: str = "k3", **kw):
    """GRPO: the clipped surrogate on group-normalised advantages with the k3 penalty towards the reference
    policy in the loss (src/xorl/ops/loss/grpo_loss.py)."""
    return policy_loss(lp, mask, old_logprobs, advantages, clip_low, clip_high, ref_logprobs=ref_logprobs,
                       kl_coef=kl_coef, kl_estimator=kl_estimator, **kw)


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


def opd_loss(lp, mask, teacher_logprobs, loss_mode: str = "score_function", **_):
    """On-policy distillation on sampled tokens.  ``score_function`` (default): log p_student - log p_teacher
    as the per-token advantage, gradient through the score function (an unbiased estimate of the reverse-KL
    gradient).  Any estimator name of ``ops.kl_losses.kl_penalty`` (``k1``, ``k2``, ``k3``, ``abs``, with or
    without the ``+`` suffix) differentiates that estimator of KL(student || teacher) instead
    (src/xorl/ops/loss/opd_loss.py:47-96)."""
    adv = (lp.detach() - teacher_logprobs)
    metrics = {"reverse_kl": _mean(adv, mask)}
    if loss_mode == "score_function":
        return _masked_sum(adv * lp, mask), metrics
    from .kl_losses import kl_penalty
    return _masked_sum(kl_penalty(lp, teacher_logprobs, loss_mode), mask), metrics


LOSS_REGISTRY: Dict[str, Callable] = {
    "causallm_loss": cross_entropy, "cross_entropy": cross_entropy,
    "importance_sampling": importance_sampling, "cispo": cispo, "policy_loss": policy_loss,
    "ppo": policy_loss, "grpo": grpo, "drgrpo": drgrpo, "opd_loss": opd_loss,
}
