"""Sampling-filter programme: support against a per-row Python restatement, renormalised
log-probabilities, validation and the identity shortcut."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xorl_b200.ops.sampling_transforms import (TOP_K_ALL, normalize_sampling_transforms,  # noqa: E402
                                               sampling_support, selected_logprob)


def _support_ref(row, k, p, m):
    order = sorted(range(len(row)), key=lambda i: (-row[i], i))
    mx = max(row)
    e = [math.exp(v - mx) for v in row]
    z = sum(e)
    keep, before = set(), 0.0
    for r, i in enumerate(order):
        pr = e[i] / z
        if r < k and before < p and pr >= m * (e[order[0]] / z):
            keep.add(i)
        before += pr
    keep.add(order[0])
    return keep


def test_support_matches_python_restatement_including_ties():
    torch.manual_seed(0)
    R, V = 40, 50
    logits = (torch.randn(R, V) * 2).round()                 # rounding makes ties
    ks = torch.randint(1, 12, (R,))
    ps = torch.rand(R).clamp(0.05, 1.0)
    ms = torch.rand(R) * 0.3
    ks[0], ps[0], ms[0] = TOP_K_ALL, 1.0, 0.0
    sup = sampling_support(logits, ks, ps, ms)
    for r in range(R):
        want = _support_ref(logits[r].tolist(), int(ks[r]), float(ps[r]), float(ms[r]))
        assert set(sup[r].nonzero().flatten().tolist()) == want, r
    assert sup[0].all()


def test_selected_logprob_renormalises_and_differentiates():
    torch.manual_seed(1)
    R, V = 70, 33
    logits = torch.randn(R, V, requires_grad=True)
    targets = logits.argmax(-1)
    lp, ok = selected_logprob(logits, targets, top_k=5, top_p=0.9, min_p=0.05, row_chunk=32)
    assert ok.all()
    full = torch.log_softmax(logits, -1).gather(1, targets.view(-1, 1)).squeeze(1)
    assert (lp >= full - 1e-6).all()                         # less mass in the denominator
    lp.sum().backward()
    sup = sampling_support(logits, torch.full((R,), 5), torch.full((R,), 0.9), torch.full((R,), 0.05))
    assert (logits.grad[~sup] == 0).all()
    # a target outside the support
    worst = logits.argmin(-1)
    lp2, ok2 = selected_logprob(logits.detach(), worst, top_k=3)
    assert not ok2.any() and torch.isinf(lp2).all()
    # identity parameters: plain log-softmax, no filter tensors built
    assert normalize_sampling_transforms(rows=R, device="cpu") == (None, None, None)
    lp3, _ = selected_logprob(logits.detach(), targets)
    torch.testing.assert_close(lp3, full.detach())


def test_validation():
    with pytest.raises(ValueError):
        normalize_sampling_transforms(top_k=0, rows=2, device="cpu")
    with pytest.raises(ValueError):
        normalize_sampling_transforms(top_p=0.0, rows=2, device="cpu")
    with pytest.raises(TypeError):
        normalize_sampling_transforms(top_k=torch.tensor([1.0, 2.0]), rows=2, device="cpu")
    with pytest.raises(ValueError):
        normalize_sampling_transforms(min_p=torch.tensor([0.1], dtype=torch.float32), rows=2, device="cpu")


def test_filtered_token_logprobs_chunks_and_gradients():
    from xorl_b200.ops.sampling_transforms import filtered_token_logprobs
    torch.manual_seed(2)
    T, H, V = 50, 16, 40
    h = torch.randn(T, H, requires_grad=True)
    w = (torch.randn(V, H) * 0.3).requires_grad_()
    logits = (h @ w.t()) / 0.7
    labels = logits.argmax(-1)
    labels[3] = -100
    ks = torch.randint(2, 9, (T,))
    lp, ok = filtered_token_logprobs(h, w, labels, temperature=0.7, top_k=ks, top_p=0.95, min_p=0.0, chunk_tokens=16)
    want, ok2 = selected_logprob(logits, labels.clamp_min(0), ks, 0.95, 0.0)
    keep = labels != -100
    torch.testing.assert_close(lp[keep], want[keep], rtol=1e-5, atol=1e-5)
    assert lp[3] == 0 and ok.all()
    g1 = torch.autograd.grad(lp.sum(), [h, w])
    g2 = torch.autograd.grad(want[keep].sum(), [h, w])
    for a, b in zip(g1, g2):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
