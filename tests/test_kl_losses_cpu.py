"""Full-vocabulary teacher-student divergences (streaming and vocabulary-parallel), single-sample
KL estimators and loss reducers against dense fp64 references."""
import os
import subprocess
import sys

import pytest
import torch

from xorl_b200.ops import kl_losses as K

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _case(N=37, H=16, V=101, seed=0):
    g = torch.Generator().manual_seed(seed)
    hs, ht = torch.randn(N, H, generator=g), torch.randn(N, H, generator=g)
    ws, wt = torch.randn(V, H, generator=g), torch.randn(V, H, generator=g)
    lab = torch.randint(0, V, (N,), generator=g)
    lab[::5] = -100
    return hs, ws, ht, wt, lab


def _dense(hs, ws, ht, wt, lab, kind):
    ls = torch.log_softmax(hs.double() @ ws.double().t(), -1)
    lt = torch.log_softmax(ht.double() @ wt.double().t(), -1)
    kl = (ls.exp() * (ls - lt)).sum(-1) if kind == "reverse_kl" else (lt.exp() * (lt - ls)).sum(-1)
    return kl * (lab != -100)


@pytest.mark.parametrize("kind", K.KINDS)
@pytest.mark.parametrize("chunk", [32, 101, 0])
def test_streaming_kl_matches_dense(kind, chunk):
    hs, ws, ht, wt, lab = _case()
    hs.requires_grad_(), ws.requires_grad_()
    out = K.streaming_kl(hs, ws, ht, wt, lab, kind, vocab_chunk=chunk)
    out.sum().backward()
    hd, wd = hs.detach().double().requires_grad_(), ws.detach().double().requires_grad_()
    ref = _dense(hd, wd, ht, wt, lab, kind)
    ref.sum().backward()
    assert torch.allclose(out.double(), ref, atol=2e-5)
    assert (out[lab == -100] == 0).all()
    assert torch.allclose(hs.grad.double(), hd.grad, atol=5e-5) and torch.allclose(ws.grad.double(), wd.grad, atol=5e-5)


def test_kl_penalty_estimators():
    torch.manual_seed(0)
    lp, ref = torch.randn(64, requires_grad=True), torch.randn(64)
    d = (lp - ref).detach()
    assert torch.allclose(K.kl_penalty(lp, ref, "k1"), d)
    assert torch.allclose(K.kl_penalty(lp, ref, "abs"), d.abs())
    assert torch.allclose(K.kl_penalty(lp, ref, "k2"), 0.5 * d * d)
    k3 = K.kl_penalty(lp, ref, "k3")
    assert (k3 >= -1e-6).all() and torch.allclose(k3, (torch.exp(-d) + d - 1).clamp(max=10.0), atol=1e-5)
    # "+": value of the estimator, gradient of k2
    v = K.kl_penalty(lp, ref, "k3+")
    (g,) = torch.autograd.grad(v.sum(), lp)
    assert torch.allclose(v, k3) and torch.allclose(g, d)
    with pytest.raises(ValueError):
        K.kl_penalty(lp, ref, "k9")


def test_reducers_add_up_across_shards():
    vals = torch.arange(12.0)
    mask = torch.tensor([1.0] * 10 + [0.0] * 2)
    full = K.TokenPartial(torch.tensor(10.0))(vals, mask)
    parts = sum(K.TokenPartial(torch.tensor(10.0))(vals[a:b], mask[a:b]) for a, b in ((0, 5), (5, 12)))
    assert torch.allclose(full, parts) and torch.allclose(full, vals[:10].sum() / 10)
    # two sequences of 6 tokens split over two context-parallel ranks (3 + 3 tokens each)
    glob = torch.tensor([6.0, 6.0])
    want = (vals[:6].sum() / 6 + (vals[6:] * mask[6:]).sum() / 6) / 2
    r0 = K.SequencePartial(torch.tensor(2.0), torch.tensor([0, 3, 6]), glob)(torch.cat([vals[0:3], vals[6:9]]),
                                                                            torch.cat([mask[0:3], mask[6:9]]))
    r1 = K.SequencePartial(torch.tensor(2.0), torch.tensor([0, 3, 6]), glob)(torch.cat([vals[3:6], vals[9:12]]),
                                                                            torch.cat([mask[3:6], mask[9:12]]))
    assert torch.allclose(r0 + r1, want)


def test_full_vocab_diagnostics():
    hs, ws, ht, wt, lab = _case()
    rk, fk, agree = K.full_vocab_diagnostics(hs, ws, ht, wt, lab, vocab_chunk=40)
    n = (lab != -100).sum()
    assert torch.allclose(rk.double(), _dense(hs, ws, ht, wt, lab, "reverse_kl").sum() / n, atol=1e-5)
    assert torch.allclose(fk.double(), _dense(hs, ws, ht, wt, lab, "forward_kl").sum() / n, atol=1e-5)
    same = K.full_vocab_diagnostics(hs, ws, hs, ws, lab, vocab_chunk=40)
    assert same[0].abs() < 1e-6 and same[2] == 1.0


def test_vocab_parallel_kl_two_ranks():
    env = dict(os.environ, PYTHONPATH=REPO, MASTER_ADDR="127.0.0.1", MASTER_PORT="29631", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, __file__], env=dict(env, RANK=str(r), WORLD_SIZE="2"),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "VP_KL_OK" in outs[0]


def _worker():
    import torch.distributed as dist
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    hs, ws, ht, wt, lab = _case(V=102)
    sh = 102 // world
    for kind in K.KINDS:
        h = hs.clone().requires_grad_()
        w = ws[rank * sh:(rank + 1) * sh].clone().requires_grad_()
        out = K.vocab_parallel_kl(h, w, ht, wt[rank * sh:(rank + 1) * sh].clone(), lab, dist.group.WORLD, kind, vocab_chunk=17)
        out.sum().backward()
        hd, wd = hs.double().requires_grad_(), ws.double().requires_grad_()
        ref = _dense(hd, wd, ht, wt, lab, kind)
        ref.sum().backward()
        assert torch.allclose(out.double(), ref, atol=2e-5), kind
        assert torch.allclose(h.grad.double(), hd.grad, atol=5e-5), kind          # summed over ranks
        assert torch.allclose(w.grad.double(), wd.grad[rank * sh:(rank + 1) * sh], atol=5e-5), kind
    dist.barrier()
    if rank == 0:
        print("VP_KL_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    _worker()


def test_policy_losses_with_reference_penalty_and_statistics():
    from xorl_b200.ops import rl_losses as R
    torch.manual_seed(0)
    T = 40
    lp = (torch.randn(T) * 0.3 - 2).requires_grad_()
    old = lp.detach() + torch.randn(T) * 0.1
    ref = lp.detach() + torch.randn(T) * 0.2
    adv = torch.randn(T)
    mask = (torch.rand(T) > 0.2).float()
    base, m0 = R.policy_loss(lp, mask, old, adv)
    pen, m1 = R.policy_loss(lp, mask, old, adv, ref_logprobs=ref, kl_coef=0.5, kl_estimator="k3", compute_kl_stats=True)
    k3 = K.kl_penalty(lp, ref, "k3")
    assert torch.allclose(pen, base + 0.5 * (k3 * mask).sum())
    assert torch.allclose(m1["kl_ref"], (k3 * mask).sum() / mask.sum())
    for key in ("kl_sample_train_k3", "logratio_max", "entropy_sample", "ratio_mean", "frac_ratio_outside_half_double"):
        assert key in m1 and torch.isfinite(m1[key])
    assert m1["kl_sample_train_k3"] >= 0
    # the penalty pulls towards the reference: its gradient is that of the estimator
    (g_pen,) = torch.autograd.grad(pen, lp, retain_graph=True)
    (g_base,) = torch.autograd.grad(base, lp, retain_graph=True)
    (g_k3,) = torch.autograd.grad((k3 * mask).sum(), lp)
    assert torch.allclose(g_pen, g_base + 0.5 * g_k3, atol=1e-6)
    g, _ = R.LOSS_REGISTRY["grpo"](lp, mask, old, adv, ref_logprobs=ref)
    assert torch.allclose(g, base + 0.04 * (k3 * mask).sum())
    # truncated importance sampling reports how often it truncated
    _, m2 = R.policy_loss(lp, mask, old, adv, tis_cap=1.05, sampling_logprobs=old - 0.2)
    assert float(m2["tis_clipfrac"]) == 1.0 and float(m2["tis_mean"]) > 1.05
    # OPD: estimator modes
    sf, ms = R.opd_loss(lp, mask, ref)
    k2, _ = R.opd_loss(lp, mask, ref, loss_mode="k2")
    assert torch.allclose(k2, (0.5 * (lp - ref) ** 2 * mask).sum()) and "reverse_kl" in ms
    (gs,) = torch.autograd.grad(sf, lp, retain_graph=True)
    (g2,) = torch.autograd.grad(k2, lp)
    assert torch.allclose(gs, g2, atol=1e-6)          # score-function advantage and k2 share their gradient
