"""ZeRO-3 engine on CPU/gloo: the tiny-Qwen3 plumbing configuration.

Two gloo ranks, fp32, tied embeddings, batch 2 x 128 uniform tokens, AdamW lr 1e-4, 10 steps: the
loss curve must match a single-process run of plain autograd + torch.optim.AdamW."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _data(step, vocab=1024, batch=2, seq=128):
    g = torch.Generator().manual_seed(1234 + step)
    ids = torch.randint(0, vocab, (batch, seq + 1), generator=g)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def reference_curve(steps=10):
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    torch.manual_seed(0)
    m = DecoderLM(preset("tiny-qwen3"), dtype=torch.float32)
    m.init_weights(0)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    losses = []
    for s in range(steps):
        x, y = _data(s)
        opt.zero_grad()
        loss = m(x, labels=y, grad_scale=1.0 / y.numel())["loss"]
        loss.backward()
        torch.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        opt.step()
        losses.append(loss.item())
    return losses


def engine_curve(steps=10, world=1, rank=0, optimizer="adamw", lr=1e-4, fixed_batch=False, recompute=True):
    import torch.distributed as dist
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import get_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    m = DecoderLM(preset("tiny-qwen3"), dtype=torch.float32, device="meta")
    eng = Zero3Engine(m, get_parallel_state(), compute_dtype=torch.float32,
                      device=torch.device("cpu"), seed=0, recompute=recompute)
    opt = build_optimizer(eng, lr=lr, weight_decay=0.0, optimizer_type=optimizer,
                          optimizer_kwargs={"muon_lr": 0.01} if optimizer == "muon" else None)
    losses = []
    for s in range(steps):
        x, y = _data(0 if fixed_batch else s)
        # each rank takes its slice of the global batch; normalisation is by the global count
        xs, ys = x[rank::world], y[rank::world]
        opt.zero_grad()
        loss = eng.forward_backward(xs, ys, grad_scale=1.0 / y.numel())
        eng.finish_grad_sync()
        norm, coef = eng.grad_norm_and_clip_coef(1.0)
        opt.step(clip_coef=coef)
        if world > 1:
            dist.all_reduce(loss)
        losses.append(loss.item())
    return losses


def test_engine_single_process_matches_autograd():
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    ref = reference_curve(4)
    got = engine_curve(4)
    for a, b in zip(ref, got):
        assert abs(a - b) < 1e-5, (ref, got)


@pytest.mark.distributed
def test_fsdp2_two_gloo_ranks_match_single_process():
    from dist_utils import run_distributed
    out = run_distributed(__file__, 2)
    got = json.loads([l for l in out.splitlines() if l.startswith("LOSSES ")][-1][7:])
    ref = reference_curve(10)
    assert len(got) == 10
    for a, b in zip(ref, got):
        assert abs(a - b) < 1e-5, (ref, got)


def test_engine_without_recompute_matches_autograd():
    """Activations kept from the forward pass (no recomputation): same losses, one process and two
    gloo ranks (parameters stay gathered between a layer's forward and its backward)."""
    from dist_utils import run_distributed
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    ref = reference_curve(6)
    got = engine_curve(6, recompute=False)
    out = run_distributed(__file__, 2, "norecompute")
    got2 = json.loads([l for l in out.splitlines() if l.startswith("LOSSES ")][-1][7:])
    for a, b, c in zip(ref, got, got2):
        assert abs(a - b) < 1e-5 and abs(a - c) < 1e-5, (ref, got, got2)


def test_muon_single_process_descends_and_orthogonalises():
    from xorl_b200.optim.muon import gram_newton_schulz, newton_schulz
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    torch.manual_seed(0)
    for shape in ((48, 160), (160, 48)):
        G = torch.randn(shape)
        X, Y = newton_schulz(G).float(), gram_newton_schulz(G).float()
        sv = torch.linalg.svdvals(X)
        assert sv.min() > 0.5 and sv.max() < 1.3                 # all singular values pushed towards 1
        assert (X - Y).norm() / X.norm() < 0.06                  # Gram form is the same iteration
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    got = engine_curve(8, optimizer="muon", lr=1e-3, fixed_batch=True)
    assert got[-1] < got[0] - 0.05, got


@pytest.mark.distributed
def test_muon_two_gloo_ranks_match_single_process():
    from dist_utils import run_distributed
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    out = run_distributed(__file__, 2, "muon")
    got = json.loads([l for l in out.splitlines() if l.startswith("LOSSES ")][-1][7:])
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    ref = engine_curve(6, optimizer="muon", lr=1e-3, fixed_batch=True)
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-3, (ref, got)                      # bf16 iteration, shard-independent


def _distsign_probe(world, rank):
    """One majority-vote sign SGD step; returns the update of one weight matrix."""
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import get_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    m = DecoderLM(preset("tiny-qwen3"), dtype=torch.float32, device="meta")
    eng = Zero3Engine(m, get_parallel_state(), compute_dtype=torch.float32, device=torch.device("cpu"), seed=0)
    opt = build_optimizer(eng, lr=1e-2, weight_decay=0.0, optimizer_type="distsignsgd")
    name = "layers.0.mlp.down_proj.weight"
    before = dict(eng.iter_full_tensors("master"))[name].clone()
    x, y = _data(0)
    opt.zero_grad()
    eng.forward_backward(x[rank::world], y[rank::world], grad_scale=1.0 / y.numel())
    eng.finish_grad_sync()
    opt.step()
    after = dict(eng.iter_full_tensors("master"))[name]
    return (after - before)


@pytest.mark.distributed
def test_distsignsgd_votes_before_the_reduction():
    """Two ranks: the update is -lr * (sign(g_0) + sign(g_1)) / 2 with g_r the gradient of rank r's
    own micro-batch, not -lr * sign(g_0 + g_1)."""
    from dist_utils import run_distributed
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim.optimizer import MultiOptimizer
    out = run_distributed(__file__, 2, "distsign")
    got = torch.tensor(json.loads([l for l in out.splitlines() if l.startswith("UPDATE ")][-1][7:]))
    m = DecoderLM(preset("tiny-qwen3"), dtype=torch.float32)
    m.init_weights(0)
    x, y = _data(0)
    votes = 0
    for r in range(2):
        m.zero_grad()
        m(x[r::2], labels=y[r::2], grad_scale=1.0 / y.numel())["loss"].backward()
        votes = votes + torch.sign(m.layers["0"].mlp.down_proj.weight.grad)
    want = -1e-2 * votes / 2
    assert (got - want[:4, :16]).abs().max() < 1e-6, (got, want[:4, :16])
    assert set(torch.unique((got / -1e-2 * 2).round()).tolist()) <= {-2.0, -1.0, 0.0, 1.0, 2.0}
    with pytest.raises(ValueError):
        MultiOptimizer({})


if __name__ == "__main__":
    import torch.distributed as dist
    from xorl_b200.parallel.state import init_parallel_state
    dist.init_process_group("gloo")
    init_parallel_state(device_type="cpu", dp_mode="fsdp2")
    if len(sys.argv) > 1 and sys.argv[1] == "distsign":
        upd = _distsign_probe(dist.get_world_size(), dist.get_rank())
        if dist.get_rank() == 0:
            print("UPDATE " + json.dumps(upd[:4, :16].tolist()))
        dist.destroy_process_group()
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "muon":
        curve = engine_curve(6, dist.get_world_size(), dist.get_rank(), optimizer="muon", lr=1e-3,
                             fixed_batch=True)
    elif len(sys.argv) > 1 and sys.argv[1] == "norecompute":
        curve = engine_curve(6, dist.get_world_size(), dist.get_rank(), recompute=False)
    else:
        curve = engine_curve(10, dist.get_world_size(), dist.get_rank())
    if dist.get_rank() == 0:
        print("LOSSES " + json.dumps(curve))
    dist.destroy_process_group()


def test_eval_loss_equals_the_training_loss_at_the_same_weights():
    """``eval_loss`` (no gradients, units gathered one by one, lm-head log-probabilities) on a packed batch with
    ignored labels gives the loss that ``forward_backward`` reports for that batch before its update."""
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    eng = Zero3Engine(DecoderLM(preset("tiny-qwen3"), device="meta"), ps, compute_dtype=torch.float32,
                      device=torch.device("cpu"))
    opt = build_optimizer(eng, lr=1e-3, weight_decay=0.0)
    ids = torch.randint(0, 1024, (1, 257))
    x, y = ids[:, :-1], ids[:, 1:].clone()
    y[0, 99] = -100
    cu = torch.tensor([0, 100, 256], dtype=torch.int32)
    pos = torch.cat([torch.arange(100), torch.arange(156)])[None]
    for _ in range(3):
        s, n = eng.eval_loss(x, y, position_ids=pos, cu_seqlens=cu)
        assert int(n) == 255
        opt.zero_grad()
        loss = eng.forward_backward(x, y, position_ids=pos, cu_seqlens=cu, grad_scale=1.0 / float(n))
        eng.finish_grad_sync()
        opt.step()
        assert abs(float(s / n) - float(loss)) < 1e-5
    reset_parallel_state()


def test_anyprecision_adamw_memory_options_change_no_value():
    """Moments in host memory and the update in chunks: the same weights after three steps as the plain
    bf16-moment optimizer, bit for bit."""
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    torch.manual_seed(0)
    ids = torch.randint(0, 1024, (2, 65))
    results = []
    for okw in ({}, {"state_cpu_offload": True, "denominator_chunk_size": 1000}):
        reset_parallel_state()
        ps = init_parallel_state(device_type="cpu")
        eng = Zero3Engine(DecoderLM(preset("tiny-qwen3"), device="meta"), ps, compute_dtype=torch.float32,
                          device=torch.device("cpu"), seed=3)
        opt = build_optimizer(eng, lr=1e-3, weight_decay=0.01, optimizer_type="anyprecision_adamw", optimizer_dtype="bf16",
                              optimizer_kwargs=okw)
        assert opt.offload == bool(okw) and opt.chunk == okw.get("denominator_chunk_size", 0)
        for _ in range(3):
            opt.zero_grad()
            eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)
            eng.finish_grad_sync()
            _, coef = eng.grad_norm_and_clip_coef(1.0)
            opt.step(clip_coef=coef)
        results.append({n: t.clone() for n, t in eng.iter_full_tensors("master")})
    for n, t in results[0].items():
        assert torch.equal(t, results[1][n]), n
    reset_parallel_state()
