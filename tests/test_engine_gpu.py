"""Engine scheduling on one GPU: the optimizer issued on its own stream (next forward waits unit by
unit) and the per-unit early gradient norms give the same training run as the serial order."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(overlap: bool, early_norm: bool, recompute: bool, steps: int = 6, accum: int = 1):
    from xorl_b200.models import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.ops import _lib
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    torch.cuda.set_device(0)
    reset_parallel_state()
    ps = init_parallel_state(device_type="cuda")
    cfg = preset("qwen3-8b", num_hidden_layers=3, hidden_size=512, intermediate_size=1536,
                 num_attention_heads=4, num_key_value_heads=2, vocab_size=4096)
    eng = Zero3Engine(DecoderLM(cfg, device="meta"), ps, compute_dtype=torch.bfloat16,
                      device=torch.device("cuda", 0), recompute=recompute)
    eng.overlap_optimizer, eng.early_grad_norm = overlap, early_norm
    opt = build_optimizer(eng, lr=1e-3, weight_decay=0.01)
    T = 512
    g = torch.Generator(device="cpu").manual_seed(0)
    data = [torch.randint(0, cfg.vocab_size, (T + 1,), generator=g).cuda() for _ in range(2)]
    cu = torch.tensor([0, 200, 512], device="cuda", dtype=torch.int32)
    losses, norms = [], []
    for s in range(steps):
        opt.zero_grad()
        total = 0.0
        for a in range(accum):
            ids = data[(s + a) % 2]
            eng.final_micro_batch = a == accum - 1
            total = total + eng.forward_backward(ids[:-1], ids[1:], cu_seqlens=cu, grad_scale=1.0 / (T * accum))
        eng.finish_grad_sync()
        norm, coef = eng.grad_norm_and_clip_coef(1.0)
        opt.step(clip_coef=coef)
        losses.append(total)
        norms.append(norm)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    eng.sync_optimizer()
    weights = torch.cat([g_.master.flatten() for g_ in eng.all_groups()]).clone()
    return [float(l) for l in losses], [float(n) for n in norms], weights


@pytest.mark.parametrize("recompute", [True, False])
def test_overlapped_optimizer_is_bit_identical_to_serial(recompute):
    l0, n0, w0 = _run(False, True, recompute)
    l1, n1, w1 = _run(True, True, recompute)
    assert l0 == l1 and n0 == n1, (l0, l1, n0, n1)
    assert torch.equal(w0, w1)
    assert min(l0) < l0[0] - 0.3 and all(x == x for x in l0), l0      # the run learns its two batches


def test_early_gradient_norms_match_the_single_pass():
    l0, n0, _ = _run(True, False, True)
    l1, n1, _ = _run(True, True, True)
    for a, b in zip(n0, n1):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), (n0, n1)
    for a, b in zip(l0, l1):
        assert abs(a - b) < 2e-2, (l0, l1)


def test_gradient_accumulation_with_early_norms():
    """With two micro-batches the partial norms of the first are discarded: same result as the
    single pass after the last micro-batch."""
    l0, n0, _ = _run(True, False, True, steps=4, accum=2)
    l1, n1, _ = _run(True, True, True, steps=4, accum=2)
    for a, b in zip(n0, n1):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), (n0, n1)


def test_anyprecision_adamw_with_moments_in_host_memory():
    """bf16 moments kept in pinned host memory and streamed in group by group (next group's copy under the
    current group's update), update in chunks: the weights of the plain bf16-moment optimizer, bit for bit."""
    from xorl_b200.models import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    torch.cuda.set_device(0)
    cfg = preset("qwen3-8b", num_hidden_layers=3, hidden_size=512, intermediate_size=1536,
                 num_attention_heads=4, num_key_value_heads=2, vocab_size=4096)
    g = torch.Generator(device="cpu").manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (513,), generator=g).cuda()
    cu = torch.tensor([0, 200, 512], device="cuda", dtype=torch.int32)
    out = []
    for okw in ({}, {"state_cpu_offload": True, "denominator_chunk_size": 100000}):
        reset_parallel_state()
        ps = init_parallel_state(device_type="cuda")
        eng = Zero3Engine(DecoderLM(cfg, device="meta"), ps, compute_dtype=torch.bfloat16, device=torch.device("cuda", 0))
        opt = build_optimizer(eng, lr=1e-3, weight_decay=0.01, optimizer_type="anyprecision_adamw",
                              optimizer_dtype="bf16", optimizer_kwargs=okw)
        if okw:
            assert all(t.device.type == "cpu" and t.is_pinned() for t in opt.exp_avg.values())
        for _ in range(4):
            opt.zero_grad()
            eng.forward_backward(ids[:-1], ids[1:], cu_seqlens=cu, grad_scale=1.0 / 512)
            eng.finish_grad_sync()
            _, coef = eng.grad_norm_and_clip_coef(1.0)
            opt.step(clip_coef=coef)
        eng.sync_optimizer()
        out.append({n: t.float().clone() for n, t in eng.iter_full_tensors("master")})
    for n, t in out[0].items():
        assert torch.equal(t, out[1][n]), n
    reset_parallel_state()
