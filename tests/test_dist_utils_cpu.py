"""Token-normalised loss, padding synchronisation, bf16 stochastic reduce-scatter, replicated
gradient sync (two gloo ranks), activation offload and the per-component timer (single process)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def test_activation_offload_matches_plain_engine():
    from test_zero_cpu import engine_curve
    from xorl_b200.parallel import zero
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    ref = engine_curve(3)
    orig = zero.Zero3Engine.__init__

    def patched(self, *a, **k):
        k["activation_offload"] = True
        orig(self, *a, **k)

    zero.Zero3Engine.__init__ = patched
    try:
        got = engine_curve(3)
    finally:
        zero.Zero3Engine.__init__ = orig
    assert got == ref


def test_offloader_pools_host_buffers():
    from xorl_b200.parallel.zero import ActivationOffloader

    class E:
        device = torch.device("cpu")

    off = ActivationOffloader(E())
    x = torch.randn(8, 4)
    item = off.offload((x, None))
    back = off.fetch(item)
    assert torch.equal(back[0], x) and back[1] is None
    item2 = off.offload((x * 2, None))
    assert item2.host[0].data_ptr() == item.host[0].data_ptr()      # buffer reused
    assert off.bytes_offloaded == 2 * x.numel() * 4


def test_stochastic_rounding_is_unbiased():
    from xorl_b200.parallel.dist_utils import stochastic_round_bf16
    g = torch.Generator().manual_seed(0)
    x = torch.full((200000,), 1.0 + 2 ** -10)          # between two bf16 values (spacing 2^-7)
    r = stochastic_round_bf16(x, g).float()
    assert set(r.unique().tolist()) == {1.0, 1.0 + 2 ** -7}
    assert abs(r.mean().item() - x[0].item()) < 2e-4


def test_per_component_timer():
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.utils.component_timer import PerComponentTimer
    m = DecoderLM(preset("tiny-qwen3"), dtype=torch.float32)
    m.init_weights(0)
    t = PerComponentTimer(m)
    ids = torch.randint(0, 1024, (1, 64))
    m(ids, labels=ids)
    tot = t.flush()
    assert t.counts["Attention"] == 2 and t.counts["MLP"] == 2 and tot["Attention"] > 0
    t.remove()
    assert "Attention" in t.summary()


@pytest.mark.distributed
def test_two_rank_helpers():
    from dist_utils import run_distributed
    out = run_distributed(__file__, 2)
    assert "HELPERS_OK" in out


def _worker():
    import torch.distributed as dist
    from xorl_b200.parallel import dist_utils as du
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = dist.group.WORLD
    # token-normalised loss: rank r has r+1 tokens with per-token loss r+1
    lm = torch.tensor(float(rank + 1), requires_grad=True)
    out = du.token_normalised_loss(lm, torch.tensor(rank + 1), g)
    assert abs(out.item() - (1 * 1 + 2 * 2) / 3) < 1e-6
    out.backward()
    assert abs(lm.grad.item() - (rank + 1) / 3 * world) < 1e-6
    # padding: rank 0 has 5 tokens, rank 1 has 9 -> both 12 with multiple_of 4
    T = 5 if rank == 0 else 9
    mb = {"input_ids": torch.ones(1, T, dtype=torch.long), "labels": torch.ones(1, T, dtype=torch.long),
          "position_ids": torch.arange(T).unsqueeze(0), "cu_seqlens": torch.tensor([0, T], dtype=torch.int32)}
    (p,) = du.synchronize_micro_batch_padding([mb], g, multiple_of=4)
    assert p["input_ids"].shape[-1] == 12 and (p["labels"][0, T:] == -100).all()
    assert p["cu_seqlens"].tolist() == [0, T, 12] and p["position_ids"][0, T:].tolist() == list(range(12 - T))
    # bf16 all-to-all reduce-scatter: exact for values representable in bf16
    grad = (torch.arange(8, dtype=torch.float32) + 1) * (rank + 1)
    shard = torch.zeros(4)
    du.stochastic_bf16_all_to_all_reduce_scatter(grad, shard, g)
    expect = (torch.arange(8, dtype=torch.float32) + 1)[rank * 4:(rank + 1) * 4] * 3
    assert torch.equal(shard, expect), (shard, expect)
    du.stochastic_bf16_all_to_all_reduce_scatter(grad, shard, g, accumulate=True)
    assert torch.equal(shard, 2 * expect)
    dist.barrier()
    if rank == 0:
        print("HELPERS_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    _worker()


def test_lr_schedule_matches_the_reference_lambdas():
    """(step, lr) pairs of the three decay styles against the closed forms of
    src/xorl/optim/lr_scheduler.py:117,146,183: warm-up is ``step / max(1, warmup)`` starting at
    ``lr_start`` on step 0, the full rate arrives at step ``warmup``."""
    import math
    from xorl_b200.optim.lr_scheduler import build_lr_scheduler

    class Opt:
        lr = None

        def set_lr(self, lr):
            self.lr = lr

    def ref(step, style, total=100, lr=1e-3, lr_min=1e-5, lr_start=1e-4, warm=0.1, decay=0.8):
        w, d = int(total * warm), int(total * decay)
        if step < w:
            return lr_start + (lr - lr_start) * step / max(1, w)
        if style == "constant":
            return lr
        if step >= d:
            return lr_min
        prog = (step - w) / max(1, d - w)
        r = lr_min / lr
        f = (1 - prog) if style == "linear" else 0.5 * (1 + math.cos(math.pi * prog))
        return lr * (r + (1 - r) * f)

    for style in ("constant", "linear", "cosine"):
        o = Opt()
        sch = build_lr_scheduler(o, 100, 1e-3, 1e-5, 1e-4, 0.1, style, 0.8)
        for step in range(100):
            assert abs(o.lr - ref(step, style)) < 1e-12, (style, step, o.lr, ref(step, style))
            sch.step()
    o = Opt()
    build_lr_scheduler(o, 100, 1e-3, lr_start=0.0, lr_warmup_ratio=0.1)
    assert o.lr == 0.0                      # step 0 trains at lr_start
