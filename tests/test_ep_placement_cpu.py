"""Which experts a rank holds, and what a checkpoint written under expert parallelism contains.

* Random initialisation: expert ``e`` on EP rank ``r`` is expert ``r * E / ep + e`` of the
  single-process model, bit for bit.
* Full ``[E, ...]`` tensors handed to ``load_full_tensors`` (the Hugging Face import path) land as
  this rank's rows, and ``iter_full_tensors`` returns all ``E`` experts again.
* A run at 4 ranks / EP 2 (expert grid 2 x 2: ``Shard(0)`` over ep, ``Shard(1)`` over ep_fsdp)
  trains, saves, and the checkpoint continues with the same losses at 1 rank, at 2 ranks / EP 2 and
  at 4 ranks / EP 4; all of them follow the single-process loss curve.
"""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

STEPS_BEFORE, STEPS_AFTER = 3, 3


def _data(step, vocab=1024, batch=4, seq=96):
    g = torch.Generator().manual_seed(4321 + step)
    ids = torch.randint(0, vocab, (batch, seq + 1), generator=g)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def _build(ep: int):
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import get_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    cfg = preset("tiny-qwen3-moe", router_aux_loss_coef=0.0)
    m = DecoderLM(cfg, dtype=torch.float32, device="meta")
    eng = Zero3Engine(m, get_parallel_state(), compute_dtype=torch.float32, device=torch.device("cpu"), seed=0)
    opt = build_optimizer(eng, lr=5e-3, weight_decay=0.0)
    return cfg, eng, opt


def _train(eng, opt, first_step, n, world, rank):
    import torch.distributed as dist
    losses = []
    for s in range(first_step, first_step + n):
        x, y = _data(s % 2)           # two alternating batches: the loss falls as they are learnt
        opt.zero_grad()
        loss = eng.forward_backward(x[rank::world], y[rank::world], grad_scale=1.0 / y.numel())
        eng.finish_grad_sync()
        _, coef = eng.grad_norm_and_clip_coef(1.0)
        opt.step(clip_coef=coef)
        if world > 1:
            dist.all_reduce(loss)
        losses.append(loss.item())
    return losses


def _worker(mode: str, ep: int, workdir: str):
    import torch.distributed as dist
    from xorl_b200.checkpoint.checkpointer import DistributedCheckpointer
    from xorl_b200.parallel.state import init_parallel_state
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    init_parallel_state(device_type="cpu", ep_size=ep, dp_mode="fsdp2")
    cfg, eng, opt = _build(ep)
    ck = DistributedCheckpointer(eng, opt, os.path.join(workdir, "ckpt"))
    if mode == "placement":
        local = {n: t.clone() for n, t in eng.iter_full_tensors("master", ep_full=False) if ".experts." in n}
        full = {n: t.clone() for n, t in eng.iter_full_tensors("master") if ".experts." in n}
        torch.save({"local": local, "full": full, "ep_rank": eng.ps.rank_in("ep")},
                   os.path.join(workdir, f"placement_{rank}.pt"))
        # the import path: full tensors in, this rank's rows kept
        g = torch.Generator().manual_seed(7)
        given = {n: torch.randn(t.shape, generator=g) for n, t in full.items()}
        eng.load_full_tensors(given, strict=False)
        back = {n: t for n, t in eng.iter_full_tensors("master") if ".experts." in n}
        ok = all(torch.equal(back[n], given[n]) for n in given)
        flag = torch.tensor([1.0 if ok else 0.0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print("IMPORT_OK " + json.dumps(bool(flag.item())))
    elif mode == "save":
        a = _train(eng, opt, 0, STEPS_BEFORE, world, rank)
        ck.save(STEPS_BEFORE, path=os.path.join(workdir, "ckpt", "step"))
        b = _train(eng, opt, STEPS_BEFORE, STEPS_AFTER, world, rank)
        if rank == 0:
            print("LOSSES " + json.dumps(a + b))
    else:
        ck.load(os.path.join(workdir, "ckpt", "step"))
        b = _train(eng, opt, STEPS_BEFORE, STEPS_AFTER, world, rank)
        if rank == 0:
            print("LOSSES " + json.dumps(b))
    dist.barrier()
    dist.destroy_process_group()


def _single_process(tmp=None, load=None):
    from xorl_b200.checkpoint.checkpointer import DistributedCheckpointer
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    cfg, eng, opt = _build(1)
    if load is None:
        return cfg, eng, _train(eng, opt, 0, STEPS_BEFORE + STEPS_AFTER, 1, 0)
    DistributedCheckpointer(eng, opt, str(tmp)).load(load)
    return cfg, eng, _train(eng, opt, STEPS_BEFORE, STEPS_AFTER, 1, 0)


def _losses(out):
    return json.loads([l for l in out.splitlines() if l.startswith("LOSSES ")][-1][7:])


@pytest.mark.distributed
def test_expert_rows_of_each_ep_rank_match_the_single_process_model(tmp_path):
    from dist_utils import run_distributed
    out = run_distributed(__file__, 2, "placement", "2", str(tmp_path))
    assert "IMPORT_OK true" in out, out[-2000:]
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    _, eng, _ = _build(1)
    whole = {n: t.clone() for n, t in eng.iter_full_tensors("master") if ".experts." in n}
    assert whole
    seen = set()
    for r in range(2):
        rec = torch.load(tmp_path / f"placement_{r}.pt")
        er = rec["ep_rank"]
        seen.add(er)
        for n, t in rec["local"].items():
            El = whole[n].shape[0] // 2
            assert t.shape[0] == El
            assert torch.equal(t, whole[n][er * El:(er + 1) * El]), (n, r)       # bit for bit
            assert not torch.equal(t, whole[n][(1 - er) * El:(2 - er) * El])
        for n, t in rec["full"].items():
            assert torch.equal(t, whole[n]), n
    assert seen == {0, 1}


@pytest.mark.distributed
def test_checkpoint_written_under_ep_reloads_at_other_ep_sizes(tmp_path):
    from dist_utils import run_distributed
    ref = _single_process()[2]
    saved = _losses(run_distributed(__file__, 4, "save", "2", str(tmp_path), timeout=900))
    assert len(saved) == STEPS_BEFORE + STEPS_AFTER
    for a, b in zip(ref, saved):
        assert abs(a - b) < 3e-4, (ref, saved)
    assert ref[-1] < ref[0] - 0.05, ref                      # the curve moves: a wrong state would show
    ckpt = str(tmp_path / "ckpt" / "step")
    runs = {
        "1 rank": _single_process(tmp_path, ckpt)[2],
        "2 ranks ep 2": _losses(run_distributed(__file__, 2, "load", "2", str(tmp_path), timeout=900)),
        "4 ranks ep 4": _losses(run_distributed(__file__, 4, "load", "4", str(tmp_path), timeout=900)),
    }
    for name, got in runs.items():
        for a, b in zip(ref[STEPS_BEFORE:], got):
            assert abs(a - b) < 3e-4, (name, ref, got)


if __name__ == "__main__":
    _worker(sys.argv[1], int(sys.argv[2]), sys.argv[3])
