"""Hugging Face weight import on two gloo ranks: the three load modes fill identical shards, and a
rank that cannot read the checkpoint makes every rank fail together."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _worker(tmp):
    import datetime
    import torch.distributed as dist
    from xorl_b200.checkpoint.hf_io import MultiStreamH2D, load_hf_weights, save_hf_weights
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.parallel.state import init_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank = dist.get_rank()
    ps = init_parallel_state(device_type="cpu")
    cfg = preset("tiny-qwen3")

    def engine(seed):
        m = DecoderLM(cfg, dtype=torch.float32, device="meta")
        return Zero3Engine(m, ps, compute_dtype=torch.float32, device=torch.device("cpu"), seed=seed)

    src = engine(0)
    save_hf_weights(src, tmp, cfg, dtype=torch.float32)
    want = [g.master.clone() for g in src.all_groups()]
    for mode in ("all_ranks", "broadcast", "grouped"):
        dst = engine(1 + rank)
        assert not load_hf_weights(dst, tmp, cfg, mode=mode)
        for g, w in zip(dst.all_groups(), want):
            assert torch.equal(g.master, w), (mode, g.name)
        if mode != "all_ranks":
            st = dst.loaded_weight_stats
            assert st["reader"] == 0 and (st["h2d_copies"] > 0) == (rank == 0)
    # rank 1 is pointed at an empty directory: both ranks raise, nobody is left in a collective
    empty = os.path.join(tmp, "empty")
    os.makedirs(empty, exist_ok=True)
    with pytest.raises(RuntimeError, match="rank 1"):
        load_hf_weights(engine(3), empty if rank == 1 else tmp, cfg, mode="all_ranks")
    assert MultiStreamH2D(torch.device("cpu")).to_device(torch.ones(3)).sum() == 3
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.distributed
def test_load_modes_agree_and_fail_together(tmp_path):
    from dist_utils import run_distributed
    run_distributed(__file__, 2, str(tmp_path))


if __name__ == "__main__":
    _worker(sys.argv[1])
