"""Checkpoint pieces taken straight from flat shards: box decomposition, placement maps, and a
checkpoint written under tensor parallelism + ZeRO that a single process resumes from."""
import math
import os
import random
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from xorl_b200.checkpoint.boxes import BoxedTensor, RowMap, flat_range_boxes  # noqa: E402


def test_flat_ranges_tile_into_boxes():
    rng = random.Random(0)
    for shape in [(7,), (5, 7), (3, 4, 5), (2, 3, 4, 5), (1, 9), ()]:
        n = math.prod(shape) if shape else 1
        full = torch.arange(float(n)).reshape(shape if shape else (1,))
        for _ in range(40):
            a = rng.randrange(0, n)
            b = rng.randrange(a, n + 1)
            boxes = flat_range_boxes(shape, a, b)
            assert len(boxes) <= 2 * max(len(shape) - 1, 0) + 1
            got = []
            pos = a
            for off, size, fa, fb in boxes:
                assert fa == pos and fb - fa == math.prod(size)         # flat order, no gaps
                pos = fb
                sl = tuple(slice(o, o + s) for o, s in zip(off, size))
                got.append(full[sl].reshape(-1))
            assert pos == b
            if boxes:
                assert torch.equal(torch.cat(got), full.reshape(-1)[a:b])


def test_row_sections_and_column_slices_land_in_the_full_tensor():
    full = torch.arange(12.0 * 6).reshape(12, 6)
    sections, tp = (8, 2, 2), 2                                      # fused q | k | v rows
    rebuilt = torch.full_like(full, -1)
    for rank in range(tp):
        local = torch.cat([full[0 + rank * 4:0 + rank * 4 + 4], full[8 + rank:9 + rank], full[10 + rank:11 + rank]])
        flat = local.reshape(-1).clone()
        # two ZeRO shards of the local slice
        for a, b in ((0, 17), (17, flat.numel())):
            bt = BoxedTensor.from_flat(flat, local.shape, a, b, 0, full.shape, RowMap.row_sections(sections, tp, rank))
            for off, size, t in bt.boxes:
                rebuilt[off[0]:off[0] + size[0], off[1]:off[1] + size[1]] = t
    assert torch.equal(rebuilt, full)
    rebuilt.fill_(-1)
    for rank in range(tp):                                          # row-parallel weight: column halves
        local = full[:, rank * 3:(rank + 1) * 3].contiguous()
        bt = BoxedTensor.from_flat(local.reshape(-1), local.shape, 5, 31, 0, full.shape,
                                   RowMap([(0, 12, 0)], col_offset=rank * 3))
        for off, size, t in bt.boxes:
            rebuilt[off[0]:off[0] + size[0], off[1]:off[1] + size[1]] = t
        assert torch.equal(rebuilt.reshape(12, 2, 3)[:, rank].reshape(-1)[5:31], local.reshape(-1)[5:31])


@pytest.mark.distributed
def test_checkpoint_written_under_tp2_zero2_resumes_without_tp(tmp_path):
    """tp 2 x ZeRO 2 writes its pieces; a ZeRO-2 run without tensor parallelism (same data-parallel
    size, hence the same batches) resumes from them and continues the uninterrupted loss curve."""
    import yaml
    from dist_utils import run_distributed
    from test_pp_cpu import _cfg, _losses
    cfg = _cfg(tmp_path, "tp", tensor_parallel_size=2, max_steps=4, save_steps=2)
    run_distributed("-m", 4, "xorl_b200.cli.train", cfg)
    ref = _losses(tmp_path, "tp")
    ckpt = tmp_path / "tp" / "checkpoints" / "global_step_2"
    assert (ckpt / ".metadata").exists()
    cfg2 = _cfg(tmp_path, "resumed", max_steps=4, load_checkpoint_path=str(ckpt))
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg2)
    got = _losses(tmp_path, "resumed")
    assert len(got) >= 2
    for a, b in zip(ref[2:], got[-2:]):
        assert abs(a - b) < 3e-4, (ref, got)
