"""Parameter all-gather and gradient reduce-scatter of one decoder layer through the ZeRO engine,
fused peer-memory transport against NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m xorl_b200.utils.comm_bench

Times on the device (CUDA events on the stream the collective runs on, max over ranks), after
warm-up, and prints one JSON line per transport: milliseconds, bytes that cross NVLink per GPU and
the resulting GB/s per direction next to the measured peer-copy bandwidth (770 GB/s) -- the
roofline of a collective that has no compute to hide behind.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--nvlink-gbs", type=float, default=770.0)
    a = ap.parse_args(argv)
    from ..models import preset
    from ..models.decoder import DecoderLM
    from ..ops import _lib
    from ..parallel.state import init_parallel_state
    from ..parallel.zero import Zero3Engine
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ps = init_parallel_state(device_type="cuda", dp_mode="fsdp2")
    world, rank = dist.get_world_size(), dist.get_rank()
    cfg = preset(a.model, num_hidden_layers=2, vocab_size=8192)
    from ..parallel import symm_transport
    for mode in ("nccl", "kernel", "dma"):
        # kernel: pull kernels with peer loads; dma: copy engines move the bytes, kernels reduce locally
        model = DecoderLM(cfg, device="meta")
        eng = Zero3Engine(model, ps, compute_dtype=torch.bfloat16, device=dev, seed=0)
        symm_transport.MODE = mode
        if mode != "nccl" and not eng.attach_peer_transport(required=False):
            if rank == 0:
                print(json.dumps({"transport": mode, "unavailable": "symmetric memory could not be set up"}))
            continue
        _, layers = eng._units_by_role()
        unit = layers[0]
        g = unit.groups[0]
        stream = eng.comm_stream

        def timed(fn):
            out = []
            for i in range(a.warmup + a.iters):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                fn()
                e1.record(stream)
                torch.cuda.synchronize()
                if i >= a.warmup:
                    out.append(e0.elapsed_time(e1))
            t = torch.tensor([statistics.median(out)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        def do_gather():
            eng.gather(unit)
            eng.wait_gather(unit)
            torch.cuda.current_stream().synchronize()
            eng.release(unit)

        def do_reduce():
            eng._prepare_grad_buffers(unit)
            for gg in unit.groups:
                gg.grad_full.fill_(1e-3)
            torch.cuda.current_stream().synchronize()
            eng._reduce_unit_grads(unit, collected=True)
            eng.finish_grad_sync()

        ag_ms = timed(do_gather)
        rs_ms = timed(do_reduce)
        _lib.raise_on_status()
        if rank == 0:
            elem = g.padded
            ag_bytes = elem * 2 * (world - 1) / world                     # bf16 pulled from peers
            # bytes per element on the wire: bf16 in the fused transport, the reduce dtype through NCCL
            rs_wire = 2 if mode != "nccl" else (4 if eng.reduce_dtype == torch.float32 else 2)
            rs_bytes = elem * rs_wire * (world - 1) / world
            print(json.dumps({
                "transport": mode, "n_gpus": world, "unit_params": int(g.numel), "rs_wire_bytes_per_elem": rs_wire,
                "all_gather_ms": ag_ms, "all_gather_gbs_per_gpu": ag_bytes / ag_ms / 1e6,
                "all_gather_of_nvlink": ag_bytes / ag_ms / 1e6 / a.nvlink_gbs,
                "reduce_scatter_ms": rs_ms, "reduce_scatter_gbs_per_gpu": rs_bytes / rs_ms / 1e6,
                "reduce_scatter_of_nvlink": rs_bytes / rs_ms / 1e6 / a.nvlink_gbs}))
        del eng, model
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
