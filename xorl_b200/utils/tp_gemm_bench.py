"""All-gather -> GEMM and GEMM -> reduce-scatter of a tensor-parallel layer: the single-kernel
forms (``csrc/gemm_fused.cu``) against the collective through NCCL followed / preceded by the
plain GEMM kernel.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m xorl_b200.utils.tp_gemm_bench

Shapes are the column (qkv, gate_up) and row (o, down) linears of the chosen model at ``--tokens``
tokens split over the N ranks.  Times are CUDA events on the launching stream, after warm-up, max
over ranks; an L2-sized buffer is written between iterations.  One JSON line per case with the
roofline target: the slower of FLOPs / measured GEMM peak and NVLink bytes per GPU / 770 GB/s.
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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--nvlink-gbs", type=float, default=770.0)
    ap.add_argument("--gemm-tflops", type=float, default=1400.0)
    a = ap.parse_args(argv)
    from ..models import preset
    from ..ops import _lib
    from ..ops import gemm as gemm_ops
    from ..parallel.tp_fused import SequenceParallelTP
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    cfg = preset(a.model)
    H, I = cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    T = a.tokens
    rows = T // world
    sp = SequenceParallelTP(dist.group.WORLD, rank, world)
    flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)

    def timed(fn):
        out = []
        for i in range(a.warmup + a.iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= a.warmup:
                out.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.median(out)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def report(case, kind, ms_fused, ms_nccl, ms_gemm, flops, link_bytes):
        if rank == 0:
            target = max(flops / (a.gemm_tflops * 1e12), link_bytes / (a.nvlink_gbs * 1e9)) * 1e3
            print(json.dumps({"case": case, "kind": kind, "ranks": world, "tokens": T,
                              "fused_ms": round(ms_fused, 4), "collective_then_gemm_ms": round(ms_nccl, 4),
                              "gemm_alone_ms": round(ms_gemm, 4), "roofline_ms": round(target, 4),
                              "fused_of_roofline": round(target / ms_fused, 3),
                              "speedup_vs_unfused": round(ms_nccl / ms_fused, 3)}), flush=True)

    for name, n_out, k_in, kind in (("qkv_proj", qkv // world, H, "ag"), ("gate_up_proj", 2 * I // world, H, "ag"),
                                    ("o_proj", H, cfg.num_attention_heads * cfg.head_dim // world, "rs"),
                                    ("down_proj", H, I // world, "rs")):
        w = (torch.randn(n_out, k_in, device=dev) * 0.02).to(torch.bfloat16)
        flops = 2.0 * T * n_out * k_in
        if kind == "ag":
            x_s = torch.randn(rows, k_in, device=dev).to(torch.bfloat16)
            full = torch.empty(T, k_in, device=dev, dtype=torch.bfloat16)

            def unfused():
                dist.all_gather_into_tensor(full, x_s)
                return gemm_ops.gemm(full, w)

            ref = unfused()
            sp.fused = True
            got, _ = sp.all_gather_gemm(x_s, w)
            torch.cuda.synchronize()
            err = (got.float() - ref.float()).abs().max().item()
            assert err <= 1e-2 * ref.float().abs().max().item() + 1e-3, (name, err)
            ms_f = timed(lambda: sp.all_gather_gemm(x_s, w))
            ms_n = timed(unfused)
            ms_g = timed(lambda: gemm_ops.gemm(full, w))
            report(name, "all_gather->gemm", ms_f, ms_n, ms_g, flops, (world - 1) * rows * k_in * 2)
        else:
            h = torch.randn(T, k_in, device=dev).to(torch.bfloat16)
            out = torch.empty(rows, n_out, device=dev, dtype=torch.bfloat16)

            def unfused():
                y = gemm_ops.gemm(h, w)
                dist.reduce_scatter_tensor(out, y)
                return out

            ref = unfused().clone()
            got = sp.gemm_reduce_scatter(h, w)
            torch.cuda.synchronize()
            err = (got.float() - ref.float()).abs().max().item()
            assert err <= 2e-2 * ref.float().abs().max().item() + 1e-3, (name, err)
            ms_f = timed(lambda: sp.gemm_reduce_scatter(h, w))
            ms_n = timed(unfused)
            ms_g = timed(lambda: gemm_ops.gemm(h, w))
            report(name, "gemm->reduce_scatter", ms_f, ms_n, ms_g, flops, (world - 1) * rows * n_out * 2)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    if rank == 0:
        print(json.dumps({"fused_calls": sp.fused_calls, "unfused_calls": sp.fallback_calls}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
