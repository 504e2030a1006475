#!/usr/bin/env python
"""Headline benchmark: training tokens/s of Qwen3-8B (bf16, ZeRO-3/FSDP2, seq 4096, micro-batch 1
per GPU, packed documents with lengths uniform in [256, 4096], AdamW with fp32 master weights and
states), weak scaling over the GPUs of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with the
step inputs already on the device; ``e2e`` is the same metric through ``Trainer.train_step`` with,
every step, the host->device copy of the inputs from pinned memory and a device->host read of the
loss.  Data are synthetic, weights random-init.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count")
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"])
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--ulysses", type=int, default=1, help="Ulysses sequence-parallel size (long-context runs)")
    ap.add_argument("--ring", type=int, default=1, help="ring-attention size (long-context runs)")
    ap.add_argument("--single-doc", action="store_true", help="one document of --seq-len tokens per step")
    ap.add_argument("--ep", type=int, default=0,
                    help="expert-parallel size for MoE models (0: all ranks for MoE, 1 for dense)")
    ap.add_argument("--ep-dispatch", default="fused", choices=["fused", "alltoall"])
    ap.add_argument("--experts-dtype", default="fp8", choices=["fp8", "bf16"],
                    help="MoE models: block-scaled fp8 expert GEMMs (1x128 activation / 128x128 weight scales), "
                         "the precision the Qwen3-30B-A3B configuration names, or bf16")
    ap.add_argument("--recompute", default="auto", choices=["auto", "full", "none"],
                    help="activation recomputation; auto keeps activations when they fit (both arms "
                         "use their own gradient_checkpointing_method key)")
    ap.add_argument("--scratch-dir", default=os.environ.get("XORL_BENCH_SCRATCH", ""),
                    help="where the run may write its output directory (default: a temp dir)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
def make_packed_batch(seq_len: int, vocab: int, seed: int, single_doc: bool = False):
    """One packed row: documents with lengths uniform in [256, seq_len], tokens uniform over the
    vocabulary; the last document is cut so the row holds exactly seq_len tokens.  Returned in
    pinned host memory (next-token labels, last target of every document ignored)."""
    import numpy as np
    import torch
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=seq_len + 1, dtype=np.int64)
    cu = [0]
    while cu[-1] < seq_len:
        cu.append(seq_len if single_doc else min(seq_len, cu[-1] + int(rng.integers(256, seq_len + 1))))
    labels = ids[1:].copy()
    pos = np.zeros(seq_len, dtype=np.int64)
    for a, b in zip(cu[:-1], cu[1:]):
        pos[a:b] = np.arange(b - a)
        labels[b - 1] = -100
    row = {"input_ids": torch.from_numpy(ids[:-1].copy()), "labels": torch.from_numpy(labels),
           "position_ids": torch.from_numpy(pos), "cu_seqlens": torch.tensor(cu, dtype=torch.int32)}
    if torch.cuda.is_available():
        row = {k: v.pin_memory() for k, v in row.items()}
    row["num_valid_tokens"] = int((labels != -100).sum())
    return row


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of this process's GPU every 200 ms."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def scratch_dir(a) -> str:
    if a.scratch_dir:
        os.makedirs(a.scratch_dir, exist_ok=True)
        return a.scratch_dir
    import tempfile
    d = os.path.join(tempfile.gettempdir(), "xorl_b200_bench")
    os.makedirs(d, exist_ok=True)
    return d


def resolve_recompute(a, cfg, world: int) -> str:
    """Recomputation costs one extra forward per layer; it is only needed when the activations of
    all layers do not fit beside the sharded state.  ``auto`` turns it off whenever a rank's
    parameter/optimizer state (18 bytes per parameter over the shard group) plus the stored
    activations stay below the device memory with a safety margin."""
    if a.recompute == "full":
        return "recompute_full_layer"
    if a.recompute == "none":
        return "no_recompute"
    import torch
    total = torch.cuda.get_device_properties(0).total_memory if torch.cuda.is_available() else 0
    if cfg.is_moe:
        return "recompute_full_layer"      # expert workspaces are reused layer by layer
    params = cfg.num_parameters() if hasattr(cfg, "num_parameters") else 8.2e9
    state = 18.0 * params / world + (2.0 * params if world > 1 else 0.0)      # ZeRO shards over dp x cp
    L, H, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    acts = a.seq_len / max(1, a.ulysses * a.ring) * 2.0 * L * (6 * H + 2 * qkv + 3 * I)
    return "no_recompute" if state + acts + 12e9 < total else "recompute_full_layer"


def launch_total():
    from xorl_b200.ops import activation, attention, embedding, fp8_grouped, gemm, loss, moe, norm, optim
    return sum(m.launch_count() for m in (activation, attention, embedding, fp8_grouped, gemm, loss, moe, norm, optim))


# ------------------------------------------------------------------------------------------------
def run_ours(a):
    import torch
    import torch.distributed as dist
    from xorl_b200.arguments import (Arguments, DataArguments, ModelArguments, TrainingArguments)
    from xorl_b200.models import preset
    from xorl_b200.trainers.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    overrides = {"num_hidden_layers": a.layers} if a.layers else {}
    cfg = preset(a.model, **overrides)
    ep = (a.ep or (world if cfg.is_moe else 1)) if cfg.is_moe else 1
    # the load-balancing loss comes from the model config (router_aux_loss_coef = 1e-3)
    moe_train = dict(expert_parallel_size=ep) if cfg.is_moe else {}
    if cfg.is_moe and a.experts_dtype == "fp8":
        moe_train.update(enable_fp8_training=True, fp8_training_allow_blackwell=True,
                         fp8_training_target_modules=["experts"])
    out_dir = os.path.join(scratch_dir(a), "bench_out")
    recompute = resolve_recompute(a, cfg, world)
    args = Arguments(
        model=ModelArguments(config_path=a.model, ep_dispatch=a.ep_dispatch),
        data=DataArguments(datasets=[{"path": "dummy", "max_seq_len": 64, "num_samples": 8}],
                           sample_packing_sequence_len=a.seq_len, dataloader_pin_memory=False),
        train=TrainingArguments(output_dir=out_dir, optimizer="adamw", lr=1e-5, weight_decay=0.01,
                                max_grad_norm=1.0, micro_batch_size=1, gradient_accumulation_steps=1,
                                data_parallel_mode="fsdp2", enable_mixed_precision=True,
                                enable_gradient_checkpointing=True,
                                gradient_checkpointing_method=recompute, init_device="meta",
                                load_weights_mode="skip", save_hf_weights=False, use_wandb=False, save_steps=0,
                                save_epochs=0,
                                comm_backend=a.comm, max_steps=10 ** 9, ce_num_chunks=4,
                                ulysses_parallel_size=a.ulysses, ringattn_parallel_size=a.ring, **moe_train))
    trainer = Trainer(args, model_config=cfg)
    dev = trainer.device
    torch.cuda.reset_peak_memory_stats()
    n_total = a.warmup + a.steps
    cp = a.ulysses * a.ring
    if cp > 1:
        # every rank of a context-parallel group works on the same row and keeps its shard of it
        from xorl_b200.data import SequenceShardCollator
        ps = trainer.ps
        shard = SequenceShardCollator(a.ring, a.ulysses, ps.ringattn_rank, ps.ulysses_rank)
        host_batches = []
        for s in range(n_total):
            row = make_packed_batch(a.seq_len, cfg.vocab_size, 1000 * ps.dp_rank + s, a.single_doc)
            row.pop("num_valid_tokens")
            host_batches.append({k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in shard(row).items()})
    else:
        host_batches = [make_packed_batch(a.seq_len, cfg.vocab_size, 1000 * rank + s, a.single_doc)
                        for s in range(n_total)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- phase A: device-timed, inputs staged on the device --------------------------------------
    dev_batches = [{k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in b.items()}
                   for b in host_batches]
    for s in range(a.warmup):
        trainer.train_step([dev_batches[s]])
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = launch_total()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(a.warmup, n_total):
        out = trainer.train_step([dev_batches[s]])
    e1.record()
    barrier()
    clocks = sampler.stop()
    launches = launch_total() - l0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = ms.item() / a.steps
    tokens_per_step = a.seq_len * world // cp
    value = tokens_per_step / (ms_per_step / 1e3)
    last_loss = float(out["loss"])

    # ---- phase B: end to end through the public API -----------------------------------------------
    e2e = None
    if not a.skip_e2e:
        barrier()
        t0 = time.perf_counter()
        for s in range(a.warmup, n_total):
            out = trainer.train_step([host_batches[s]])   # pinned host tensors -> H2D inside
            _ = float(out["loss"])                          # D2H read of the step result
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values() if torch.is_tensor(v))
        e2e = {"value": tokens_per_step * a.steps / dt.item(), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": 4 * world}
    from xorl_b200.ops import _lib
    status = _lib.read_status()
    if rank == 0:
        fused = trainer.engine.symm is not None
        line = {
            "metric": "tokens/sec (device-timed, max over ranks) Qwen3-8B/30B-A3B at 1/2/4/8 B200",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {"model": a.model + (f"[{a.layers} layers: DEBUG, not the named model]" if a.layers else ""),
                       "global_batch": world // cp, "seq_len": a.seq_len,
                       "parallelism": f"fsdp{world}" + ("-fused" if fused else "-nccl" if world > 1 else "")
                       + (f"-ep{ep}-{a.ep_dispatch}" if ep > 1 else "")
                       + (f"-ring{a.ring}-ulysses{a.ulysses}" if cp > 1 else ""),
                       "optimizer": "adamw fp32 master+states", "recompute": recompute,
                       **({"experts": "block_fp8 e4m3 (1x128 / 128x128 power-of-two scales), bf16 elsewhere"
                           if a.experts_dtype == "fp8" else "bf16"} if cfg.is_moe else {}),
                       "l2": "per-step working set (16 GB of bf16 weights + activations) >> 126 MB L2",
                       "packed_docs": ("one document per row" if a.single_doc else "lengths U[256,seq_len]") + ", tokens U[vocab]"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "loss": last_loss, "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
            "status_words": status[:4],
        }
        if cfg.is_moe:
            from xorl_b200.parallel.ep_fused import PhaseTimes
            if PhaseTimes.enabled:
                line["ep_phase_ms_total"] = PhaseTimes.report()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    a = parse()
    if a.impl == "reference":
        from baseline.run_reference import run_reference
        run_reference(a)
        return
    run_ours(a)


if __name__ == "__main__":
    main()
