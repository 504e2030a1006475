"""Host-side cost of staging rollout-routing-replay payloads (the expert choices an inference engine
recorded, ``[tokens, moe_layers, top_k]`` per datum) from a request to a packed micro-batch:

    python -m xorl_b200.utils.r3_staging_bench --datums 64 --tokens 2048 --layers 48 --top-k 8

Times (a) writing the payloads to the side-payload store and reading them back, (b) packing the
datums (tokens, targets and routing rows) into micro-batches, (c) the pinned host -> device copy of
the packed routing tensor when a GPU is present.  One JSON line on stdout.  Same purpose as the
reference's benchmarks/r3_replay_staging_benchmark.py."""
from __future__ import annotations

import argparse
import json
import tempfile
import time

import torch


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--datums", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--pack-len", type=int, default=8192)
    a = ap.parse_args(argv)

    from ..server.packing import datums_to_micro_batch, pack_best_fit
    from ..server.side_payloads import FilesystemPayloadStore

    g = torch.Generator().manual_seed(0)
    datums = []
    for _ in range(a.datums):
        toks = torch.randint(1, 1000, (a.tokens,), generator=g).tolist()
        routed = torch.randint(0, a.experts, (a.tokens, a.layers, a.top_k), generator=g, dtype=torch.int16)
        # the flat per-datum form the orchestrator hands to the packer
        datums.append({"tokens": toks, "target_tokens": toks[1:] + [-100], "routed_experts": routed})
    payload_bytes = a.datums * a.tokens * a.layers * a.top_k * 2
    with tempfile.TemporaryDirectory() as root:
        store = FilesystemPayloadStore(root)
        t0 = time.perf_counter()
        refs = [store.put(d["routed_experts"]) for d in datums]
        t_put = time.perf_counter() - t0
        t0 = time.perf_counter()
        back = [store.get(r, delete=True) for r in refs]
        t_get = time.perf_counter() - t0
    assert all(torch.equal(b, d["routed_experts"]) for b, d in zip(back, datums))
    t0 = time.perf_counter()
    bins = pack_best_fit([len(d["tokens"]) for d in datums], a.pack_len)
    mbs = []
    for b in bins:
        ds = []
        for i in b:
            d = dict(datums[i])
            d["datum_index"] = i
            ds.append(d)
        mbs.append(datums_to_micro_batch(ds, pad_to=128))
    t_pack = time.perf_counter() - t0
    out = {"bench": "r3_replay_staging", "datums": a.datums, "tokens_per_datum": a.tokens, "moe_layers": a.layers,
           "top_k": a.top_k, "payload_mb": payload_bytes / 1e6, "store_put_s": t_put, "store_get_s": t_get,
           "pack_s": t_pack, "micro_batches": len(mbs),
           "store_mb_per_s": payload_bytes / 1e6 / max(t_put + t_get, 1e-9)}
    if torch.cuda.is_available():
        r = mbs[0]["routed_experts"].pin_memory()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r.cuda(non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        out["h2d_ms_first_micro_batch"] = e0.elapsed_time(e1)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
