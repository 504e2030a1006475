"""Hugging Face safetensors import / export for models held by the ZeRO engine.

Export gathers one unit at a time (fp32 master -> bf16), splits fused tensors back to HF names and
writes sharded ``model-xxxxx-of-yyyyy.safetensors`` with an index plus ``config.json``
(src/xorl/models/module_utils.py:2594-2825).  Import streams the safetensors files and fills each
rank's shard (src/xorl/models/module_utils.py:1337-1917)."""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch
import torch.distributed as dist

from .handlers import get_checkpoint_handler


def save_hf_weights(engine, out_dir: str, cfg, dtype: torch.dtype = torch.bfloat16,
                    max_shard_bytes: int = 5 * 2 ** 30) -> None:
    from safetensors.torch import save_file
    rank0 = engine.ps.rank == 0
    handler = get_checkpoint_handler(cfg)
    if rank0:
        os.makedirs(out_dir, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    tied = cfg.tie_word_embeddings
    for name, full in engine.iter_full_tensors("master"):
        if not rank0:
            continue
        for hf_name, t in handler.to_hf(name, full):
            t = t.to(dtype).cpu().contiguous()
            nbytes = t.numel() * t.element_size()
            if size + nbytes > max_shard_bytes and shards[-1]:
                shards.append({})
                size = 0
            shards[-1][hf_name] = t
            size += nbytes
    if rank0:
        n = len(shards)
        weight_map = {}
        for i, sd in enumerate(shards):
            fname = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
            save_file(sd, os.path.join(out_dir, fname), metadata={"format": "pt"})
            for k in sd:
                weight_map[k] = fname
        if n > 1:
            with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
        cfg.save_pretrained(out_dir)
    if dist.is_initialized():
        dist.barrier()


def _open_index(path: str) -> Dict[str, str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return json.load(f)["weight_map"]
    from safetensors import safe_open
    out = {}
    for fn in sorted(os.listdir(path)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(path, fn), "pt") as f:
                for k in f.keys():
                    out[k] = fn
    return out


class MultiStreamH2D:
    """Host -> device copies spread over a few CUDA streams with pinned staging buffers, so that
    the page-locked copy of tensor i + 1 overlaps the DMA of tensor i
    (src/xorl/models/module_utils.py:926, ``_MultiStreamDMA``).  On CPU it is a plain copy."""

    def __init__(self, device: torch.device, streams: int = 2, staging_bytes: int = 256 << 20):
        self.device = device
        self.cuda = device.type == "cuda"
        self.n = max(1, streams)
        self.i = 0
        self.copies = 0
        if self.cuda:
            self.streams = [torch.cuda.Stream(device) for _ in range(self.n)]
            self.staging = [torch.empty(staging_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(self.n)]
            self.events = [None] * self.n

    def to_device(self, t: torch.Tensor) -> torch.Tensor:
        self.copies += 1
        if not self.cuda:
            return t.to(self.device)
        k = self.i
        self.i = (self.i + 1) % self.n
        nbytes = t.numel() * t.element_size()
        if nbytes > self.staging[k].numel():
            return t.to(self.device)                      # larger than a staging slot: direct copy
        if self.events[k] is not None:
            self.events[k].synchronize()                  # the slot's previous DMA has finished
        pinned = self.staging[k][:nbytes].view(t.dtype).reshape(t.shape)
        pinned.copy_(t)
        out = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        with torch.cuda.stream(self.streams[k]):
            out.copy_(pinned, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.streams[k])
        self.events[k] = ev
        torch.cuda.current_stream().wait_event(ev)
        return out


def _weight_signature(weight_map: Dict[str, str]) -> str:
    import hashlib
    h = hashlib.sha256()
    for k in sorted(weight_map):
        h.update(k.encode())
        h.update(b"\0")
    return h.hexdigest()[:16]


def check_weight_signatures(path: str, readers_only_ok: bool, is_reader: bool) -> Dict[str, str]:
    """Every rank reports whether it can open the checkpoint and a digest of its tensor names; all
    ranks raise together when one cannot or the digests differ, before any sub-group collective
    could leave the others waiting (src/xorl/models/module_utils.py:1889-1917)."""
    err, sig, wm = "", "", {}
    if is_reader or not readers_only_ok:
        try:
            wm = _open_index(path)
            sig = _weight_signature(wm)
            if not wm:
                err = f"no safetensors tensors under {path}"
        except Exception as e:  # noqa: BLE001
            err = f"{type(e).__name__}: {e}"
    if dist.is_initialized() and dist.get_world_size() > 1:
        reports = [None] * dist.get_world_size()
        dist.all_gather_object(reports, (err, sig))
    else:
        reports = [(err, sig)]
    errs = [f"rank {r}: {e}" for r, (e, _) in enumerate(reports) if e]
    sigs = {s_ for _, s_ in reports if s_}
    if errs:
        raise RuntimeError("checkpoint not readable on every reader: " + "; ".join(errs))
    if len(sigs) > 1:
        raise RuntimeError(f"ranks see different checkpoints under {path}: digests {sorted(sigs)}")
    return wm


def _reader_ranks(mode: str) -> List[int]:
    """``broadcast``: rank 0 reads.  ``grouped``: the lowest rank of every host reads and serves the
    ranks of its host (src/xorl/models/module_utils.py:1861)."""
    world = dist.get_world_size()
    if mode == "broadcast":
        return [0] * world
    import socket
    hosts = [None] * world
    dist.all_gather_object(hosts, socket.gethostname())
    first: Dict[str, int] = {}
    for r, h in enumerate(hosts):
        first.setdefault(h, r)
    return [first[h] for h in hosts]


def load_hf_weights(engine, path: str, cfg, strict: bool = True, mode: str = "all_ranks",
                    h2d_streams: int = 2) -> List[str]:
    """Fills every rank's shards from a Hugging Face safetensors directory.

    ``all_ranks``: every rank reads the tensors that overlap its shard (the page cache serves
    repeats).  ``broadcast`` / ``grouped``: one reader (rank 0 / the first rank of each host) reads
    and transforms every tensor once and broadcasts it to the ranks it serves, which keep their
    slice; file-system traffic drops from world x checkpoint to one (or hosts) x checkpoint."""
    multi = dist.is_initialized() and dist.get_world_size() > 1
    ps = engine.ps
    # served modes walk the same parameter list on every rank and broadcast whole tensors: with
    # pipeline stages (different lists) or expert parallelism (different expert slices per rank)
    # every rank reads for itself
    same_lists = getattr(ps, "pp_size", 1) == 1 and getattr(ps, "ep_size", 1) == 1
    if mode in ("broadcast", "grouped") and multi and same_lists:
        return _load_hf_weights_served(engine, path, cfg, strict, mode, h2d_streams)
    check_weight_signatures(path, readers_only_ok=False, is_reader=True)
    return _load_hf_weights_all_ranks(engine, path, cfg, strict)


def _is_adapter_param(pname: str) -> bool:
    """LoRA matrices are created by this framework, never read from a base-model checkpoint."""
    return "lora_A" in pname or "lora_B" in pname


class _PackedSource:
    """QLoRA bases: the parameter ``<module>.qparts.<part>`` is filled by quantising the module's
    full-precision weight from the checkpoint (src/xorl/qlora/utils.py:346 ``maybe_quantize_qlora``).
    ``base_name`` maps the packed parameter to the name its weight would have without QLoRA."""

    def __init__(self, model):
        self.model = model
        self._last = (None, None)

    @staticmethod
    def split(pname: str):
        if ".qparts." not in pname:
            return None
        mod, key = pname.split(".qparts.")
        return mod, key

    @staticmethod
    def base_name(mod: str) -> str:
        return mod[:-2] if mod.endswith("_q") else mod + ".weight"      # experts.gate_up_proj_q / linear

    def part(self, mod: str, key: str, full_weight: torch.Tensor) -> torch.Tensor:
        if self._last[0] != mod:
            m = self.model.get_submodule(mod)
            w = m.local_slice(full_weight) if hasattr(m, "local_slice") else full_weight
            self._last = (mod, m.quantize_parts(w))
        return self._last[1][key]


def _load_hf_weights_served(engine, path, cfg, strict, mode, h2d_streams) -> List[str]:
    from safetensors import safe_open
    rank = dist.get_rank()
    readers = _reader_ranks(mode)
    my_reader = readers[rank]
    is_reader = my_reader == rank
    wm = check_weight_signatures(path, readers_only_ok=True, is_reader=is_reader)
    # one sub-group per reader (created by every rank, in the same order)
    groups = {}
    for rd in sorted(set(readers)):
        members = [r for r, x in enumerate(readers) if x == rd]
        groups[rd] = dist.new_group(members) if len(set(readers)) > 1 else None
    pg = groups[my_reader]
    handler = get_checkpoint_handler(cfg)
    h2d = MultiStreamH2D(engine.device, h2d_streams)
    handles: Dict[str, object] = {}
    packed = _PackedSource(engine.model)

    def read(name: str) -> torch.Tensor:
        fn = wm[name]
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), "pt")
        return handles[fn].get_tensor(name)

    missing: List[str] = []
    for g in engine.all_groups():
        # the ranks served by one reader may hold different slices: walk all parameters of the
        # group in the same order everywhere
        for pname, p in g.named_params:
            if _is_adapter_param(pname):
                continue
            packed_of = _PackedSource.split(pname)
            src_name = _PackedSource.base_name(packed_of[0]) if packed_of else pname
            srcs = handler.hf_sources(src_name)
            if cfg.tie_word_embeddings and pname.startswith("lm_head"):
                srcs = ["model.embed_tokens.weight"]
            meta = [None]
            if is_reader:
                if all(s_ in wm for s_ in srcs):
                    t = handler.from_hf(src_name, [read(s_) for s_ in srcs]).contiguous()
                    if packed_of:
                        t = packed.part(packed_of[0], packed_of[1], t).contiguous()
                    meta = [(tuple(t.shape), t.dtype)]
            dist.broadcast_object_list(meta, src=my_reader, group=pg)
            if meta[0] is None:
                missing.append(pname)
                continue
            shape, dtype = meta[0]
            buf = h2d.to_device(t) if is_reader else torch.empty(shape, dtype=dtype, device=engine.device)
            dist.broadcast(buf, src=my_reader, group=pg)
            engine.load_full_tensors({pname: buf}, strict=False)
    engine.loaded_weight_stats = {"mode": mode, "reader": my_reader, "h2d_copies": h2d.copies}
    if strict and missing:
        raise KeyError(f"weights missing from {path}: {missing[:8]}")
    return missing


def _load_hf_weights_all_ranks(engine, path: str, cfg, strict: bool = True) -> List[str]:
    """Every rank reads the tensors it needs (all ranks read; the page cache serves repeats)."""
    from safetensors import safe_open
    handler = get_checkpoint_handler(cfg)
    weight_map = _open_index(path)
    handles: Dict[str, object] = {}

    def read(name: str) -> torch.Tensor:
        fn = weight_map[name]
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), "pt")
        return handles[fn].get_tensor(name)

    missing: List[str] = []
    packed = _PackedSource(engine.model)
    for g in engine.all_groups():
        tensors = {}
        for i, _, _ in g.param_segments_in_shard():
            pname = g.named_params[i][0]
            if _is_adapter_param(pname):
                continue
            packed_of = _PackedSource.split(pname)
            src_name = _PackedSource.base_name(packed_of[0]) if packed_of else pname
            srcs = handler.hf_sources(src_name)
            if cfg.tie_word_embeddings and pname.startswith("lm_head"):
                srcs = ["model.embed_tokens.weight"]
            if not all(s in weight_map for s in srcs):
                missing.append(pname)
                continue
            t = handler.from_hf(src_name, [read(s) for s in srcs])
            tensors[pname] = packed.part(packed_of[0], packed_of[1], t) if packed_of else t
        engine.load_full_tensors(tensors, strict=False) if tensors else None
    if strict and missing:
        raise KeyError(f"weights missing from {path}: {missing[:8]}")
    return missing
