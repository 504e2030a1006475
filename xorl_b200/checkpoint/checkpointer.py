"""DCP save / load of the ZeRO engine's state.

Directory layout ``{output_dir}/checkpoints/global_step_{N}/`` with ``.metadata``,
``__{rank}_0.distcp``, ``extra_state/extra_state_rank_{r}.pt`` and ``checkpoint_metadata.json``;
state keys ``model.<fqn>`` and ``optimizer.state.<fqn>.{exp_avg,exp_avg_sq}`` — the layout of
src/xorl/checkpoint/checkpointer.py:795-1072.  Every rank writes the pieces of each parameter that
its flat shards hold (``checkpoint/boxes.py``: rectangular views of the shard with their offsets in
the full tensor), so a save moves no parameter between ranks and a load writes into the shards in
place; DCP stores a tensor as such a chunk list, so a checkpoint written at one world size or
parallel layout loads at another, and ``DTensor``-saved checkpoints of the same keys load too.
Expert tensors appear under their full ``[E, ...]`` shape (the reference restores them as
``Shard(0)`` over ep x ``Shard(1)`` over ep_fsdp, checkpointer.py:107-160: the same logical tensor).
"""
from __future__ import annotations

import json
import os
import re
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from ..utils.logging import info_rank0
from .handlers import from_checkpoint_fqn, to_checkpoint_fqn

_STEP_RE = re.compile(r"global_step_(\d+)$")


def resolve_checkpoint_path(path: str, checkpoint_dir: str) -> Optional[str]:
    """``auto`` -> newest ``global_step_N`` under ``checkpoint_dir`` (None when there is none)."""
    if path != "auto":
        return path
    if not os.path.isdir(checkpoint_dir):
        return None
    steps = []
    for d in os.listdir(checkpoint_dir):
        m = _STEP_RE.search(d)
        if m and os.path.exists(os.path.join(checkpoint_dir, d, ".metadata")):
            steps.append((int(m.group(1)), d))
    return os.path.join(checkpoint_dir, max(steps)[1]) if steps else None


class DistributedCheckpointer:
    def __init__(self, engine, optimizer=None, checkpoint_dir: str = "checkpoints",
                 save_async: bool = False, lora_only: bool = False):
        self.engine = engine
        self.optimizer = optimizer
        self.dir = checkpoint_dir
        self.save_async = save_async
        # lora.save_lora_only: frozen base weights stay out of the checkpoint (adapters, their
        # optimizer state and the trainer state only); loading such a checkpoint leaves the base alone
        self.lora_only = lora_only
        self._pending = None
        self._meshes: Dict[int, Any] = {}

    # ---- pieces of the flat shards ----------------------------------------------------------------
    def _placement(self, p, lshape):
        """(full shape, RowMap) of a parameter that is a tensor- or expert-parallel slice, else (None, None)."""
        from .boxes import RowMap
        ps = self.engine.ps
        spec = getattr(p, "_xb_tp", None)
        if spec is not None and ps.tp_size > 1:
            full = tuple(p._xb_full_shape)
            if spec[0] == "col":
                return full, RowMap.row_sections(spec[1] or (full[0],), ps.tp_size, ps.rank_in("tp"))
            return full, RowMap([(0, lshape[0], 0)], col_offset=ps.rank_in("tp") * lshape[1])
        if getattr(p, "_xb_ep", None) is not None and ps.ep_size > 1:
            return tuple(p._xb_full_shape), RowMap([(0, lshape[0], ps.rank_in("ep") * lshape[0])])
        if getattr(p, "_xb_lmtp", None) is not None:
            return tuple(p._xb_full_shape), RowMap([(0, lshape[0], p._xb_lmtp[0] * lshape[0])])
        return None, None

    def _state_sources(self):
        srcs = [("model.{fqn}", None)]
        opt = self.optimizer
        if opt is not None:
            for sname, per_group in opt.state.items():
                srcs.append((f"optimizer.state.{{fqn}}.{sname}", per_group))
        return srcs

    def build_state_dict(self, include_frozen: bool = True) -> Dict[str, Any]:
        """{key: BoxedTensor} over views of this rank's shards (weights: the fp32 masters, or the
        compute-dtype shard of a frozen group; optimizer state: its flat shards)."""
        from .boxes import BoxedTensor
        sd: Dict[str, Any] = {}
        eng = self.engine
        eng.sync_optimizer()
        for g in eng.all_groups():
            frozen = getattr(g, "frozen", False)
            if frozen and not include_frozen:
                continue
            s0, _ = g.shard_range()
            segs = g.param_segments_in_shard()
            for key_fmt, per_group in self._state_sources():
                if per_group is None:
                    flat = g.master if g.master is not None else g.shard_lp
                else:
                    if frozen or id(g) not in per_group:
                        continue
                    flat = per_group[id(g)]
                for i, a, b in segs:
                    name, p = g.named_params[i]
                    lshape, o = tuple(g.shapes[i]) or (1,), g.offsets[i]
                    full_shape, row_map = self._placement(p, lshape)
                    sd[key_fmt.format(fqn=to_checkpoint_fqn(name))] = BoxedTensor.from_flat(
                        flat, lshape, a + s0 - o, b + s0 - o, o - s0, full_shape, row_map)
        return sd

    # ---- save -----------------------------------------------------------------------------------
    def save(self, global_step: int, extra_state: Optional[Dict[str, Any]] = None,
             path: Optional[str] = None) -> str:
        path = path or os.path.join(self.dir, f"global_step_{global_step}")
        rank = self.engine.ps.rank
        os.makedirs(os.path.join(path, "extra_state"), exist_ok=True)
        t0 = time.time()
        if self._pending is not None:
            self._pending.result()
            self._pending = None
        sd = self.build_state_dict(include_frozen=not self.lora_only)
        extra = dict(extra_state or {})
        if self.optimizer is not None:
            extra["optimizer_meta"] = self.optimizer.state_dict()
        torch.save(extra, os.path.join(path, "extra_state", f"extra_state_rank_{rank}.pt"))
        from .boxes import BoxSavePlanner
        writer = dcp.FileSystemWriter(path, single_file_per_rank=True, thread_count=1)
        if dist.is_initialized():
            if self.save_async:
                # the shards keep training: the writer thread gets a host snapshot of the pieces
                sd = {k: v.to_host() for k, v in sd.items()}
                self._pending = dcp.async_save(sd, storage_writer=writer, planner=BoxSavePlanner())
            else:
                dcp.save(sd, storage_writer=writer, planner=BoxSavePlanner())
        else:
            dcp.save(sd, storage_writer=writer, planner=BoxSavePlanner(), no_dist=True)
        if rank == 0:
            with open(os.path.join(path, "checkpoint_metadata.json"), "w") as f:
                json.dump({"global_step": global_step, "world_size": self.engine.ps.world_size,
                           "format": "dcp", "keys": len(sd), "saved_at": time.time(),
                           "has_optimizer": self.optimizer is not None}, f, indent=2)
        info_rank0(f"saved checkpoint {path} in {time.time() - t0:.1f}s")
        return path

    # ---- load -----------------------------------------------------------------------------------
    def load(self, path: str, load_optimizer: bool = True, allow_partial_load: bool = False) -> Dict[str, Any]:
        eng = self.engine
        sd = self.build_state_dict()
        allow_partial_load = allow_partial_load or self.lora_only
        if not load_optimizer:
            sd = {k: v for k, v in sd.items() if k.startswith("model.")}
        reader = dcp.FileSystemReader(path)
        if allow_partial_load:
            have = set(reader.read_metadata().state_dict_metadata.keys())
            sd = {k: v for k, v in sd.items() if k in have}
        from .boxes import BoxLoadPlanner
        planner = BoxLoadPlanner(allow_partial_load=allow_partial_load)
        # the pieces are views of the shards: DCP reads every chunk that intersects one straight into it
        if dist.is_initialized():
            dcp.load(sd, storage_reader=reader, planner=planner)
        else:
            dcp.load(sd, storage_reader=reader, planner=planner, no_dist=True)
        from ..ops.fp8_grouped import invalidate_weight_cache
        invalidate_weight_cache()
        for g in eng.all_groups():
            eng.refresh_compute_copy(g)
        extra_path = os.path.join(path, "extra_state", f"extra_state_rank_{eng.ps.rank}.pt")
        if not os.path.exists(extra_path):
            extra_path = os.path.join(path, "extra_state", "extra_state_rank_0.pt")
        extra = torch.load(extra_path, weights_only=False) if os.path.exists(extra_path) else {}
        if load_optimizer and self.optimizer is not None and "optimizer_meta" in extra:
            self.optimizer.load_state_dict(extra["optimizer_meta"])
        return extra

    def wait(self) -> None:
        if self._pending is not None:
            self._pending.result()
            self._pending = None


def build_checkpointer(trainer) -> DistributedCheckpointer:
    t = trainer.args.train
    return DistributedCheckpointer(trainer.engine, trainer.optimizer, t.checkpoint_dir, t.save_async,
                                   lora_only=bool(trainer.args.lora.enable_lora and trainer.args.lora.save_lora_only))
