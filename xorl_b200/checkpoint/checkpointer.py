"""DCP save / load of the ZeRO engine's state.

Directory layout ``{output_dir}/checkpoints/global_step_{N}/`` with ``.metadata``,
``__{rank}_0.distcp``, ``extra_state/extra_state_rank_{r}.pt`` and ``checkpoint_metadata.json``;
state keys ``model.<fqn>`` and ``optimizer.state.<fqn>.{exp_avg,exp_avg_sq}`` — the layout of
src/xorl/checkpoint/checkpointer.py:795-1072.  The engine's flat shards are re-expressed as
per-parameter ``Shard(0)`` DTensors over the shard group, so a checkpoint written at one world
size loads at another (DCP reshards), and one written by a single process is a plain-tensor
checkpoint that sharded runs can read.
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


def _chunk_bounds(dim0: int, world: int, rank: int):
    per = -(-dim0 // world)
    a = min(dim0, rank * per)
    return a, min(dim0, a + per)


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

    # ---- DTensor views ------------------------------------------------------------------------
    def _mesh_for(self, g):
        from torch.distributed.device_mesh import DeviceMesh
        key = id(g.pg)
        if key not in self._meshes:
            ranks = dist.get_process_group_ranks(g.pg)
            self._meshes[key] = DeviceMesh.from_group(g.pg, self.engine.device.type, mesh=ranks)
        return self._meshes[key]

    def _wrap(self, g, shape, full_view: torch.Tensor):
        """Local Shard(0) chunk of one full parameter as a DTensor (plain tensor when world==1)."""
        if g.world == 1 or g.pg is None:
            return full_view  # a view of the shard itself: saved from / loaded into in place
        from torch.distributed.tensor import DTensor, Shard
        t = full_view if full_view.dim() > 0 else full_view.reshape(1)
        a, b = _chunk_bounds(t.shape[0], g.world, g.rank)
        local = t[a:b].clone()
        stride = torch.empty(t.shape, device="meta").stride()
        return DTensor.from_local(local, self._mesh_for(g), [Shard(0)], run_check=False,
                                  shape=t.shape, stride=stride)

    def _ep_mesh(self):
        """(ep, ep_fsdp) device mesh of this rank's expert-parallel grid (1-D over ep when every
        rank of a stage is its own ep_fsdp group)."""
        if "ep" in self._meshes:
            return self._meshes["ep"]
        from torch.distributed.device_mesh import DeviceMesh
        ps = self.engine.ps
        ep_ranks, epf_ranks = ps.group_ranks("ep"), ps.group_ranks("ep_fsdp")
        dev = self.engine.device.type
        if len(epf_ranks) == 1:
            mesh = DeviceMesh.from_group(ps.group("ep"), dev, mesh=ep_ranks, mesh_dim_names=("ep",))
        else:
            # the expert grid is a reshape of consecutive ranks, hence affine in both coordinates
            grid = [[e + f - ps.rank for f in epf_ranks] for e in ep_ranks]
            assert grid[ps.rank_in("ep")][ps.rank_in("ep_fsdp")] == ps.rank
            mesh = DeviceMesh.from_group([ps.group("ep"), ps.group("ep_fsdp")], dev,
                                         mesh=torch.tensor(grid), mesh_dim_names=("ep", "ep_fsdp"))
        self._meshes["ep"] = mesh
        return mesh

    def _wrap_expert(self, p, local_view: torch.Tensor):
        """Expert-parallel parameter: this rank's experts ``[E / ep, d1, ...]`` (already gathered over
        ep_fsdp) as a DTensor of the full ``[E, d1, ...]`` shape, ``Shard(0)`` over ep and
        ``Shard(1)`` over ep_fsdp -- the placement the reference restores for expert tensors
        (src/xorl/checkpoint/checkpointer.py:107-160)."""
        from torch.distributed.tensor import DTensor, Shard
        ps = self.engine.ps
        full_shape = tuple(p._xb_full_shape)
        stride = torch.empty(full_shape, device="meta").stride()
        mesh = self._ep_mesh()
        if mesh.ndim == 1:
            return DTensor.from_local(local_view.clone(), mesh, [Shard(0)], run_check=False,
                                      shape=full_shape, stride=stride)
        a, b = _chunk_bounds(full_shape[1], ps.ep_fsdp_size, ps.rank_in("ep_fsdp"))
        return DTensor.from_local(local_view[:, a:b].clone(), mesh, [Shard(0), Shard(1)], run_check=False,
                                  shape=full_shape, stride=stride)

    def _state_sources(self):
        srcs = [("model", "master", None)]
        opt = self.optimizer
        if opt is not None:
            for sname, per_group in opt.state.items():
                srcs.append((f"optimizer.state.{{fqn}}.{sname}", "extra", per_group))
        return srcs

    def build_state_dict(self, include_frozen: bool = True) -> Dict[str, Any]:
        sd: Dict[str, Any] = {}
        eng = self.engine
        group_of = {name: g for g in eng.all_groups() for name, _ in g.named_params}
        param_of = {name: p for g in eng.all_groups() for name, p in g.named_params}
        for key_fmt, what, extra in self._state_sources():
            for name, view in eng.iter_full_tensors(what, extra, ep_full=False):
                g = group_of[name]
                if getattr(g, "frozen", False) and not include_frozen:
                    continue
                fqn = to_checkpoint_fqn(name)
                key = f"model.{fqn}" if key_fmt == "model" else key_fmt.format(fqn=fqn)
                val = view.float() if what != "master" else view
                if getattr(param_of[name], "_xb_ep", None) is not None and eng.ps.ep_size > 1:
                    sd[key] = self._wrap_expert(param_of[name], val)
                else:
                    sd[key] = self._wrap(g, view.shape, val)
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
        writer = dcp.FileSystemWriter(path, single_file_per_rank=True, thread_count=1)
        if dist.is_initialized():
            if self.save_async:
                self._pending = dcp.async_save(sd, storage_writer=writer)
            else:
                dcp.save(sd, storage_writer=writer)
        else:
            dcp.save(sd, storage_writer=writer, no_dist=True)
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
        if dist.is_initialized():
            dcp.load(sd, storage_reader=reader)
        else:
            dcp.load(sd, storage_reader=reader, no_dist=True)
        # scatter the loaded per-parameter chunks back into the flat shards
        def full_of(v):
            return v.full_tensor() if hasattr(v, "full_tensor") else v
        model_full: Dict[str, torch.Tensor] = {}
        for g in eng.all_groups():
            tensors = {}
            for (name, _), shape in zip(g.named_params, g.shapes):
                key = f"model.{to_checkpoint_fqn(name)}"
                if key in sd:
                    tensors[name] = full_of(sd[key])
            if tensors:
                eng.load_full_tensors(tensors, strict=False)
        if load_optimizer and self.optimizer is not None:
            for sname, per_group in self.optimizer.state.items():
                for g in eng.all_groups():
                    tensors = {}
                    for (name, _), shape in zip(g.named_params, g.shapes):
                        key = f"optimizer.state.{to_checkpoint_fqn(name)}.{sname}"
                        if key in sd:
                            tensors[name] = full_of(sd[key])
                    if tensors:
                        eng.load_full_tensors(tensors, strict=False, target="extra", extra=per_group)
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
