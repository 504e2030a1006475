"""Per-rank worker of the training service.

``ModelRunner`` owns the same ZeRO engine / optimizer as the CLI trainer and exposes the service
operations: ``forward_backward`` (accumulates un-normalised gradients and the number of valid
tokens of the current gradient epoch), ``optim_step`` (scales by 1/accumulated tokens, clips, steps
with the client's Adam parameters), ``forward`` (log-probs only), ``save_weights`` /
``load_weights``, ``sync_inference_weights``, ``sleep`` / ``wake_up`` and ``abort_gradient_epoch``
(src/xorl/server/runner/model_runner.py:8084-9113).  ``RunnerDispatcher`` is the rank-0 bridge for
multi-rank fleets: rank 0 broadcasts every command over a gloo group, all ranks execute it, and
errors are agreed on with an all-reduce before anybody continues
(src/xorl/server/runner/runner_dispatcher.py:257-395).
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import rl_losses
from ..ops.sampling_transforms import filtered_token_logprobs
from ..ops.loss import fused_linear_token_loss
from .packing import datums_to_micro_batch

OUT_OF_SUPPORT_LOGPROB = -1.0e30     # reported for a label the sampling filter excludes

IGNORE_INDEX = -100


def validate_token_ids(datums: List[Dict[str, Any]], vocab_size: int) -> None:
    """Reject ids outside the vocabulary on the host, before they reach an embedding lookup
    (src/xorl/server/runner/utils/validation.py)."""
    for i, d in enumerate(datums):
        for key in ("tokens", "target_tokens"):
            for t in d.get(key, []):
                if t != IGNORE_INDEX and not (0 <= int(t) < vocab_size):
                    raise ValueError(f"datum {i}: {key} contains id {t} outside [0, {vocab_size})")


class ModelRunner:
    def __init__(self, trainer, max_adapters: Optional[int] = None, moe_metrics: bool = True,
                 sync_bucket_size_mb: Optional[int] = None):
        """``max_adapters``: adapters kept per base model (the active one included; default
        ``XORL_MAX_ADAPTERS_PER_MODEL`` or 8); ``moe_metrics``: expert-load statistics per forward_backward;
        ``sync_bucket_size_mb``: default bucket of a weight sync that names none."""
        self.trainer = trainer
        self.max_adapters = max_adapters
        self.sync_bucket_size_mb = sync_bucket_size_mb
        self.engine = trainer.engine
        self.optimizer = trainer.optimizer
        self.model = trainer.model
        self.device = trainer.device
        self.ps = trainer.ps
        self.accumulated_tokens = 0
        self.epoch_open = False
        self.step = 0
        self.asleep = False
        self.poisoned: Optional[str] = None
        self.output_dir = trainer.args.train.output_dir
        self.adapters = None                 # AdapterManager, created with the first extra adapter
        from .side_payloads import FilesystemPayloadStore, RoutingPayloads
        self.payloads = RoutingPayloads(FilesystemPayloadStore(os.path.join(self.output_dir, "side_payloads")))
        if self.ps.rank == 0:
            self.payloads.store.sweep()          # chunks a crashed predecessor left behind (older than the time-to-live)
        self.host_group = None               # gloo group of all ranks (set by the dispatcher); None: default group
        # expert-load metrics of MoE models: one JSON line per forward_backward in moe_metrics.jsonl
        self.moe_metrics = None
        n_exp = int(getattr(self.model.config, "num_experts", 0) or 0)
        if n_exp > 0 and os.environ.get("XORL_ENABLE_MOE_METRICS", "1") != "0" \
                and moe_metrics and getattr(trainer, "enable_moe_metrics", True):
            from ..utils.moe_metrics import ExpertLoadTracker
            self.moe_metrics = ExpertLoadTracker(n_exp, self.output_dir, self.ps.rank, self.ps.group("dp"))
            self.engine.expert_load_tracker = self.moe_metrics

    # ---- helpers --------------------------------------------------------------------------------
    def _local_batches(self, datums, plan) -> List[Dict[str, Any]]:
        bins = plan[self.ps.dp_rank] if plan else [list(range(len(datums)))]
        out = []
        for b in bins:
            ds = []
            for i in b:
                d = dict(datums[i])
                if self.payloads is not None:
                    d = self.payloads.resolve(d)         # this rank's rows of a routing payload parked beside the command
                d["datum_index"] = i
                ds.append(d)
            out.append(datums_to_micro_batch(ds, pad_to=128))
        return out

    def _loss_closure(self, loss_fn: str, cfg: Dict[str, Any], mb: Dict[str, Any]):
        fn = rl_losses.LOSS_REGISTRY.get(loss_fn)
        if fn is None:
            raise ValueError(f"unknown loss_fn {loss_fn!r}; choose from {sorted(rl_losses.LOSS_REGISTRY)}")
        extras = {k: v.to(self.device) for k, v in mb.items()
                  if torch.is_tensor(v) and v.dtype == torch.float32}
        if "logprobs" in extras and "old_logprobs" not in extras:
            extras["old_logprobs"] = extras.pop("logprobs")
        return lambda lp, mask: fn(lp, mask, **extras, **cfg)

    def _activate(self, model_id: str) -> None:
        if self.adapters is not None:
            self.adapters.activate(model_id)
        elif model_id != "default":
            raise KeyError(f"unknown model_id {model_id!r}")

    def create_model(self, model_id, base_model=None, lora_config=None, **_):
        """Registers a new named adapter (needs LoRA; the base weights are shared and frozen)."""
        if not self.trainer.args.lora.enable_lora:
            raise ValueError("create_model needs a server started with enable_lora")
        if self.adapters is None:
            from .adapters import AdapterManager
            self.adapters = AdapterManager(self, max_adapters=self.max_adapters,
                                           spill_dir=os.path.join(self.output_dir, "adapter_spill"))
        self.adapters.create(model_id, lora_config)
        return {"model_id": model_id, "adapters": self.adapters.list(),
                "session": self.adapters.session_spec(model_id)}

    def unload_model(self, model_id, **_):
        if self.adapters is not None:
            self.adapters.unload(model_id)
        return {"model_id": model_id}

    def _replay_extra(self, mb) -> Optional[Dict[str, Any]]:
        """Rollout routing replay: ``routed_experts`` [T, moe_layers, k] recorded by the inference
        engine forces the same expert choices in training (src/xorl/server/runner/utils/
        routing_replay_handler.py).  Padding tokens carry -1 and keep the router's own choice."""
        r = mb.get("routed_experts")
        if r is None:
            return None
        return {"routing_replay_all": r.to(self.device).long()}

    def _gather_per_datum(self, local: Dict[int, Any]) -> Dict[int, Any]:
        """Per-datum outputs live on the data-parallel rank that ran the datum; the caller (rank 0)
        needs all of them.  Ranks that hold the same datum (tensor / context / pipeline peers) carry
        identical values."""
        if self.ps.world_size == 1 or not dist.is_initialized():
            return local
        parts: List[Optional[Dict[int, Any]]] = [None] * dist.get_world_size(self.host_group)
        dist.all_gather_object(parts, local, group=self.host_group)
        merged: Dict[int, Any] = {}
        for part in parts:
            merged.update(part or {})
        return merged

    def _check_usable(self) -> None:
        if self.poisoned:
            raise RuntimeError(f"runner is poisoned after a failed mutation: {self.poisoned}")
        if self.asleep:
            raise RuntimeError("runner is asleep; call wake_up first")

    def preflight(self, op: str, args: Dict[str, Any]) -> None:
        """Host-only checks that may fail on one rank and not on another.  They run, and their
        outcome is agreed on by all ranks, before any rank enters the collectives of ``op``."""
        if op in ("sleep", "wake_up", "abort_gradient_epoch", "unload_model"):
            return
        if op == "create_model":
            if not self.trainer.args.lora.enable_lora:
                raise ValueError("create_model needs a server started with enable_lora")
            return
        self._check_usable()
        if op in ("forward_backward", "forward"):
            validate_token_ids(args.get("datums", []), self.model.config.vocab_size)
            if args.get("loss_fn", "cross_entropy") not in rl_losses.LOSS_REGISTRY:
                raise ValueError(f"unknown loss_fn {args.get('loss_fn')!r}")
        elif op == "optim_step" and not self.epoch_open:
            raise RuntimeError("optim_step without a preceding forward_backward")
        elif op == "load_weights":
            if not os.path.isdir(self._weights_path(args.get("model_id", "default"), args["path"])):
                raise ValueError(f"no saved weights at {args['path']}")

    # ---- operations -------------------------------------------------------------------------------
    def forward_backward(self, model_id, datums, plan, loss_fn="cross_entropy", loss_fn_config=None):
        self._check_usable()
        self._activate(model_id)
        validate_token_ids(datums, self.model.config.vocab_size)
        cfg = dict(loss_fn_config or {})
        if not self.epoch_open:
            self.optimizer.zero_grad()
            self.epoch_open = True
            self.accumulated_tokens = 0
        logprobs: Dict[int, List[float]] = {}
        total = 0.0
        eng = self.engine
        t_start = time.time()
        if self.trainer.pp_runner is not None:
            return self._forward_backward_pp(datums, plan, loss_fn, cfg, t_start)
        for mb in self._local_batches(datums, plan):
            d = {k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in mb.items()}
            self.accumulated_tokens += mb["num_valid_tokens"]
            closure = self._loss_closure(loss_fn, cfg, mb)
            holder = {}

            def head(h, res, labels, ctx, grad_scale, _c=closure, _h=holder):
                hidden = self.model.forward_head(h, res, ctx)
                loss, lp, metrics = fused_linear_token_loss(hidden, self.model.lm_head.weight, labels,
                                                            _c, grad_scale, self.model.loss_chunk_tokens)
                _h["lp"], _h["metrics"] = lp, metrics
                return loss

            orig = self.model.head_loss
            self.model.head_loss = head
            try:
                loss = eng.forward_backward(d["input_ids"], d["labels"], position_ids=d["position_ids"],
                                            cu_seqlens=d["cu_seqlens"], grad_scale=1.0,
                                            extra=self._replay_extra(mb))
            finally:
                self.model.head_loss = orig
            total += float(loss)
            lp = holder["lp"].float().cpu()
            for idx, (s, e) in zip(mb["datum_index"], mb["datum_spans"]):
                logprobs[idx] = lp[s:e].tolist()
        if self.ps.world_size > 1 and self.ps.group("dp") is not None:
            t = torch.tensor([total, float(self.accumulated_tokens)], device=self.device)
            dist.all_reduce(t, group=self.ps.group("dp"))
            total = float(t[0])
        logprobs = self._gather_per_datum(logprobs)
        metrics = {"loss:sum": total}
        if self.moe_metrics is not None:
            m = self.moe_metrics.collect(self.step, time.time() - t_start)
            self.moe_metrics.write(m)
            if "expert_load" in m:
                metrics["moe/mean_imbalance_ratio"] = m["expert_load"]["mean_imbalance_ratio"]
                metrics["moe/max_imbalance_ratio"] = m["expert_load"]["max_imbalance_ratio"]
        return {"loss": total, "num_tokens": sum(len(d["tokens"]) for d in datums),
                "logprobs": [logprobs.get(i, []) for i in range(len(datums))],
                "metrics": metrics}

    # ---- pipeline parallelism -------------------------------------------------------------------
    def _pp_runner_for(self, n_mb: int):
        """The trainer's pipeline runner re-planned for ``n_mb`` micro-batches (a request brings as many
        as its datums pack into); process groups and stage layout are shared."""
        base = self.trainer.pp_runner
        if n_mb == base.n_mb:
            return base
        cache = self.__dict__.setdefault("_pp_runners", {})
        if n_mb not in cache:
            import copy
            from ..parallel import pp_schedules as S
            r = copy.copy(base)
            r.n_mb = n_mb
            r.actions = S.build_schedule(r.schedule, r.pp, n_mb, r.virtual_stages)
            S.simulate(r.actions, r.schedule, r.pp, n_mb, r.virtual_stages)
            r._send_order = r._message_orders()
            r.bubble_stats = {}
            cache[n_mb] = r
        return cache[n_mb]

    def _forward_backward_pp(self, datums, plan, loss_fn, cfg, t_start, zero_loss: bool = False):
        """One pipelined pass over this rank's micro-batches (src/xorl/server/runner/model_runner.py
        ``_forward_backward_pp``): the last stage evaluates the token loss of every micro-batch as its
        activations arrive and keeps the per-token log-probabilities; loss and log-probabilities reach
        the caller through the reductions below.  The micro-batch count is padded with label-free
        batches to a multiple of the pipeline size, which every schedule accepts."""
        pp = self.ps.pp_size
        batches = self._local_batches(datums, plan)
        while len(batches) % pp or not batches:
            batches.append(datums_to_micro_batch([], pad_to=128))
        dev = [{k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in mb.items()} for mb in batches]
        slot = {id(d["labels"]): i for i, d in enumerate(dev)}
        closures = [self._loss_closure(loss_fn, cfg, mb) for mb in batches]
        lps: Dict[int, torch.Tensor] = {}

        def head(h, res, labels, ctx, grad_scale):
            i = slot[id(labels)]
            hidden = self.model.forward_head(h, res, ctx)
            fn = (lambda lp, mask: (lp.sum() * 0, {})) if zero_loss else closures[i]
            loss, lp, _ = fused_linear_token_loss(hidden, self.model.lm_head.weight, labels, fn, grad_scale,
                                                  self.model.loss_chunk_tokens)
            lps[i] = lp
            return loss

        orig = self.model.head_loss
        self.model.head_loss = head
        try:
            total_t = self._pp_runner_for(len(dev)).run(dev, 1.0)
        finally:
            self.model.head_loss = orig
        logprobs: Dict[int, List[float]] = {}
        for i, lp in lps.items():
            lp = lp.float().cpu()
            for idx, (s, e) in zip(batches[i]["datum_index"], batches[i]["datum_spans"]):
                logprobs[idx] = lp[s:e].tolist()
        if not zero_loss:
            self.accumulated_tokens += sum(mb["num_valid_tokens"] for mb in batches)
        t = torch.tensor([float(total_t)], device=self.device)
        if self.ps.group("dp") is not None:    # the pipeline runner already shares the loss over the stages
            dist.all_reduce(t, group=self.ps.group("dp"))
        total = float(t[0])
        logprobs = self._gather_per_datum(logprobs)
        return {"loss": total, "num_tokens": sum(len(d["tokens"]) for d in datums),
                "logprobs": [logprobs.get(i, []) for i in range(len(datums))],
                "metrics": {"loss:sum": total}}

    @torch.no_grad()
    def forward(self, model_id, datums, plan, loss_fn="cross_entropy", loss_fn_config=None):
        self._check_usable()
        self._activate(model_id)
        validate_token_ids(datums, self.model.config.vocab_size)
        logprobs: Dict[int, List[float]] = {}
        cfg = loss_fn_config or {}
        filt = {k: cfg[k] for k in ("top_k", "top_p", "min_p") if cfg.get(k) is not None}
        temperature = float(cfg.get("temperature", 1.0))
        outside = 0
        if self.trainer.pp_runner is not None:
            if filt or temperature != 1.0:
                raise NotImplementedError("filtered / tempered log-probabilities are not available under pipeline parallelism")
            # the pipelined pass with a zero loss: log-probabilities come out of the last stage, the
            # backward half of the schedule adds exact zeros to the gradient accumulators
            with torch.enable_grad():
                out = self._forward_backward_pp(datums, plan, loss_fn, dict(cfg), time.time(), zero_loss=True)
            return {"logprobs": out["logprobs"], "metrics": {}}
        if cfg.get("reference"):
            # reference-policy pass: log-probabilities of the frozen base model, adapters bypassed
            from ..adapters.lora import adapters_disabled
            with adapters_disabled(self.model) as n:
                if n == 0:
                    raise ValueError("a reference pass needs LoRA adapters over a frozen base model")
                return self.forward(model_id, datums, plan, loss_fn, {k: v for k, v in cfg.items() if k != "reference"})
        for mb in self._local_batches(datums, plan):
            d = {k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in mb.items()}
            hidden = self.engine.forward_only(d["input_ids"], position_ids=d["position_ids"],
                                              cu_seqlens=d["cu_seqlens"])
            root, _ = self.engine._units_by_role()
            self.engine.gather(root)
            self.engine.wait_gather(root)
            if filt or temperature != 1.0:
                # the sampler drew from a filtered distribution: report the log-probability on the
                # same support (ops/sampling_transforms.py)
                lp, ok = filtered_token_logprobs(hidden, self.model.lm_head.weight, d["labels"],
                                                 temperature=temperature, **filt)
                outside += int((~ok).sum())
                lp = lp.clamp_min(OUT_OF_SUPPORT_LOGPROB)       # JSON has no -inf
            else:
                _, lp, _ = fused_linear_token_loss(hidden, self.model.lm_head.weight, d["labels"],
                                                   lambda lp, mask: (lp.sum() * 0, {}), 1.0)
            lp = lp.float().cpu()
            for idx, (s, e) in zip(mb["datum_index"], mb["datum_spans"]):
                logprobs[idx] = lp[s:e].tolist()
        metrics = {"out_of_support_tokens": outside} if (filt or temperature != 1.0) else {}
        logprobs = self._gather_per_datum(logprobs)
        return {"logprobs": [logprobs.get(i, []) for i in range(len(datums))], "metrics": metrics}

    def optim_step(self, model_id, adam_params=None, gradient_clip=None, **_):
        self._check_usable()
        self._activate(model_id)
        if not self.epoch_open:
            raise RuntimeError("optim_step without a preceding forward_backward")
        ap = adam_params or {}
        tokens = self.accumulated_tokens
        if self.ps.world_size > 1 and self.ps.group("dp_sp") is not None:
            t = torch.tensor([float(tokens)], device=self.device)
            dist.all_reduce(t, group=self.ps.group("dp_sp"))
            tokens = int(t.item())
        self.engine.finish_grad_sync()
        scale = 1.0 / max(1, tokens)
        opt = self.optimizer
        opt.set_lr(float(ap.get("learning_rate", opt.lr)))
        if hasattr(opt, "betas"):
            opt.betas = (float(ap.get("beta1", opt.betas[0])), float(ap.get("beta2", opt.betas[1])))
            opt.eps = float(ap.get("eps", opt.eps))
        norm, coef = self.engine.grad_norm_and_clip_coef(0.0)
        norm_scaled = norm * scale
        clip = float(gradient_clip) if gradient_clip else 0.0
        if clip > 0:
            coef = torch.clamp(clip / (norm_scaled + 1e-6), max=1.0)
        opt.step(clip_coef=coef if clip > 0 else None, grad_scale=scale)
        self.epoch_open = False
        self.step += 1
        if self.adapters is not None:
            self.adapters.validate_replica_coherence()
        return {"metrics": {"grad_norm": float(norm_scaled), "step": float(self.step),
                            "learning_rate": opt.lr, "tokens": float(tokens)}}

    def abort_gradient_epoch(self, model_id="default"):
        self._activate(model_id)
        self.optimizer.zero_grad()
        self.epoch_open = False
        self.accumulated_tokens = 0
        return {"aborted": True}

    def _weights_path(self, model_id: str, path: str) -> str:
        """``xorl://{model}/{weights|sampler_weights}/{name}``, a bare name, or a path: all resolve
        below the server's output directory (or ``XORL_SERVER_ARTIFACT_ROOT`` when a path lies
        elsewhere); symlinked components and ``..`` escapes are refused."""
        from .security import ARTIFACT_ROOT_ENV, confine_path, validate_identifier
        if path.startswith("xorl://"):
            parts = path[len("xorl://"):].split("/")
            if len(parts) != 3 or parts[1] not in ("weights", "sampler_weights"):
                raise ValueError(f"malformed weights URI {path!r}")
            mid, kind, name = (validate_identifier(x, "weights URI component") for x in parts)
            return os.path.join(self.output_dir, kind, mid, name)
        if os.path.isabs(path) or os.sep in path:
            try:
                return str(confine_path(self.output_dir, path))
            except ValueError:
                root = os.environ.get(ARTIFACT_ROOT_ENV, "").strip()
                if not root:
                    raise
                return str(confine_path(root, path))
        return os.path.join(self.output_dir, "weights", validate_identifier(model_id, "model_id"),
                            validate_identifier(path, "checkpoint name"))

    def save_weights(self, model_id, path=None, **_):
        self._activate(model_id)
        name = path or f"step_{self.step:06d}"
        out = self._weights_path(model_id, name)
        self.trainer.checkpointer.save(self.step, {"global_step": self.step, "runner_step": self.step}, path=out)
        self.trainer.checkpointer.wait()
        uri = name if name.startswith("xorl://") or os.sep in name else f"xorl://{model_id}/weights/{name}"
        return {"path": uri, "directory": out}

    def load_weights(self, model_id, path, load_optimizer=True, **_):
        self._activate(model_id)
        p = self._weights_path(model_id, path)
        if not os.path.isdir(p):
            raise ValueError(f"no saved weights at {path}")
        try:
            extra = self.trainer.checkpointer.load(p, load_optimizer=load_optimizer)
        except Exception as e:  # noqa: BLE001
            # shards may be half overwritten: refuse further work instead of training on them
            self.poisoned = f"load_weights({path}) failed midway: {e}"
            raise
        self.step = int((extra or {}).get("runner_step", self.step))
        self.abort_gradient_epoch(model_id)
        return {"path": path}

    def save_sampler_weights(self, model_id, name, quantization=None, merged: bool = False, **_):
        """Weights an inference engine can load, under ``sampler_weights/{name}``: for a LoRA session its
        adapter alone as a PEFT directory at the session's own rank (the base model is unchanged, engines
        hot-load adapters), otherwise -- or with ``merged`` -- full Hugging Face weights (adapter folded
        in) (src/xorl/server/api_server/weights.py:700-760)."""
        from .security import validate_identifier
        d = os.path.join(self.output_dir, "sampler_weights", validate_identifier(name, "sampler weights name"))
        if os.path.exists(d):
            raise ValueError(f"sampler weights {name!r} exist already; use another name or delete them first")
        self._activate(model_id)
        if self.trainer.args.lora.enable_lora and not merged:
            from ..adapters.lora import save_lora_checkpoint
            spec = self.adapters.session_spec(model_id) if self.adapters is not None else {}
            save_lora_checkpoint(self.engine, d, self.trainer.args.model.model_path or "",
                                 rank=spec.get("rank"), alpha=spec.get("alpha"))
            if dist.is_initialized():
                dist.barrier(group=self.host_group) if getattr(self, "host_group", None) is not None else dist.barrier()
            return {"directory": d, "kind": "lora_adapter", "lora_path": d}
        out = self.sync_inference_weights(model_id, backend="file", directory=d, quantization=quantization)
        return {**out, "directory": d, "kind": "full_weights"}

    def sync_inference_weights(self, model_id, **kw):
        from .weight_sync import WeightSyncHandler
        handler = getattr(self, "_sync", None) or WeightSyncHandler(self)
        self._sync = handler
        if not kw.get("bucket_size_mb"):
            kw["bucket_size_mb"] = int(self.sync_bucket_size_mb or 1024)
        return handler.sync(**kw)

    def sleep(self):
        """Release device memory that can be rebuilt (buffer pools) and refuse work until woken."""
        self.engine._full_pool.clear()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        self.asleep = True
        return {"asleep": True}

    def wake_up(self):
        self.asleep = False
        return {"asleep": False}


class RunnerDispatcher:
    """Rank 0 receives commands and broadcasts them to all ranks over a gloo group; after every
    command the ranks agree on success (all-reduce MAX of an error flag, then gather of messages)."""

    def __init__(self, runner: ModelRunner, cpu_group=None):
        self.runner = runner
        self.cpu_group = cpu_group
        runner.host_group = cpu_group
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1

    def execute(self, command: Optional[Dict[str, Any]]) -> Dict[str, Any]:
        """Called on every rank; only rank 0 passes a command."""
        box = [command]
        if self.world > 1:
            dist.broadcast_object_list(box, src=0, group=self.cpu_group)
        cmd = box[0]
        if cmd is None or cmd.get("op") == "shutdown":
            return {"shutdown": True}
        op, args = cmd["op"], cmd.get("args", {})
        err = None
        try:
            self.runner.preflight(op, args)
        except Exception as e:  # noqa: BLE001
            err = f"rank {self.rank}: {type(e).__name__}: {e}"
        out = self._sync_error_state(err, None)
        if "error" in out:
            return out
        err, result = None, None
        try:
            fn = getattr(self.runner, op)
            result = fn(**args) if op in ("sleep", "wake_up") else fn(cmd.get("model_id", "default"), **args)
        except Exception as e:  # noqa: BLE001
            err = f"rank {self.rank}: {type(e).__name__}: {e}"
        return self._sync_error_state(err, result)

    def _sync_error_state(self, err: Optional[str], result):
        if self.world > 1:
            flag = torch.tensor([1 if err else 0])
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.cpu_group)
            if int(flag.item()):
                msgs: List[Optional[str]] = [None] * self.world
                dist.all_gather_object(msgs, err, group=self.cpu_group)
                return {"error": "; ".join(m for m in msgs if m)}
            return {"result": result}
        return {"error": err} if err else {"result": result}

    def worker_loop(self) -> None:
        while True:
            out = self.execute(None)
            if out.get("shutdown"):
                return
