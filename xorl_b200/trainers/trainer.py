"""Training loop shared by the CLI and the server runner.

Phases follow the reference trainer (src/xorl/trainers/trainer.py:340-376 start-up, :1369-1499
loop, :1743-1880 step): bootstrap process groups -> build model on the meta device -> ZeRO engine
materialises and shards it -> data -> optimizer / LR schedule -> resume -> loop.  A step is:
count valid tokens (all-reduce over dp x sp) -> forward/backward over the micro-batches with
losses pre-scaled by 1/global_tokens -> finish gradient reduction -> global-norm clip coefficient
on the device -> fused optimizer step -> LR step.  Artifacts: ``xorl_cli.yaml``,
``startup_metrics.json``, ``training_metrics.json``, ``checkpoints/global_step_N``.
"""
from __future__ import annotations

import gc
import json
import os
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..arguments import Arguments, save_args
from ..data import build_dataloader, prepare_datasets
from ..models import build_model_config, build_model
from ..optim import build_lr_scheduler, build_optimizer
from ..parallel.dist_utils import synchronize_micro_batch_padding
from ..parallel.state import get_parallel_state, init_parallel_state, process_group_timeout
from ..parallel.zero import Zero3Engine
from ..utils.diagnostics import nvtx_range
from ..utils.helper import CudaTimer, EnvironMeter, create_profiler, set_seed
from ..utils.logging import get_logger, info_rank0

logger = get_logger(__name__)
IGNORE_INDEX = -100


def resolve_device(pref: str = "auto") -> torch.device:
    if pref == "cpu" or (pref == "auto" and not torch.cuda.is_available()):
        return torch.device("cpu")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    return torch.device("cuda", local)


class Trainer:
    def __init__(self, args: Arguments, dataset=None, model_config=None):
        self.args = args
        self.startup: Dict[str, float] = {}
        self.global_step = 0
        self.loss_history: List[float] = []
        self.metrics_history: List[Dict[str, float]] = []
        self._timed("bootstrap", self._bootstrap)
        self._timed("build_model", lambda: self._build_model(model_config))
        self._timed("build_data", lambda: self._build_data(dataset))
        self._timed("build_optimizer", self._build_optimizer)
        self._timed("observability", self._setup_observability)
        if args.train.enable_qarl and args.train.qarl_calib_data:
            self._timed("qarl_calibration", self._qarl_calibration)
        self._timed("resume", self._resume_checkpoint)
        head_rows = [p.shape[0] for n, p in self.model.named_parameters() if n.endswith("lm_head.weight")]
        self.startup["lm_head_rows_per_rank"] = head_rows[0] if head_rows else 0
        if self.ps.rank == 0:
            os.makedirs(args.train.output_dir, exist_ok=True)
            with open(os.path.join(args.train.output_dir, "startup_metrics.json"), "w") as f:
                json.dump(self.startup, f, indent=2)

    def _timed(self, name, fn):
        t0 = time.perf_counter()
        fn()
        self.startup[name + "_s"] = time.perf_counter() - t0

    # ------------------------------------------------------------------------------------------
    def _bootstrap(self) -> None:
        t = self.args.train
        self.device = resolve_device(t.device)
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1 and not dist.is_initialized():
            backend = "nccl" if self.device.type == "cuda" else "gloo"
            kw = {"device_id": self.device} if backend == "nccl" else {}
            dist.init_process_group(backend, timeout=process_group_timeout(), **kw)
        set_seed(t.seed, t.enable_full_determinism)
        lm_head_tp = t.lm_head_tensor_parallel_size
        if t.fsdp_sharded_lm_head_loss and lm_head_tp == 1 and t.tensor_parallel_size == 1:
            # the lm-head is never gathered: every rank of the data-parallel group keeps V / dp vocabulary
            # rows and the loss streams the group's tokens through them (src/xorl/arguments.py:1464-1483)
            lm_head_tp = max(1, world // max(1, t.pipeline_parallel_size * t.ulysses_parallel_size
                                             * t.ringattn_parallel_size))
        self.ps = init_parallel_state(
            dp_replicate_size=t.data_parallel_replicate_size, dp_shard_size=t.data_parallel_shard_size,
            tp_size=t.tensor_parallel_size, ep_size=t.expert_parallel_size,
            pp_size=t.pipeline_parallel_size, ulysses_size=t.ulysses_parallel_size,
            ringattn_size=t.ringattn_parallel_size, lm_head_tp_size=lm_head_tp,
            dp_mode=t.data_parallel_mode, cp_fsdp_mode=t.cp_fsdp_mode, device_type=self.device.type,
            ep_intranode=t.ep_intranode, tp_sequence_parallel=t.tensor_parallel_sequence_parallel)
        if self.ps.rank == 0:
            save_args(self.args, t.output_dir)
        self.compute_dtype = torch.bfloat16 if (t.enable_mixed_precision and self.device.type == "cuda") \
            else torch.float32

    def _build_model(self, model_config=None) -> None:
        a, t = self.args, self.args.train
        self.model_config = model_config or build_model_config(a.model)
        stage_kw = {}
        self.pp_layout = None
        if self.ps.pp_size > 1:
            from ..parallel.pp import local_stage_layout
            if self.model_config.tie_word_embeddings:
                raise ValueError("pipeline parallelism does not support tied embeddings")
            self.pp_layout = local_stage_layout(
                self.model_config.num_hidden_layers, self.ps, t.pipeline_parallel_schedule,
                t.pipeline_parallel_virtual_stages, input_weight=t.pipeline_parallel_input_weight,
                output_weight=t.pipeline_parallel_output_weight,
                first=t.pipeline_parallel_num_layers_in_first_stage,
                last=t.pipeline_parallel_num_layers_in_last_stage)
            stage_kw = dict(layer_indices=self.pp_layout["layers"],
                            has_embed=self.pp_layout["has_embed"], has_head=self.pp_layout["has_head"])
        self.model = build_model(self.model_config, a, device="meta", **stage_kw)
        if t.ce_num_chunks and t.ce_num_chunks > 0:
            self.model.loss_chunk_tokens = max(256, -(-int(a.data.sample_packing_sequence_len or 4096)
                                                      * t.micro_batch_size // t.ce_num_chunks))
        if t.fsdp_sharded_lm_head_loss and getattr(self.ps, "lm_head_tp_size", 1) > 1:
            # tokens of the whole group per chunk of the streamed loss
            local = int(a.data.sample_packing_sequence_len or 4096) * t.micro_batch_size
            self.model.loss_chunk_tokens = max(64, -(-local // max(1, t.fsdp_sharded_lm_head_loss_num_chunks))
                                               * self.ps.lm_head_tp_size)
        if self.model_config.is_moe:
            # model.train_router: whether the gradient of the expert outputs flows into the routing
            # weights (off by default: the router then learns from the load-balancing loss only);
            # model.freeze_router: the router weights do not train at all
            for m in self.model.modules():
                if hasattr(m, "train_router"):
                    m.train_router = bool(a.model.train_router)
                    if a.model.freeze_router:
                        for prm in m.gate.parameters():
                            prm.requires_grad_(False)
            self.model.ctx_defaults["ep_dispatch"] = a.model.ep_dispatch
            # every EP rank must size its peer-memory workspace identically
            self.model.ctx_defaults["ep_max_slots"] = int(a.data.sample_packing_sequence_len or 4096) \
                * t.micro_batch_size * self.model_config.num_experts_per_tok
            # the load-balancing loss of the routers is weighted by the model's own
            # router_aux_loss_coef (src/xorl/trainers/trainer.py:2081-2091)
            coef = float(self.model_config.router_aux_loss_coef or 0.0)
            if coef > 0:
                for m in self.model.modules():
                    if hasattr(m, "aux_coef"):
                        m.aux_coef = coef
                self.model.aux_loss_enabled = True
                if t.moe_global_load_balancing:
                    self.model.ctx_defaults["aux_global_group"] = self.ps.group("dp")
        if t.softmax_auxiliary_loss:
            # z-loss on the lm-head logits: auxiliary_loss_multiplier * logsumexp(logits)^2 per
            # supervised token (src/xorl/trainers/trainer.py:481-487)
            if t.pipeline_parallel_size > 1:
                raise NotImplementedError("softmax_auxiliary_loss (z-loss) is not supported with "
                                          "pipeline parallelism")
            self.model.z_loss_coef = float(t.auxiliary_loss_multiplier)
        from ..parallel.cp import attach_cp_strategy
        attach_cp_strategy(self.model, self.ps)
        recompute = t.enable_gradient_checkpointing and t.gradient_checkpointing_method != "no_recompute"
        self.engine = Zero3Engine(
            self.model, self.ps, compute_dtype=self.compute_dtype, device=self.device,
            reduce_dtype=torch.float32 if t.fsdp_reduce_dtype == "fp32" else torch.bfloat16,
            activation_offload=t.enable_activation_offload,
            reshard_after_forward=True if t.reshard_after_forward is None else t.reshard_after_forward,
            recompute=recompute, seed=t.seed, comm_backend=t.comm_backend,
            forward_prefetch=bool(t.enable_forward_prefetch),
            backward_prefetch=True if t.enable_backward_prefetch is None else bool(t.enable_backward_prefetch),
            moe_grad_reduce_mode=t.moe_grad_reduce_mode)
        if t.comm_backend in ("auto", "fused") and self.device.type == "cuda" and self.ps.world_size > 1:
            self.engine.attach_peer_transport(required=(t.comm_backend == "fused"))
        self.teacher_engine = None
        if a.distill.enable_distillation:
            self._build_teacher()
        self.pp_runner = None
        if self.pp_layout is not None:
            from ..parallel.pp import PipelineRunner
            self.pp_runner = PipelineRunner(self.engine, self.ps, t.pipeline_parallel_schedule,
                                            t.pipeline_parallel_virtual_stages, self.pp_layout,
                                            t.gradient_accumulation_steps)
        weights = a.model.model_path
        if weights and t.load_weights_mode != "skip" and os.path.isdir(weights) and any(
                f.endswith(".safetensors") for f in os.listdir(weights)):
            from ..checkpoint.hf_io import load_hf_weights
            load_hf_weights(self.engine, weights, self.model_config, mode=t.load_weights_mode)

    def _build_teacher(self) -> None:
        """``distill.enable_distillation``: a frozen teacher of the family named by
        ``distill.teacher_model_path`` (a directory with config.json and, optionally, safetensors
        weights, or a preset name) runs a forward pass over every micro-batch; its final hidden states
        and lm-head give the target distribution of the KL term in the head loss."""
        a, d = self.args, self.args.distill
        if not d.teacher_model_path:
            raise ValueError("distill.enable_distillation needs distill.teacher_model_path")
        if self.pp_layout is not None or self.ps.tp_size > 1:
            raise NotImplementedError("distillation is not supported with pipeline or tensor parallelism")
        from ..models.config import ModelConfig, preset
        path = d.teacher_model_path
        tcfg = ModelConfig.from_pretrained(path) if os.path.isdir(path) else preset(path)
        if tcfg.vocab_size != self.model_config.vocab_size:
            raise ValueError(f"teacher vocabulary {tcfg.vocab_size} != student vocabulary {self.model_config.vocab_size}")
        teacher = build_model(tcfg, None, device="meta")
        for p in teacher.parameters():
            p.requires_grad_(False)
        from ..parallel.cp import attach_cp_strategy
        attach_cp_strategy(teacher, self.ps)
        self.teacher_engine = Zero3Engine(teacher, self.ps, compute_dtype=self.compute_dtype, device=self.device,
                                          reshard_after_forward=False, recompute=False, seed=a.train.seed + 1)
        if os.path.isdir(path) and any(f.endswith(".safetensors") for f in os.listdir(path)):
            from ..checkpoint.hf_io import load_hf_weights
            load_hf_weights(self.teacher_engine, path, tcfg, mode=a.train.load_weights_mode
                            if a.train.load_weights_mode != "skip" else "all_ranks")
        self.teacher_config = tcfg

    def _teacher_targets(self, d: Dict[str, torch.Tensor]):
        """(final hidden states, lm-head weight, loss type, loss weight) of the teacher for one micro-batch."""
        te = self.teacher_engine
        hidden = te.forward_only(d["input_ids"], position_ids=d.get("position_ids"), cu_seqlens=d.get("cu_seqlens"))
        tm = te.model
        w = tm.embed_tokens.weight if self.teacher_config.tie_word_embeddings else tm.lm_head.weight
        dd = self.args.distill
        return hidden.detach(), w, dd.distillation_loss_type, float(dd.distillation_loss_weight)

    def _tokenizer(self):
        """Tokenizer for text / chat datasets (local files only); None when the model names none."""
        m = self.args.model
        src = m.tokenizer_path or m.model_path
        if not src or not os.path.isdir(src):
            return None
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(src, local_files_only=True)
        except Exception as e:  # noqa: BLE001
            logger.warning("no tokenizer could be loaded from %s (%s): only tokenised datasets can be used", src, e)
            return None

    def _build_data(self, dataset=None) -> None:
        a = self.args
        self.eval_dataloader, self.eval_history = None, []
        if dataset is None:
            from ..data.datasets import prepare_train_eval
            dataset, eval_dataset = prepare_train_eval(a.data, tokenizer=self._tokenizer(),
                                                       vocab_size=self.model_config.vocab_size, seed=a.train.seed)
            if eval_dataset is not None:
                if self.ps.tp_size > 1 or self.ps.pp_size > 1 or self.ps.sp_size > 1 \
                        or getattr(self.ps, "lm_head_tp_size", 1) > 1:
                    # said at start-up, not at the first checkpoint
                    raise NotImplementedError("data.val_set_size / data.test_datasets: the evaluation pass runs on "
                                              "data-parallel layouts (no tensor, pipeline, context or lm-head parallelism)")
                self.eval_dataloader = self._build_eval_dataloader(eval_dataset)
        shard = None
        if self.ps.sp_size > 1:
            from ..data import SequenceShardCollator
            shard = SequenceShardCollator(self.ps.ringattn_size, self.ps.ulysses_size,
                                          self.ps.ringattn_rank, self.ps.ulysses_rank)
        self.dataloader = build_dataloader(dataset, a.data, a.train, self.ps, shard)
        spe = max(1, len(self.dataloader))
        self.train_steps = a.train.max_steps or spe * a.train.num_train_epochs
        self.steps_per_epoch = spe

    def _build_eval_dataloader(self, eval_dataset):
        """Evaluation rows in a fixed order, one micro-batch per step and rank.  ``data.eval_sample_packing:
        false`` gives every sample a row of its own; over several ranks the ragged tail (fewer rows than
        ranks) is dropped so that every rank runs the same number of forward passes."""
        from ..data.data_loader import PackedDataLoader
        d, t = self.args.data, self.args.train
        loader = PackedDataLoader(
            eval_dataset, packing_len=int(d.sample_packing_sequence_len or 4096), micro_batch_size=t.micro_batch_size,
            grad_accum=1, dp_rank=self.ps.dp_rank, dp_size=self.ps.dp_size,
            packing_method=d.sample_packing_method or "sequential", group_size=int(d.sample_packing_group_size or 100000),
            pad_to_multiple_of=int(d.pad_to_multiple_of or 1), shuffle=False, seed=t.seed,
            drop_last=self.ps.dp_size > 1, pin_memory=bool(d.dataloader_pin_memory))
        if d.eval_sample_packing is False:
            loader.bins = [[i] for i in range(len(eval_dataset))]
            per_step = loader.mbs * loader.dp_size
            loader.steps_per_epoch = len(loader.bins) // per_step if loader.drop_last else -(-len(loader.bins) // per_step)
        return loader

    def evaluate(self) -> Optional[Dict[str, float]]:
        """Mean next-token loss over the evaluation set (``data.test_datasets``, or the ``data.val_set_size``
        split of the training data), summed over ranks by token."""
        if self.eval_dataloader is None:
            return None
        import math
        nll = torch.zeros((), device=self.device, dtype=torch.float64)
        count = torch.zeros((), device=self.device, dtype=torch.float64)
        self.eval_dataloader.epoch, self.eval_dataloader.cursor = 0, 0
        for rows in self.eval_dataloader:
            for mb in rows:
                d = self._to_device(mb)
                s, n = self.engine.eval_loss(d["input_ids"], d["labels"], position_ids=d.get("position_ids"),
                                             cu_seqlens=d.get("cu_seqlens"))
                nll += s.double()
                count += n.double()
        if self.ps.world_size > 1 and dist.is_initialized():
            both = torch.stack([nll, count])
            dist.all_reduce(both, group=self.ps.group("dp"))
            nll, count = both[0], both[1]
        loss = float(nll / count.clamp_min(1))
        out = {"step": self.global_step, "eval_loss": loss, "eval_tokens": float(count),
               "eval_perplexity": math.exp(min(loss, 50.0))}
        self.eval_history.append(out)
        logger.info("step %d: eval loss %.4f over %d tokens", self.global_step, loss, int(count))
        if getattr(self, "sink", None) is not None and hasattr(self.sink, "log"):
            self.sink.log({"eval/loss": loss, "eval/tokens": float(count)}, self.global_step)
        return out

    def _build_optimizer(self) -> None:
        t = self.args.train
        self.optimizer = build_optimizer(
            self.engine, lr=t.lr, weight_decay=t.weight_decay, optimizer_type=t.optimizer,
            optimizer_dtype=t.optimizer_dtype, no_decay_modules=t.no_decay_modules,
            no_decay_params=t.no_decay_params, cautious_weight_decay=t.cautious_weight_decay,
            optimizer_kwargs={k: getattr(t, k) for k in vars(t) if k.startswith("muon_")}
            if t.optimizer == "muon" else
            dict(state_cpu_offload=t.anyprecision_adamw_state_cpu_offload,
                 denominator_chunk_size=t.anyprecision_adamw_denominator_chunk_size)
            if t.optimizer == "anyprecision_adamw" else None)
        self.lr_scheduler = build_lr_scheduler(self.optimizer, self.train_steps, t.lr, t.lr_min,
                                               t.lr_start, t.lr_warmup_ratio, t.lr_decay_style,
                                               t.lr_decay_ratio)

    def _qarl_calibration(self) -> None:
        """Calibration batches through the fake-quantised model before training: fills the wrapped modules'
        statistics and writes them to ``qarl_calibration.json`` (src/xorl/qarl/calibration.py:110-138)."""
        from ..adapters import qarl
        t = self.args.train
        out = qarl.calibrate(lambda ids: self.engine.forward_only(ids), self.model, t.qarl_calib_data,
                             t.qarl_calib_size, t.qarl_quant_sequence_length, device=self.device)
        self.qarl_calibration = out
        if self.ps.rank == 0:
            os.makedirs(t.output_dir, exist_ok=True)
            with open(os.path.join(t.output_dir, "qarl_calibration.json"), "w") as f:
                json.dump(out, f, indent=2)

    def _setup_observability(self) -> None:
        t = self.args.train
        self.meter = EnvironMeter(self.model_config, self.ps.world_size, self.ps.group("dp"),
                                  recompute=t.enable_gradient_checkpointing)
        self.timer = CudaTimer(t.enable_step_phase_timing)
        self.component_timer = None
        if t.enable_per_component_timing:
            from ..utils.component_timer import PerComponentTimer
            self.component_timer = PerComponentTimer(self.model)
        self.profiler = None
        if t.enable_profiling and (not t.profile_rank0_only or self.ps.rank == 0):
            self.profiler = create_profiler(t.profile_start_step, t.profile_end_step, t.profile_trace_dir,
                                            t.profile_record_shapes, t.profile_profile_memory,
                                            t.profile_with_stack, self.ps.rank)
            self.profiler.start()
        from ..utils.diagnostics import MemoryHistory, MetricsSink, RankWatchdog, nonfinite_scan_enabled
        self.memhist = MemoryHistory(self.ps.rank)
        self.sink = MetricsSink(t, self.ps.rank)
        self.scan_nonfinite = nonfinite_scan_enabled()
        self.watchdog = None
        self._canaries = os.environ.get("XORL_B200_CANARIES", "0") == "1"
        # equal micro-batch lengths over the data-parallel group; no collective needs it, it only balances work
        self._sync_padding = os.environ.get("XORL_B200_SYNC_PADDING", "0") == "1" and self.ps.ulysses_size * self.ps.ringattn_size == 1
        if getattr(self.ps, "lm_head_tp_size", 1) > 1:
            # the ranks of an lm-head group pool their tokens for the loss: they need the same number of
            # micro-batches of the same lengths
            if self.ps.ulysses_size * self.ps.ringattn_size > 1 or self.ps.pp_size > 1 or self.ps.ep_size > 1 \
                    or (self.ps.size("dp_replicate") > 1 and self.ps.size("dp_shard") > 1):
                raise NotImplementedError("lm_head_tensor_parallel_size > 1 is built for plain data parallelism "
                                          "(no context, pipeline or expert parallelism, no HSDP)")
            self._sync_padding = True
        if self.ps.world_size > 1 and dist.is_initialized() \
                and os.environ.get("XORL_RANK_WATCHDOG", "1") not in ("0", "false"):
            store = dist.distributed_c10d._get_default_store()
            self.watchdog = RankWatchdog(
                store, self.ps.rank, self.ps.world_size,
                interval_s=float(os.environ.get("XORL_RANK_WATCHDOG_INTERVAL_S", "5")),
                timeout_s=float(os.environ.get("XORL_RANK_WATCHDOG_TIMEOUT_S", "300"))).start()
        if self.ps.rank == 0:
            from ..models.numerics import pin_kernel_configs
            pin = pin_kernel_configs(t.output_dir, strict=t.enable_full_determinism)
            if pin["mismatch"]:
                logger.warning("kernels differ from %s/kernel_pin.json: %s", t.output_dir, pin["mismatch"])
        from ..checkpoint import build_checkpointer
        self.checkpointer = build_checkpointer(self)

    def _resume_checkpoint(self) -> None:
        path = self.args.train.load_checkpoint_path
        if not path:
            return
        from ..checkpoint import resolve_checkpoint_path
        path = resolve_checkpoint_path(path, self.args.train.checkpoint_dir)
        if path is None:
            info_rank0("no checkpoint to resume from; starting fresh")
            return
        extra = self.checkpointer.load(path, load_optimizer=self.args.train.load_optimizer)
        self.global_step = int(extra.get("global_step", 0))
        if "lr_scheduler" in extra:
            self.lr_scheduler.load_state_dict(extra["lr_scheduler"])
        if "train_dataloader" in extra:
            self.dataloader.load_state_dict(extra["train_dataloader"])
        if "environ_meter" in extra:
            self.meter.load_state_dict(extra["environ_meter"])
        if "torch_rng_state" in extra:
            torch.set_rng_state(extra["torch_rng_state"])
        info_rank0(f"resumed from {path} at step {self.global_step}")

    # ------------------------------------------------------------------------------------------
    def count_valid_tokens(self, micro_batches) -> int:
        """Global number of supervised tokens of this step (labels != -100), summed over the
        dp x sp ranks (src/xorl/trainers/training_utils.py:229-249)."""
        local = sum(int(mb["num_valid_tokens"]) if "num_valid_tokens" in mb
                    else int((mb["labels"] != IGNORE_INDEX).sum()) for mb in micro_batches)
        pg_name = self.ps.loss_group_name
        if self.ps.world_size > 1 and pg_name in self.ps.groups and self.ps.groups[pg_name].pg is not None:
            t = torch.tensor([local], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, group=self.ps.group(pg_name))
            return int(t.item())
        return local

    def _to_device(self, mb: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v)
                for k, v in mb.items()}

    def train_step(self, micro_batches: List[Dict[str, torch.Tensor]]) -> Dict[str, Any]:
        t = self.args.train
        global_tokens = max(1, self.count_valid_tokens(micro_batches))
        self.optimizer.zero_grad()
        total = None
        if self.pp_runner is not None:
            for mb in micro_batches:
                self.meter.add(mb)
            total = self.pp_runner.run([self._to_device(mb) for mb in micro_batches],
                                       1.0 / global_tokens)
            if self.pp_runner.bubble_stats:
                b = self.pp_runner.bubble_stats
                logger.info("pp rank %d: waited %.3f s of %.3f s (%.1f%%; unit-cost estimate %.1f%%), sent %.1f MB",
                            self.ps.pp_rank, b["wait_s"], b["step_s"], 100 * b["measured_bubble_fraction"],
                            100 * b["analytic_bubble_fraction"], b["p2p_sent_bytes"] / 1e6)
            micro_batches = []
        for i, mb in enumerate(micro_batches):
            self.meter.add(mb)
            d = self._to_device(mb)
            phase = self.timer.scope("forward_backward")
            phase.__enter__()
            # gradient norms are taken unit by unit during the last micro-batch's backward
            self.engine.final_micro_batch = i == len(micro_batches) - 1
            extra = {"local_cu_seqlens": mb.get("local_cu_seqlens")}
            if self.teacher_engine is not None:
                extra["distill"] = self._teacher_targets(d)
            loss = self.engine.forward_backward(
                d["input_ids"], d["labels"], position_ids=d.get("position_ids"),
                cu_seqlens=d.get("cu_seqlens"), grad_scale=1.0 / global_tokens,
                extra_loss_fn=self._extra_loss_fn(), extra=extra)
            total = loss if total is None else total + loss
            phase.__exit__(None, None, None)
        with self.timer.scope("grad_sync"):
            self.engine.finish_grad_sync()
        dump = os.environ.get("XORL_DEBUG_DUMP_GRADS")
        if dump and self.global_step == 0:
            self._dump_full_gradients(dump)
        if self.scan_nonfinite:
            from ..utils.diagnostics import nonfinite_gradient_report
            bad = nonfinite_gradient_report(self.engine)
            if bad:
                logger.warning("step %d rank %d: non-finite gradients in %s", self.global_step + 1,
                               self.ps.rank, ", ".join(bad[:20]))
        with self.timer.scope("grad_norm"):
            norm, coef = self.engine.grad_norm_and_clip_coef(t.max_grad_norm)
        with self.timer.scope("optimizer"):
            self.optimizer.step(clip_coef=coef if t.max_grad_norm > 0 else None)
        self.lr_scheduler.step()
        if self._canaries:
            from ..utils import canary
            canary.check_all()                      # XORL_B200_CANARIES=1: guard words around workspaces intact?
        if self.ps.world_size > 1 and self.ps.group(self.ps.loss_group_name) is not None:
            dist.all_reduce(total, group=self.ps.group(self.ps.loss_group_name))
        self.global_step += 1
        la = self.args.lora
        if la.enable_lora and la.merge_lora_interval and self.global_step % la.merge_lora_interval == 0:
            self.maybe_merge_lora()
        return {"loss": total, "grad_norm": norm, "lr": self.optimizer.lr, "tokens": global_tokens}

    def maybe_merge_lora(self) -> None:
        """ReLoRA-style merge: fold the adapters into the (gathered) base weights, write the shards
        back, restart B at zero and optionally reset the optimizer moments
        (src/xorl/trainers/training_utils.py:346-372)."""
        from ..adapters.lora import ExpertsLoRA, LoraLinear
        eng = self.engine
        if hasattr(eng, "sync_optimizer"):
            eng.sync_optimizer()
        with torch.no_grad():
            for unit in eng.units:
                eng.gather(unit)
                eng.wait_gather(unit)
                touched = False
                for mod in unit.modules:
                    for m in mod.modules():
                        if isinstance(m, LoraLinear) and hasattr(m, "weight"):
                            m.merge()
                            touched = True
                        elif isinstance(getattr(m, "lora", None), ExpertsLoRA):
                            m.lora.merge_into(m)
                            touched = True
                if touched:
                    for g in unit.groups:
                        s0, s1 = g.shard_range()
                        if g.master is None:
                            # frozen group: the merged base weights live in the compute-dtype shard
                            if g.full is not g.shard_lp:
                                g.shard_lp.copy_(g.full[s0:s1])
                            continue
                        # trainable group: only lora_B restarts (at zero); every other trainable
                        # parameter (lora_A, unfrozen weights) keeps its fp32 master value
                        for i, a, b in g.param_segments_in_shard():
                            if ".lora_B." in g.named_params[i][0] or g.named_params[i][0].endswith("_lora_B"):
                                g.master[a:b].zero_()
                                if g.shard_lp is not g.master:
                                    g.shard_lp[a:b].zero_()
                if eng.reshard:
                    eng.release(unit)
        if self.args.lora.reset_optimizer_on_merge:
            for st in self.optimizer.state.values():
                for v in st.values():
                    v.zero_()

    def _dump_full_gradients(self, out_dir: str) -> None:
        """Debug aid (``XORL_DEBUG_DUMP_GRADS=<dir>``): after the first step's backward, the fully
        reduced fp32 gradient of every parameter, gathered to its unsharded shape, is written by the
        first rank of every pipeline stage.  Runs under any parallel layout, so two layouts can be
        compared parameter by parameter."""
        grads = {n: t.detach().float().cpu().clone() for n, t in self.engine.iter_full_tensors("grad")}
        ps = self.ps
        first_of_stage = ps.rank == min(ps.group_ranks("stage")) if "stage" in ps.groups else ps.rank == 0
        if first_of_stage or ps.world_size == 1:
            os.makedirs(out_dir, exist_ok=True)
            torch.save(grads, os.path.join(out_dir, f"grads_pp{ps.pp_rank if ps.pp_size > 1 else 0}.pt"))

    def _extra_loss_fn(self):
        return None

    # ------------------------------------------------------------------------------------------
    def train(self) -> Dict[str, Any]:
        t = self.args.train
        done = False
        # train.gc_steps > 0: the cyclic collector runs only at those steps, so that its pauses are the
        # same on every rank instead of stalling one rank inside a collective
        gc_was_enabled = gc.isenabled()
        if t.gc_steps and t.gc_steps > 0:
            gc.disable()
        while not done:
            for micro_batches in self.dataloader:
                if self.global_step >= self.train_steps:
                    done = True
                    break
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                if self.watchdog is not None:
                    self.watchdog.check()           # a dead peer is noticed before the next launch
                t0 = time.time()
                if self._sync_padding:
                    # lm-head parallelism needs equal lengths inside each lm-head group only
                    pad_group = self.ps.group("lm_head_tp") if getattr(self.ps, "lm_head_tp_size", 1) > 1 \
                        and os.environ.get("XORL_B200_SYNC_PADDING", "0") != "1" else self.ps.group("dp")
                    micro_batches = synchronize_micro_batch_padding(
                        micro_batches, pad_group, multiple_of=max(1, self.args.data.pad_to_multiple_of or 1))
                try:
                    with nvtx_range("train_step"):
                        out = self.train_step(micro_batches)
                    loss = float(out["loss"])       # device -> host read of the step result
                except BaseException as e:
                    if isinstance(e, torch.OutOfMemoryError):
                        self.memhist.on_oom()
                    if self.watchdog is not None:
                        self.watchdog.report_failure(f"{type(e).__name__}: {e}")
                    raise
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                dt = time.time() - t0
                metrics = self.meter.step(dt, self.global_step)
                metrics.update(loss=loss, grad_norm=float(out["grad_norm"]), lr=out["lr"],
                               step=self.global_step, step_time=dt)
                if t.enable_step_phase_timing:
                    # per-phase device time of this step (CUDA events; reading them synchronises, which
                    # step_phase_timing_sync_cuda=false defers to every 10th step)
                    if t.step_phase_timing_sync_cuda or self.global_step % 10 == 0:
                        for k, v in self.timer.summary().items():
                            metrics[f"phase/{k}_ms"] = v
                    if self.component_timer is not None:
                        for k, v in self.component_timer.flush().items():
                            metrics[f"component/{k}_ms"] = v
                        self.component_timer.reset()
                    if t.enable_step_memory_profiling and self.device.type == "cuda":
                        metrics["memory/peak_allocated_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
                        torch.cuda.reset_peak_memory_stats()
                self.loss_history.append(loss)
                self.metrics_history.append(metrics)
                self._maybe_log(metrics)
                self.sink.log(metrics, self.global_step)
                self.memhist.after_step(self.global_step)
                if self.profiler is not None:
                    self.profiler.step()
                self._maybe_save_checkpoint()
                if t.gc_steps and self.global_step % t.gc_steps == 0:
                    gc.collect()                 # automatic collection is off during training (see train())
                if t.empty_cache_steps and self.global_step % t.empty_cache_steps == 0 \
                        and self.device.type == "cuda":
                    torch.cuda.empty_cache()
            else:
                if self.global_step >= self.train_steps:
                    done = True
            if len(self.dataloader) == 0:
                break
        if gc_was_enabled:
            gc.enable()
        return self._finalize()

    def _maybe_log(self, m: Dict[str, float]) -> None:
        if self.ps.rank != 0:
            return
        logger.info("step %d/%d loss %.4f grad_norm %.3f lr %.3e tok/s %.1fK mfu %.3f step %.3fs",
                    m["step"], self.train_steps, m["loss"], m["grad_norm"], m["lr"],
                    m["tokens_per_second(K)"], m["efficiency/mfu"], m["step_time"])

    def _maybe_save_checkpoint(self, force: bool = False) -> None:
        t = self.args.train
        # train.save_steps: every N steps; train.save_epochs: every (fraction of an) epoch, counted in
        # steps like the reference does (src/xorl/trainers/trainer.py:679-683,2493-2498)
        epoch_steps = int(t.save_epochs * self.steps_per_epoch) if t.save_epochs else 0
        due = (t.save_steps and self.global_step % t.save_steps == 0) or \
            (epoch_steps and self.global_step % epoch_steps == 0)
        if not force and not due:
            return
        extra = {"global_step": self.global_step, "lr_scheduler": self.lr_scheduler.state_dict(),
                 "train_dataloader": self.dataloader.state_dict(),
                 "environ_meter": self.meter.state_dict(), "torch_rng_state": torch.get_rng_state()}
        self.checkpointer.save(self.global_step, extra)
        if due:
            self.evaluate()

    def _finalize(self) -> Dict[str, Any]:
        t = self.args.train
        if self.profiler is not None:
            self.profiler.stop()
        if self.watchdog is not None:
            self.watchdog.stop()
        if self.eval_dataloader is not None and not (self.eval_history and self.eval_history[-1]["step"] == self.global_step):
            self.evaluate()
        self.sink.close()
        self.memhist.close()
        result = {"loss_history": self.loss_history, "global_step": self.global_step,
                  "metrics": self.metrics_history[-1] if self.metrics_history else {}}
        if self.eval_history:
            result["eval_history"] = self.eval_history
        if self.pp_runner is not None and self.pp_runner.bubble_stats:
            result["pp_bubble"] = dict(self.pp_runner.bubble_stats, pp_rank=self.ps.pp_rank)
        if self.ps.sp_size > 1:
            from ..parallel.sequence_parallel import PEER_PATH_CALLS
            result["cp_peer_paths"] = dict(PEER_PATH_CALLS)
        if self.ps.tp_sequence_parallel:
            from ..parallel.tp_fused import sp_context
            sp = sp_context()
            result["tp_collective_gemms"] = {"fused": sp.fused_calls, "unfused": sp.fallback_calls}
        if t.save_hf_weights and self.global_step > 0 and t.save_steps >= 0 and \
                os.environ.get("XORL_SKIP_FINAL_EXPORT", "0") != "1":
            out_dir = os.path.join(t.output_dir, f"global_step_{self.global_step}", "hf_ckpt")
            if self.args.lora.enable_lora:
                from ..adapters.lora import save_lora_checkpoint
                save_lora_checkpoint(self.engine, out_dir, self.args.model.model_path or "")
            else:
                from ..checkpoint.hf_io import save_hf_weights
                save_hf_weights(self.engine, out_dir, self.model_config)
        if self.ps.rank == 0:
            with open(os.path.join(t.output_dir, "training_metrics.json"), "w") as f:
                json.dump(result, f, indent=2, default=float)
        if dist.is_initialized():
            dist.barrier()
        return result
