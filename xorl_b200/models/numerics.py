"""Numerical programme of a model: the set of precision and determinism choices that have to agree
between training and the serving engine for log-probabilities to match (the reference resolves
this per model family, src/xorl/models/auto.py:573 ``resolve_model_numerical_program``).

``resolve_numerical_program`` merges family defaults with ``model.*`` / ``train.*`` arguments;
``apply_numerical_program`` sets the corresponding module / context flags; ``describe`` reports
which parts of a step are bit-reproducible run to run with this framework's kernels."""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Dict


@dataclass
class NumericalProgram:
    router_fp32: bool = True            # gate logits and top-k in fp32
    lm_head_fp32: bool = False          # upcast hidden states and lm-head for the loss
    rmsnorm_fp32_accum: bool = True
    rope_fp32: bool = True
    attention_softmax_fp32: bool = True
    moe_combine_fp32: bool = True       # weighted sum over the k expert outputs in fp32
    reduce_dtype: str = "fp32"          # gradient reduce-scatter accumulation
    batch_invariant: bool = False       # results independent of how sequences are packed together
    deterministic: bool = False         # no floating-point atomics anywhere in the step

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


FAMILY_DEFAULTS: Dict[str, Dict[str, Any]] = {
    "deepseek_v3": {"router_fp32": True, "moe_combine_fp32": True},
    "glm4_moe": {"router_fp32": True},
    "gpt_oss": {"router_fp32": True, "attention_softmax_fp32": True},
}


def resolve_numerical_program(cfg, model_args=None, train_args=None) -> NumericalProgram:
    prog = NumericalProgram(**FAMILY_DEFAULTS.get(getattr(cfg, "model_type", ""), {}))
    if model_args is not None:
        if getattr(model_args, "router_fp32", None) is not None:
            prog.router_fp32 = bool(model_args.router_fp32)
        if getattr(model_args, "lm_head_fp32", None) is not None:
            prog.lm_head_fp32 = bool(model_args.lm_head_fp32)
    if train_args is not None:
        prog.reduce_dtype = getattr(train_args, "fsdp_reduce_dtype", prog.reduce_dtype)
        prog.deterministic = bool(getattr(train_args, "deterministic", False))
        prog.batch_invariant = bool(getattr(train_args, "batch_invariant", False)) or prog.deterministic
    return prog


def describe(prog: NumericalProgram, on_gpu: bool = True) -> Dict[str, str]:
    """Which parts of a step reproduce bit for bit, given the kernels in this framework."""
    rep = {
        "gemm": "deterministic (fixed tile order, no split-K)",
        "attention_forward": "deterministic; per-document, so independent of packing",
        "attention_backward": ("dQ accumulates with fp32 atomics across key tiles: run-to-run differences in the "
                               "last bits" if on_gpu else "deterministic"),
        "rmsnorm_backward": "deterministic (two-pass partial reduction in a fixed order)",
        "embedding_backward": "fp32 atomics on repeated tokens" if on_gpu else "deterministic",
        "zero_reduce_scatter": "fixed rank order in the fused transport; NCCL ring order otherwise",
        "moe_combine": "fp32, fixed k order" if prog.moe_combine_fp32 else "bf16",
        "router": "fp32" if prog.router_fp32 else "compute dtype",
    }
    if prog.deterministic and on_gpu:
        rep["note"] = ("deterministic=True selects the PyTorch reference path for attention backward and "
                       "embedding backward (slower)")
    return rep


def apply_numerical_program(model, prog: NumericalProgram) -> None:
    model.numerical_program = prog
    model.ctx_defaults["deterministic"] = prog.deterministic
    for m in model.modules():
        if hasattr(m, "router_fp32"):
            m.router_fp32 = prog.router_fp32


# ---- kernel pin ---------------------------------------------------------------------------------
class KernelPinError(RuntimeError):
    """The kernels of this process differ from the ones a run was pinned to."""


def kernel_fingerprint() -> Dict[str, Any]:
    """What decides the bits a kernel produces here: the native library itself (its kernels have
    fixed tile shapes, no autotuning and no run-time cache to pin), the selectable kernel variants,
    and the PyTorch / CUDA versions behind the remaining tensor ops.  The reference pins its
    autotune caches for the same purpose (src/xorl/ops/kernel_config_pin.py:67-182)."""
    import hashlib

    import torch

    from ..ops import _lib, gemm as gemm_mod
    path = _lib.cuda_lib_path()
    digest = ""
    if path.exists():
        h = hashlib.sha256()
        with open(path, "rb") as f:
            for blk in iter(lambda: f.read(1 << 20), b""):
                h.update(blk)
        digest = h.hexdigest()
    return {"native_library_sha256": digest, "gemm_variant": getattr(gemm_mod, "_VARIANT", "pair"),
            "torch": torch.__version__, "cuda": torch.version.cuda or "",
            "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"}


def pin_kernel_configs(directory: str, strict: bool = False) -> Dict[str, Any]:
    """Writes ``kernel_pin.json`` on first use; afterwards compares.  A mismatch raises with
    ``strict`` (bit-exact lanes) and is returned under ``"mismatch"`` otherwise."""
    import json
    import os
    fp = kernel_fingerprint()
    path = os.path.join(directory, "kernel_pin.json")
    if not os.path.exists(path):
        os.makedirs(directory, exist_ok=True)
        with open(path, "w") as f:
            json.dump(fp, f, indent=2)
        return {"pinned": fp, "mismatch": {}}
    with open(path) as f:
        old = json.load(f)
    diff = {k: (old.get(k), fp.get(k)) for k in set(old) | set(fp) if old.get(k) != fp.get(k)}
    if diff and strict:
        raise KernelPinError(f"kernels differ from the pin in {path}: {diff}")
    return {"pinned": old, "mismatch": diff}
