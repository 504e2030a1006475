"""``python -m xorl_b200.cli.convert_hf_to_dcp --model-path HF_DIR --output-dir OUT [--step N]``

Turns a Hugging Face safetensors checkpoint into a DCP directory
``OUT/checkpoints/global_step_N/`` that ``train.load_checkpoint_path`` accepts, without running a
training step: the model is built on the meta device, the weights stream through the family's
checkpoint handler into a single-process ZeRO engine on CPU, and the engine's state is written
with ``load_optimizer`` left to the first real run.  (The reference ships the same kind of tool for
one family, scripts/convert_dsv4_hf_to_dcp.py; this one goes through the handler registry and works
for every family.)"""
from __future__ import annotations

import argparse
import json
import os


def main(argv=None) -> str:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-path", required=True, help="directory with config.json and *.safetensors")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--step", type=int, default=0)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    a = ap.parse_args(argv)

    import torch

    from ..checkpoint.checkpointer import DistributedCheckpointer
    from ..checkpoint.hf_io import load_hf_weights
    from ..models import build_model_config
    from ..models.registry import get_model_class
    from ..parallel.state import get_parallel_state
    from ..parallel.zero import Zero3Engine

    class _M:
        config_path, model_path, foundation = a.model_path, a.model_path, {}

    cfg = build_model_config(_M)
    model = get_model_class(cfg)(cfg, dtype=torch.float32, device="meta")
    engine = Zero3Engine(model, get_parallel_state(), compute_dtype=getattr(torch, a.dtype),
                         device=torch.device("cpu"), seed=0)
    missing = load_hf_weights(engine, a.model_path, cfg, strict=True)
    ckpt = DistributedCheckpointer(engine, None, os.path.join(a.output_dir, "checkpoints"))
    path = ckpt.save(a.step, {"global_step": a.step, "converted_from": os.path.abspath(a.model_path)})
    ckpt.wait()
    out = path or os.path.join(a.output_dir, "checkpoints", f"global_step_{a.step}")
    print(json.dumps({"checkpoint": out, "missing": missing}))
    return out


if __name__ == "__main__":
    main()
