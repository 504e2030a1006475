"""Preprocess and export command-line tools on CPU."""
import json
import os
import sys

import pytest
import torch
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_preprocess_cli(tmp_path):
    from xorl_b200.cli.preprocess import main
    rows = [{"input_ids": list(range(5, 5 + n))} for n in (30, 90, 60, 120, 10)]
    with open(tmp_path / "d.jsonl", "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    cfg = {"model": {"config_path": "tiny-qwen3"},
           "data": {"datasets": [{"path": str(tmp_path / "d.jsonl"), "type": "tokenized", "max_seq_len": 100}],
                    "sample_packing_sequence_len": 128, "dataset_prepared_path": str(tmp_path / "prep")},
           "train": {"output_dir": str(tmp_path / "o"), "device": "cpu"}}
    (tmp_path / "c.yaml").write_text(yaml.safe_dump(cfg))
    out = main([str(tmp_path / "c.yaml")])
    meta = json.load(open(os.path.join(out, "meta.json")))
    pk = json.load(open(os.path.join(out, "packing.json")))
    assert meta["num_samples"] == 5 and meta["total_tokens"] == 30 + 90 + 60 + 100 + 10
    assert sorted(i for b in pk["bins"] for i in b) == [0, 1, 2, 3, 4] and meta["num_bins"] == 3
    from xorl_b200.data.datasets import prepare_datasets
    ds = prepare_datasets([{"path": os.path.join(out, "data.arrow"), "type": "tokenized"}])
    assert len(ds) == 5 and len(ds[3]["input_ids"]) == 100
    # numbered shard files + a validation split; the directory itself is a dataset (json files beside the data
    # are not rows), with the held-out rows under ``split: eval``
    cfg["data"].update(num_dataset_shards_to_save=2, val_set_size=2, dataset_prepared_path=str(tmp_path / "prep2"))
    (tmp_path / "c2.yaml").write_text(yaml.safe_dump(cfg))
    out2 = main([str(tmp_path / "c2.yaml")])
    assert sorted(f for f in os.listdir(out2) if f.endswith(".arrow")) == \
        ["data-00000-of-00002.arrow", "data-00001-of-00002.arrow", "eval.arrow"]
    meta2 = json.load(open(os.path.join(out2, "meta.json")))
    assert meta2["num_samples"] == 3 and meta2["num_eval_samples"] == 2
    tr = prepare_datasets([{"path": out2, "type": "tokenized"}])
    ev = prepare_datasets([{"path": out2, "type": "tokenized", "split": "eval"}])
    assert len(tr) == 3 and len(ev) == 2
    assert sorted([len(tr[i]["input_ids"]) for i in range(3)] + [len(ev[i]["input_ids"]) for i in range(2)]) == [10, 30, 60, 90, 100]


def test_export_quantized_roundtrip(tmp_path):
    from safetensors.torch import load_file, save_file
    from xorl_b200.cli import export_nvfp4, export_quantized
    from xorl_b200.ops import quantize as Q
    torch.manual_seed(0)
    src = tmp_path / "src"
    os.makedirs(src)
    w = {"model.layers.0.self_attn.q_proj.weight": torch.randn(256, 128).bfloat16(),
         "model.layers.0.mlp.down_proj.weight": torch.randn(128, 384).bfloat16(),
         "model.norm.weight": torch.ones(128).bfloat16(),
         "lm_head.weight": torch.randn(512, 128).bfloat16()}
    save_file(w, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"model_type": "qwen3", "hidden_size": 128}))
    st = export_quantized.main(["--src", str(src), "--dst", str(tmp_path / "fp8"), "--format", "block_fp8"])
    assert st["quantized"] == 2 and st["kept"] == 2 and st["bytes_out"] < st["bytes_in"]
    out = load_file(str(tmp_path / "fp8" / "model-00001.safetensors"))
    q = out["model.layers.0.self_attn.q_proj.weight"]
    s = out["model.layers.0.self_attn.q_proj.weight_scale_inv"]
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 1)
    back = Q.block_fp8_dequantize_128x128(q, s, dtype=torch.float32)
    ref = w["model.layers.0.self_attn.q_proj.weight"].float()
    assert (back - ref).norm() / ref.norm() < 0.05
    assert torch.equal(out["lm_head.weight"], w["lm_head.weight"])
    cfg = json.load(open(tmp_path / "fp8" / "config.json"))
    assert cfg["quantization_config"]["weight_block_size"] == [128, 128] and cfg["hidden_size"] == 128
    # nvfp4: serving layout; q / k / v of one layer share the per-tensor scale, the lone projection has its own
    w2 = dict(w)
    w2["model.layers.0.self_attn.k_proj.weight"] = (torch.randn(64, 128) * 3).bfloat16()
    w2["model.layers.0.self_attn.v_proj.weight"] = (torch.randn(64, 128) * 0.1).bfloat16()
    src2 = tmp_path / "src2"
    os.makedirs(src2)
    save_file(w2, str(src2 / "model.safetensors"))
    (src2 / "config.json").write_text(json.dumps({"model_type": "qwen3", "hidden_size": 128}))
    amax = tmp_path / "amax.json"
    amax.write_text(json.dumps({"modules": {"model.layers.0.mlp.down_proj": {"input_amax": 5.0}}}))
    st4 = export_nvfp4.main(["--src", str(src2), "--dst", str(tmp_path / "fp4"), "--act-amax", str(amax)])
    assert st4["quantized"] == 4 and st4["kept"] == 2 and st4["fused_groups"] == 1
    out4 = load_file(str(tmp_path / "fp4" / "model-00001.safetensors"))
    k = "model.layers.0.mlp.down_proj"
    assert out4[k + ".weight"].shape == (128, 192) and out4[k + ".weight_scale"].shape == (128, 24)
    assert out4[k + ".weight_scale"].dtype == torch.float8_e4m3fn and out4[k + ".weight_scale_2"].dim() == 0
    assert abs(float(out4[k + ".input_scale"]) - 5.0 / (6 * 448)) < 1e-9
    back4 = Q.nvfp4_dequantize(out4[k + ".weight"].reshape(-1), out4[k + ".weight_scale"], out4[k + ".weight_scale_2"],
                               (128, 384), dtype=torch.float32)
    assert (back4 - w[k + ".weight"].float()).norm() / w[k + ".weight"].float().norm() < 0.15
    a = "model.layers.0.self_attn."
    shared = {float(out4[a + p + ".weight_scale_2"]) for p in ("q_proj", "k_proj", "v_proj")}
    assert len(shared) == 1 and abs(shared.pop() - float(w2[a + "k_proj.weight"].float().abs().max()) / (6 * 448)) < 1e-7
    assert a + "q_proj.input_scale" not in out4
    vb = Q.nvfp4_dequantize(out4[a + "v_proj.weight"].reshape(-1), out4[a + "v_proj.weight_scale"],
                            out4[a + "v_proj.weight_scale_2"], (64, 128), dtype=torch.float32)
    ref_v = w2[a + "v_proj.weight"].float()
    assert (vb - ref_v).norm() / ref_v.norm() < 0.2             # the small member survives the shared scale
    hq = json.load(open(tmp_path / "fp4" / "hf_quant_config.json"))["quantization"]
    assert hq["quant_algo"] == "NVFP4" and hq["exclude_modules"] == ["lm_head"]
    assert json.load(open(tmp_path / "fp4" / "config.json"))["quantization_config"]["format"] == "nvfp4"
    with pytest.raises(FileExistsError):
        export_nvfp4.main(["--src", str(src2), "--dst", str(tmp_path / "fp4")])


def test_convert_hf_to_dcp_roundtrip(tmp_path):
    """HF safetensors -> DCP directory -> a fresh engine holds the same weights."""
    import torch
    from xorl_b200.checkpoint.checkpointer import DistributedCheckpointer
    from xorl_b200.checkpoint.hf_io import save_hf_weights
    from xorl_b200.cli.convert_hf_to_dcp import main as convert
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.parallel.state import get_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    cfg = preset("tiny-qwen3")

    def engine(seed):
        m = DecoderLM(cfg, dtype=torch.float32, device="meta")
        return Zero3Engine(m, get_parallel_state(), compute_dtype=torch.float32, device=torch.device("cpu"), seed=seed)

    src = engine(0)
    hf = tmp_path / "hf"
    save_hf_weights(src, str(hf), cfg, dtype=torch.float32)
    out = convert(["--model-path", str(hf), "--output-dir", str(tmp_path / "out"), "--step", "7"])
    assert out.endswith("global_step_7") and os.path.exists(os.path.join(out, ".metadata"))
    dst = engine(1)
    DistributedCheckpointer(dst, None, str(tmp_path / "out" / "checkpoints")).load(out, load_optimizer=False)
    for a, b in zip(src.all_groups(), dst.all_groups()):
        assert torch.equal(a.master, b.master), a.name
    reset_parallel_state()


def test_every_config_key_is_read_or_accounted_for():
    """No key of the YAML schema is silently ignored: each one is read by some module, or listed as
    satisfied by design (with the reason), or raises NotImplementedError naming the key when it is set
    to a value that asks for something that is not built."""
    import dataclasses
    import re
    import pytest
    from xorl_b200 import arguments as A
    from xorl_b200 import config_policy as P
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "xorl_b200")
    src = ""
    for d, _, files in os.walk(root):
        for f in files:
            if f.endswith(".py") and f not in ("arguments.py", "config_policy.py"):
                src += open(os.path.join(d, f)).read() + "\n"
    argsrc = open(os.path.join(root, "arguments.py")).read()
    sections = {"model": A.ModelArguments, "data": A.DataArguments, "train": A.TrainingArguments,
                "lora": A.LoRAArguments, "distill": A.DistillationArguments}
    unaccounted = []
    for sec, cls in sections.items():
        for f in dataclasses.fields(cls):
            if not f.init:
                continue
            pat = r"\b" + re.escape(f.name) + r"\b"
            read = re.search(pat, src) is not None or len(re.findall(pat, argsrc)) > 1 \
                or (f.name.startswith("muon_") and "startswith(\"muon_\")" in src)
            if read or f.name in P.SATISFIED_BY_DESIGN.get(sec, {}) or f.name in P.UNSUPPORTED.get(sec, {}):
                continue
            unaccounted.append(f"{sec}.{f.name}")
    assert not unaccounted, unaccounted
    # every unsupported key raises for a value outside its accepted set, and names itself
    candidates = (True, 7, 0.37, 2.0, 64, "something-else", "true", "tilelang", "flashmla", "full_matrix",
                  "anyprecision_adamw", "residual", "deep_gemm", ["x"], {"a": 1})
    for sec, table in P.UNSUPPORTED.items():
        for key, (ok, why) in table.items():
            raised = False
            for bad in candidates:
                if ok(bad):
                    continue
                try:
                    A.build_args({sec: {key: bad}})
                except NotImplementedError as e:
                    assert key in str(e), (key, str(e))
                    raised = True
                    break
                except (ValueError, TypeError):
                    continue                     # not a value of the field's declared type: try the next
            assert raised, f"{sec}.{key} never raised NotImplementedError"
    # the defaults themselves are all accepted
    A.build_args({})


def test_the_configuration_reference_is_current():
    """``docs/config-reference.md`` is what ``python -m xorl_b200.cli.config_reference`` prints now."""
    from xorl_b200.cli.config_reference import render
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "docs", "config-reference.md")) as f:
        assert f.read() == render(), "regenerate: python -m xorl_b200.cli.config_reference > docs/config-reference.md"
