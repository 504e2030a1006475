"""LoRA on CPU: only adapters train, the delta on fused projections equals per-slice adapters,
merge folds the update into the base weight, and the PEFT export has the expected names."""
import os

import torch

from xorl_b200.arguments import LoRAArguments
from xorl_b200.models.config import preset
from xorl_b200.models.decoder import DecoderLM
from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state


def _engine(lora_args, tmp=None):
    from xorl_b200.adapters.lora import inject_lora
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    model = DecoderLM(preset("tiny-qwen3", tie_word_embeddings=False), device="meta")
    wrapped = inject_lora(model, lora_args)
    eng = Zero3Engine(model, ps, compute_dtype=torch.float32, device=torch.device("cpu"))
    return model, eng, wrapped


def test_lora_trains_only_adapters(tmp_path):
    from xorl_b200.adapters.lora import merge_lora, save_lora_checkpoint
    from xorl_b200.optim import build_optimizer
    la = LoRAArguments(enable_lora=True, lora_rank=4, lora_alpha=8, lora_b_init_std=0.01,
                       lora_target_modules=["q_proj", "v_proj", "down_proj"])
    model, eng, wrapped = _engine(la)
    assert len(wrapped) == 4  # qkv_proj and down_proj in both layers
    frozen = [g for g in eng.all_groups() if getattr(g, "frozen", False)]
    train = [g for g in eng.all_groups() if not getattr(g, "frozen", False)]
    assert frozen and train
    assert all(".lora_" in n for g in train for n, _ in g.named_params)
    base_before = {n: t.clone() for n, t in eng.iter_full_tensors("master") if ".lora_" not in n}
    opt = build_optimizer(eng, lr=1e-2, weight_decay=0.0)
    ids = torch.randint(0, 1024, (2, 65))
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)
        eng.finish_grad_sync()
        _, coef = eng.grad_norm_and_clip_coef(1.0)
        opt.step(clip_coef=coef)
        losses.append(float(loss))
    assert losses[-1] < losses[0]
    for n, t in eng.iter_full_tensors("master"):
        if ".lora_" not in n:
            assert torch.equal(t, base_before[n]), n
    save_lora_checkpoint(eng, str(tmp_path / "peft"), "tiny")
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "peft" / "adapter_model.safetensors"))
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in sd
    assert "base_model.model.model.layers.1.mlp.down_proj.lora_B.weight" in sd
    assert os.path.exists(tmp_path / "peft" / "adapter_config.json")
    # merging keeps the function
    x, y = ids[:, :-1], ids[:, 1:]
    with torch.no_grad():
        before = float(model(x, labels=y, grad_scale=1.0 / 128)["loss"])
        assert merge_lora(model) == 4
        after = float(model(x, labels=y, grad_scale=1.0 / 128)["loss"])
    assert abs(before - after) < 1e-4


def test_qlora_and_fp8_and_qarl_forward_backward():
    from xorl_b200.adapters.fp8 import FP8Linear
    from xorl_b200.adapters.qarl import fake_quant
    from xorl_b200.adapters.qlora import inject_qlora
    from xorl_b200.models.layers import Linear
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    for fmt, group in (("nf4", 64), ("nvfp4", 16), ("block_fp8", 128)):
        la = LoRAArguments(enable_lora=True, enable_qlora=True, lora_rank=4, quant_format=fmt,
                           quant_group_size=group, lora_b_init_std=0.01,
                           lora_target_modules=["q_proj", "down_proj"])
        model = DecoderLM(preset("tiny-qwen3", tie_word_embeddings=False), device="meta")
        assert len(inject_qlora(model, la)) == 4
        eng = Zero3Engine(model, ps, compute_dtype=torch.float32, device=torch.device("cpu"))
        opt = build_optimizer(eng, lr=1e-2, weight_decay=0.0)
        ids = torch.randint(0, 1024, (2, 65))
        losses = []
        for _ in range(4):
            opt.zero_grad()
            losses.append(float(eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)))
            eng.finish_grad_sync()
            opt.step()
        assert losses[-1] < losses[0], (fmt, losses)
    # fp8 linear close to the exact one, gradients flow
    torch.manual_seed(0)
    base = Linear(256, 128, dtype=torch.float32)
    torch.nn.init.normal_(base.weight, 0, 0.05)
    f8 = FP8Linear(base)
    x = torch.randn(16, 256, requires_grad=True)
    y = f8(x)
    ref = x @ base.weight.t()
    assert (y - ref).norm() / ref.norm() < 0.06
    y.sum().backward()
    assert x.grad is not None and base.weight.grad is not None
    w = torch.randn(32, 64, requires_grad=True)
    fq = fake_quant(w, "nvfp4")
    fq.sum().backward()
    assert torch.allclose(w.grad, torch.ones_like(w))


def test_relora_merge_keeps_fp32_masters_of_the_adapters():
    """A ReLoRA merge folds B A into the frozen base weight and restarts B at zero; the fp32 master
    copy of lora_A must survive it bit for bit (it is not rebuilt from its bf16 compute copy)."""
    from types import SimpleNamespace
    from xorl_b200.adapters.lora import inject_lora
    from xorl_b200.parallel.zero import Zero3Engine
    from xorl_b200.trainers.trainer import Trainer
    la = LoRAArguments(enable_lora=True, lora_rank=4, lora_alpha=8, lora_b_init_std=0.02,
                       lora_target_modules=["q_proj", "down_proj"], reset_optimizer_on_merge=False)
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    model = DecoderLM(preset("tiny-qwen3", tie_word_embeddings=False), device="meta")
    inject_lora(model, la)
    eng = Zero3Engine(model, ps, compute_dtype=torch.bfloat16, device=torch.device("cpu"))
    # give the masters values that bf16 cannot hold
    for g in eng.all_groups():
        if g.master is not None:
            g.master.add_(1e-5 * torch.arange(g.master.numel(), dtype=torch.float32).remainder(7))
            eng.refresh_compute_copy(g)
    before = {n: t.clone() for n, t in eng.iter_full_tensors("master")}
    stub = SimpleNamespace(engine=eng, args=SimpleNamespace(lora=la), optimizer=SimpleNamespace(state={}))
    Trainer.maybe_merge_lora(stub)
    after = dict(eng.iter_full_tensors("master"))
    changed_base = 0
    for n, t in after.items():
        if ".lora_A." in n:
            assert torch.equal(t, before[n]), n
            assert not torch.equal(t, t.bfloat16().float())          # still holds sub-bf16 bits
        elif ".lora_B." in n:
            assert float(t.abs().max()) == 0.0, n
        elif not torch.equal(t.float(), before[n].float()):
            changed_base += 1
    assert changed_base == 4                                          # qkv_proj + down_proj, two layers


def _moe_engine(la, seed=0):
    from xorl_b200.adapters.lora import inject_lora
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    model = DecoderLM(preset("tiny-qwen3-moe", router_aux_loss_coef=0.0), device="meta")
    wrapped = inject_lora(model, la)
    eng = Zero3Engine(model, ps, compute_dtype=torch.float32, device=torch.device("cpu"), seed=seed)
    return model, eng, wrapped


def test_moe_expert_lora_trains_adapters_and_merges(tmp_path):
    """Per-expert adapters on gate / up / down of the stacked experts: only they train, the adapter
    path equals the merged weights, and the PEFT export has one pair per expert."""
    from xorl_b200.adapters.lora import ExpertsLoRA, merge_lora, save_lora_checkpoint
    from xorl_b200.optim import build_optimizer
    la = LoRAArguments(enable_lora=True, lora_rank=8, lora_alpha=16,
                       lora_target_modules=["q_proj", "gate_proj", "up_proj", "down_proj"])
    model, eng, wrapped = _moe_engine(la)
    assert any(n.endswith("mlp.experts") for n in wrapped), wrapped
    ex = model.layers["0"].mlp.experts
    assert isinstance(ex.lora, ExpertsLoRA) and ex.lora.gate_proj_lora_A.shape == (8, 128, 8)
    assert ex.lora.down_proj_lora_B.shape == (8, 8, 128) and not ex.gate_up_proj.requires_grad
    names = [n for g in eng.all_groups() if not getattr(g, "frozen", False) for n, _ in g.named_params]
    assert names and all("lora_" in n for n in names)
    assert any(n.endswith("experts.lora.up_proj_lora_B") for n in names)
    base = {n: t.clone() for n, t in eng.iter_full_tensors("master") if "lora_" not in n}
    opt = build_optimizer(eng, lr=1e-2, weight_decay=0.0)
    ids = torch.randint(0, 1024, (2, 65))
    losses = []
    for _ in range(6):
        opt.zero_grad()
        losses.append(float(eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)))
        eng.finish_grad_sync()
        _, coef = eng.grad_norm_and_clip_coef(1.0)
        opt.step(clip_coef=coef)
    assert losses[-1] < losses[0] - 0.02, losses
    for n, t in eng.iter_full_tensors("master"):
        if "lora_" not in n:
            assert torch.equal(t, base[n]), n
    b_norm = float(ex.lora.gate_proj_lora_B.float().norm())
    assert b_norm > 0                                       # the expert adapters did move
    save_lora_checkpoint(eng, str(tmp_path / "peft"), "tiny-moe")
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "peft" / "adapter_model.safetensors"))
    k = "base_model.model.model.layers.0.mlp.experts.3.gate_proj.lora_A.weight"
    assert k in sd and tuple(sd[k].shape) == (8, 128)
    assert tuple(sd["base_model.model.model.layers.1.mlp.experts.7.down_proj.lora_B.weight"].shape) == (128, 8)
    x, y = ids[:, :-1], ids[:, 1:]
    with torch.no_grad():
        before = float(model(x, labels=y, grad_scale=1.0 / 128)["loss"])
        assert merge_lora(model) >= 3                        # q_proj of two layers + two expert stacks
        after = float(model(x, labels=y, grad_scale=1.0 / 128)["loss"])
    assert abs(before - after) < 1e-4 and float(ex.lora.gate_proj_lora_B.abs().max()) == 0.0


def test_hybrid_shared_expert_lora(tmp_path):
    """``moe_hybrid_shared_lora``: gate / up share one A over the experts, down shares one B; the shared factors
    are dense parameters, the model learns, the adapter path equals the merged weights and the PEFT export
    writes the shared factor under every expert."""
    from xorl_b200.adapters.lora import merge_lora, save_lora_checkpoint
    from xorl_b200.optim import build_optimizer
    la = LoRAArguments(enable_lora=True, lora_rank=8, lora_alpha=16, moe_hybrid_shared_lora=True, lora_b_init_std=0.01,
                       lora_target_modules=["gate_proj", "up_proj", "down_proj"])
    model, eng, wrapped = _moe_engine(la)
    ex = model.layers["0"].mlp.experts
    assert ex.lora.gate_proj_lora_A.shape == (1, 128, 8) and ex.lora.gate_proj_lora_B.shape[0] == 8
    assert ex.lora.down_proj_lora_A.shape[0] == 8 and ex.lora.down_proj_lora_B.shape == (1, 8, 128)
    kinds = {n: g.name.rsplit(".", 1)[-1] for g in eng.all_groups() for n, _ in g.named_params if "lora" in n}
    assert kinds["layers.0.mlp.experts.lora.gate_proj_lora_A"] == "dense"
    assert kinds["layers.0.mlp.experts.lora.gate_proj_lora_B"] == "expert"
    assert kinds["layers.0.mlp.experts.lora.down_proj_lora_B"] == "dense"
    opt = build_optimizer(eng, lr=1e-2, weight_decay=0.0)
    ids = torch.randint(0, 1024, (2, 65))
    losses = []
    for _ in range(6):
        opt.zero_grad()
        losses.append(float(eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)))
        eng.finish_grad_sync()
        opt.step()
    assert losses[-1] < losses[0] - 0.02, losses
    save_lora_checkpoint(eng, str(tmp_path / "peft"), "tiny-moe")
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "peft" / "adapter_model.safetensors"))
    a0 = sd["base_model.model.model.layers.0.mlp.experts.0.gate_proj.lora_A.weight"]
    a5 = sd["base_model.model.model.layers.0.mlp.experts.5.gate_proj.lora_A.weight"]
    b0 = sd["base_model.model.model.layers.0.mlp.experts.0.gate_proj.lora_B.weight"]
    b5 = sd["base_model.model.model.layers.0.mlp.experts.5.gate_proj.lora_B.weight"]
    assert torch.equal(a0, a5) and not torch.equal(b0, b5) and tuple(a0.shape) == (8, 128)
    x, y = ids[:, :-1], ids[:, 1:]
    with torch.no_grad():
        before = float(model(x, labels=y, grad_scale=1.0 / 128)["loss"])
        merge_lora(model)
        after = float(model(x, labels=y, grad_scale=1.0 / 128)["loss"])
    assert abs(before - after) < 1e-4


def test_qlora_on_moe_experts_trains_and_loads_a_full_precision_checkpoint(tmp_path):
    """QLoRA over a MoE model: expert stacks are stored packed (4-bit) with per-expert adapters on top and
    the loss falls; a Hugging Face checkpoint of the full-precision model loads into the packed storage
    (quantised on the way in), adapters untouched."""
    from xorl_b200.adapters.qlora import PackedWeight, inject_qlora
    from xorl_b200.checkpoint.hf_io import load_hf_weights, save_hf_weights
    from xorl_b200.ops import quantize as Q
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    cfg = preset("tiny-qwen3-moe", tie_word_embeddings=False)
    # a full-precision model written as a Hugging Face checkpoint
    base = Zero3Engine(DecoderLM(cfg, device="meta"), ps, compute_dtype=torch.float32, device=torch.device("cpu"), seed=3)
    save_hf_weights(base, str(tmp_path / "hf"), cfg, dtype=torch.float32)
    full = {n: t.clone() for n, t in base.iter_full_tensors()}
    la = LoRAArguments(enable_lora=True, enable_qlora=True, lora_rank=4, quant_format="nf4", quant_group_size=64,
                       lora_b_init_std=0.01, lora_target_modules=["q_proj", "gate_proj", "up_proj", "down_proj"])
    model = DecoderLM(cfg, device="meta")
    wrapped = inject_qlora(model, la)
    assert any(n.endswith("experts") for n in wrapped)
    eng = Zero3Engine(model, ps, compute_dtype=torch.float32, device=torch.device("cpu"))
    names = [n for g in eng.all_groups() for n, _ in g.named_params]
    assert any(".experts.gate_up_proj_q.qparts.packed" in n for n in names)
    assert not any(n.endswith("experts.gate_up_proj") for n in names)          # no full-precision expert stack is kept
    assert any("experts.lora.gate_proj_lora_A" in n for n in names)
    missing = load_hf_weights(eng, str(tmp_path / "hf"), cfg)
    assert missing == []
    layer = next(m for m in model.modules() if isinstance(m, PackedWeight) and m.w_shape[2] == 2 * cfg.moe_intermediate_size)
    for u in eng.units:
        eng.gather(u)
        eng.wait_gather(u)
    src = next(t for n, t in full.items() if n.endswith("layers.0.mlp.experts.gate_up_proj"))
    want = Q.dequantize_weight(Q.quantize_weight(src.float(), "nf4", 64), "nf4", 64, src.shape, torch.float32)
    first = next(m for n, m in model.named_modules() if n.endswith("layers.0.mlp.experts.gate_up_proj_q"))
    assert torch.allclose(first.dequantized().float(), want, atol=1e-6)
    opt = build_optimizer(eng, lr=1e-2, weight_decay=0.0)
    ids = torch.randint(0, 1024, (2, 65))
    losses = []
    for _ in range(4):
        opt.zero_grad()
        losses.append(float(eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)))
        eng.finish_grad_sync()
        opt.step()
    assert losses[-1] < losses[0], losses
    reset_parallel_state()


def test_qarl_config_grids_and_scope():
    import pytest
    from xorl_b200.adapters import qarl
    assert qarl.normalize_quant_cfg(None)["format"] == "fp8_e4m3" and qarl.normalize_quant_cfg(None)["activation"]
    nv = qarl.normalize_quant_cfg("nvfp4")
    assert nv == {"format": "nvfp4", "weight": True, "activation": False, "dynamic": True, "group_size": 16}
    assert qarl.normalize_quant_cfg({"quant_method": "FP8_DEFAULT_CFG", "weight_block_size": [64, 128]})["weight_block_size"] == [64, 128]
    for bad in ({"format": "int3"}, {"format": "nvfp4", "group_size": 32}, {"dynamic": False}, {"blocks": 1},
                {"weight_block_size": [0, 128]}, 7):
        with pytest.raises(ValueError):
            qarl.normalize_quant_cfg(bad)
    assert qarl.unsupported_scope({"num_nextn_predict_layers": 1}) and qarl.unsupported_scope({"model_type": "Mamba2"})
    assert qarl.unsupported_scope(None, ["model.mtp_head.proj"]) and qarl.unsupported_scope({"model_type": "qwen3"}) is None
    # grids: values land on the grid, the gradient passes straight through
    torch.manual_seed(0)
    w = torch.randn(96, 160, requires_grad=True)
    fq, scales = qarl.fake_quant_fp8_blocks(w, (64, 128))
    assert scales.shape == (2, 2)
    again, _ = qarl.fake_quant_fp8_blocks(fq.detach(), (64, 128))
    assert torch.allclose(again, fq.detach(), rtol=0, atol=1e-6)           # already on the grid
    assert 0 < float((fq - w).detach().abs().max()) < 0.2
    fq.square().sum().backward()
    assert torch.allclose(w.grad, 2 * fq.detach())
    x = torch.randn(8, 160)
    xq, s = qarl.fake_quant_fp8_tensor(x)
    assert abs(float(s) - float(x.abs().max()) / 448.0) < 1e-9 and float((xq - x).abs().max()) < float(x.abs().max()) / 14
    e = torch.randn(3, 32, 20)                                              # [E, K, N]: groups along K
    eq = qarl.fake_quant_nvfp4(e, 16, dim=1)
    per_group = eq.transpose(1, 2).reshape(3, 20, 2, 16)
    assert all(len(torch.unique(per_group[i, j, g].abs())) <= 8 for i in range(3) for j in range(3) for g in range(2))


def test_qarl_trains_dense_fp8_and_moe_nvfp4(tmp_path):
    """Dense model on the fp8 grid (weights + activations) and a MoE model on the nvfp4 grid (linears and
    stacked experts): both learn, the masters stay full precision, the statistics fill up, calibration
    writes its summary and the sync configuration lists exactly the wrapped modules."""
    import json
    import pytest
    from xorl_b200.adapters import qarl
    from xorl_b200.arguments import TrainingArguments
    from xorl_b200.models.moe import Experts
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    ps = init_parallel_state(device_type="cpu")
    calib = tmp_path / "calib.jsonl"
    calib.write_text("\n".join(json.dumps({"input_ids": list(range(5 + i, 45 + i))}) for i in range(3)))
    for name, cfgq, n_experts in (("tiny-qwen3", None, 0), ("tiny-qwen3-moe", "nvfp4", 2)):
        ta = TrainingArguments(output_dir=str(tmp_path / name), enable_qarl=True, qarl_quant_cfg=cfgq,
                               qarl_exclude_modules=["o_proj"], device="cpu")
        model = DecoderLM(preset(name, tie_word_embeddings=False), device="meta")
        wrapped = qarl.inject_fake_quant(model, ta)
        assert wrapped and not any("o_proj" in w or "lm_head" in w or w.endswith(".gate") for w in wrapped)
        assert sum(isinstance(m, Experts) for m in model.modules()) == len(model._xb_qarl_config["experts"]) == n_experts
        eng = Zero3Engine(model, ps, compute_dtype=torch.float32, device=torch.device("cpu"))
        opt = build_optimizer(eng, lr=3e-3, weight_decay=0.0)
        summary = qarl.calibrate(lambda ids: eng.forward_only(ids), model, str(calib), size=2, sequence_length=32)
        assert summary["calibration_batches"] == 2 and summary["enabled"]
        assert all(v["forward_count"] == 2 and v["weight_amax"] > 0 for v in summary["modules"].values())
        ids = torch.randint(0, 1024, (2, 65))
        losses = []
        for _ in range(5):
            opt.zero_grad()
            losses.append(float(eng.forward_backward(ids[:, :-1], ids[:, 1:], grad_scale=1.0 / 128)))
            eng.finish_grad_sync()
            opt.step()
        assert losses[-1] < losses[0] - 0.05, (name, losses)
        full = dict(eng.iter_full_tensors("master"))
        some = next(v for k, v in full.items() if "q_proj" in k or "qkv_proj" in k)
        regrid = qarl.fake_quant(some, "nvfp4" if cfgq else "fp8")
        assert float((regrid - some).abs().max()) > 0                       # the masters are not on the grid
        sync = qarl.sync_quantization_config(model)
        assert sync["quant_method"] == ("nvfp4" if cfgq else "fp8")
        assert set(sync["qarl"]["folded_modules"]) == set(wrapped)
        assert any("o_proj" in m for m in sync["modules_to_not_convert"]) and "lm_head" in sync["modules_to_not_convert"]
        assert not set(sync["modules_to_not_convert"]) & set(wrapped)
    # fp8 on a MoE model is refused
    with pytest.raises(ValueError, match="nvfp4"):
        qarl.inject_fake_quant(DecoderLM(preset("tiny-qwen3-moe"), device="meta"),
                               TrainingArguments(output_dir=str(tmp_path / "x"), enable_qarl=True, device="cpu"))
    reset_parallel_state()


def test_lora_target_manifest_pins_the_adapter_coverage(tmp_path):
    import json
    import pytest
    from xorl_b200.adapters import target_manifest as tm
    from xorl_b200.adapters.lora import inject_lora
    cfg = preset("tiny-qwen3", tie_word_embeddings=False)
    L = cfg.num_hidden_layers
    good = {"schema_version": 1, "target_modules": ["q_proj", "v_proj", "down_proj"],
            "expected_modules": [{"pattern": "model.layers.*.self_attn.q_proj", "count": L, "rank": 4},
                                 {"pattern": "model.layers.*.self_attn.v_proj", "count": L},
                                 {"pattern": "model.layers.*.mlp.down_proj", "count": L, "rank": 4}]}
    path = tmp_path / "manifest.json"
    path.write_text(json.dumps(good))
    la = LoRAArguments(enable_lora=True, lora_rank=4, lora_target_manifest=str(path))
    model = DecoderLM(cfg, device="meta")
    inject_lora(model, la)                                     # targets come from the manifest; coverage matches
    units = tm.adapter_units(model)
    assert len(units) == 3 * L and units["model.layers.0.self_attn.q_proj"] == 4
    assert not any("k_proj" in u for u in units)               # the fused qkv projection adapts two of its three slices
    # every kind of mismatch is reported
    bad = json.loads(json.dumps(good))
    bad["expected_modules"][0]["count"] = L + 1
    bad["expected_modules"][1]["rank"] = 8
    bad["expected_modules"].pop(2)
    with pytest.raises(ValueError) as e:
        tm.validate(model, bad)
    msg = str(e.value)
    assert "expects %d" % (L + 1) in msg and "rank 8 expected" in msg and "no pattern lists" in msg
    bad["allow_unlisted"] = True
    bad["expected_modules"] = [{"pattern": "model.layers.*", "count": 3 * L}, {"pattern": "*.q_proj", "count": L}]
    with pytest.raises(ValueError, match="earlier pattern"):
        tm.validate(model, bad)
    # configured leaves that disagree with the manifest, and malformed manifests
    with pytest.raises(ValueError, match="differ"):
        inject_lora(DecoderLM(cfg, device="meta"), LoRAArguments(enable_lora=True, lora_rank=4, lora_target_modules=["q_proj"],
                                                                 lora_target_manifest=good))
    for broken in ({**good, "schema_version": 2}, {**good, "target_modules": []}, {**good, "allow_unlisted": "no"},
                   {**good, "expected_modules": [{"pattern": "x", "count": -1}]}):
        with pytest.raises(ValueError):
            tm.load_manifest(broken)
    # a MoE model: the stacked experts are one unit per layer
    moe = DecoderLM(preset("tiny-qwen3-moe"), device="meta")
    inject_lora(moe, LoRAArguments(enable_lora=True, lora_rank=4, lora_target_modules=["gate_proj", "up_proj", "down_proj"]))
    assert sum(u.endswith(".mlp.experts") for u in tm.adapter_units(moe)) > 0


def test_adaptive_quantisation_noise_has_the_size_of_the_grid_and_is_off_outside_training():
    """``lora.enable_aqn``: training forwards see base weights jittered by ``aqn_alpha * N(0, 1) * step`` with the
    step taken from the stored scales; evaluation and no-grad passes see the plain dequantised weights."""
    from xorl_b200.adapters.qlora import QLoRALinear
    from xorl_b200.models.layers import Linear
    from xorl_b200.ops import quantize as Q
    torch.manual_seed(0)
    for fmt, group in (("nf4", 64), ("nvfp4", 16), ("block_fp8", 128), ("int4", 128), ("mxfp4", 32)):
        base = Linear(256, 128, dtype=torch.float32)
        q = QLoRALinear(base, 4, 8, [("x_proj", 0, 128)], fmt, group)
        w = torch.randn(128, 256) * 0.05
        for p in q.parameters():
            if p.is_meta or p.numel() == 0:
                continue
        torch.nn.init.zeros_(q.lora_B["x_proj"])
        torch.nn.init.normal_(q.lora_A["x_proj"], 0, 0.02)
        q.load_base_weight(w)
        step = q.quantisation_step()
        deq = q.dequantized_weight().float()
        assert step.shape == (128, 256) and float(step.min()) >= 0
        err = (deq - w).abs()
        if fmt == "block_fp8":
            # the spacing of e4m3 around one, in the block's scale: a floor (larger codes are spaced wider)
            assert abs(float(step.max()) - 0.125 * float(w.abs().max()) / 448.0) < 1e-9
            assert float(err.mean()) > float(step.mean())
        else:
            # 4-bit grids: the step is of the order of the rounding error the format makes
            assert float(err.mean()) < 2.5 * float(step.mean()) and float(step.mean()) < 40 * float(err.mean()), \
                (fmt, float(err.mean()), float(step.mean()))
        x = torch.eye(256)
        q.enable_aqn, q.aqn_alpha = True, 0.5
        q.train()
        noisy = q(x).t()                                        # = jittered weight (B = 0)
        ratio = ((noisy.detach() - deq) / step.clamp_min(1e-12))[step > 0]
        assert abs(float(ratio.std()) - 0.5) < 0.03 and abs(float(ratio.mean())) < 0.02, (fmt, float(ratio.std()))
        assert not torch.equal(q(x), q(x))                      # fresh noise every forward
        with torch.no_grad():
            assert torch.equal(q(x).t(), deq)
        q.eval()
        assert torch.equal(q(x).t(), deq)


def test_fp8_module_overrides_choose_the_backward_precision_per_module():
    import pytest
    from xorl_b200.adapters.fp8 import FP8Linear, inject_fp8_training
    from xorl_b200.arguments import TrainingArguments
    ta = TrainingArguments(output_dir="o", device="cpu", enable_fp8_training=True, fp8_training_allow_blackwell=True,
                           fp8_training_backward="fp8",
                           fp8_training_module_overrides={"*.self_attn.o_proj": {"backward_mode": "bf16"},
                                                          "down_proj": {"backward_mode": "bf16", "block_size": 128}})
    model = DecoderLM(preset("tiny-qwen3", tie_word_embeddings=False), device="meta")
    inject_fp8_training(model, ta)
    modes = {n: m.fp8_backward for n, m in model.named_modules() if isinstance(m, FP8Linear)}
    assert modes and all(v == (not (n.endswith("o_proj") or n.endswith("down_proj"))) for n, v in modes.items()), modes
    ta.fp8_training_module_overrides = {"q*": {"smoothquant_alpha": 0.5}}
    with pytest.raises(NotImplementedError, match="smoothquant_alpha"):
        inject_fp8_training(DecoderLM(preset("tiny-qwen3"), device="meta"), ta)
