"""Feature paths on the GPU in bf16, each against the same run in fp32 on the host: LoRA and QLoRA (dense
and MoE experts), the training service's runner (token losses, filtered log-probabilities, multi-tenant
adapters with the reference pass), trainer-side distillation with the streaming KL."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
pytestmark = pytest.mark.gpu


def _adapter_curve(device, dtype, preset_name, fmt, steps=6):
    from xorl_b200.arguments import LoRAArguments
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import get_parallel_state, init_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    init_parallel_state(device_type=device.type)
    cfg = preset(preset_name, tie_word_embeddings=False)
    la = LoRAArguments(enable_lora=True, enable_qlora=fmt is not None, lora_rank=8, lora_alpha=16,
                       quant_format=fmt or "nf4", quant_group_size={"nvfp4": 16, "nf4": 64, None: 64}[fmt],
                       lora_b_init_std=0.01, lora_target_modules=["q_proj", "v_proj", "gate_proj", "up_proj", "down_proj"])
    model = DecoderLM(cfg, dtype=dtype, device="meta")
    if fmt is None:
        from xorl_b200.adapters.lora import inject_lora
        inject_lora(model, la)
    else:
        from xorl_b200.adapters.qlora import inject_qlora
        inject_qlora(model, la)
    eng = Zero3Engine(model, get_parallel_state(), compute_dtype=dtype, device=device, seed=0)
    opt = build_optimizer(eng, lr=5e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (1, 257), generator=g)
    x, y = ids[:, :-1].clone().to(device), ids[:, 1:].clone().to(device)
    cu = torch.tensor([0, 96, 256], dtype=torch.int32, device=device)
    pos = torch.cat([torch.arange(96), torch.arange(160)]).unsqueeze(0).to(device)
    out = []
    for _ in range(steps):
        opt.zero_grad()
        out.append(float(eng.forward_backward(x, y, position_ids=pos, cu_seqlens=cu, grad_scale=1.0 / 256)))
        eng.finish_grad_sync()
        opt.step()
    reset_parallel_state()
    return out


@pytest.mark.parametrize("preset_name,fmt", [("tiny-qwen3", None), ("tiny-qwen3", "nf4"), ("tiny-qwen3", "nvfp4"),
                                             ("tiny-qwen3-moe", None), ("tiny-qwen3-moe", "nf4")])
def test_lora_and_qlora_train_on_the_gpu(preset_name, fmt):
    from xorl_b200.ops import _lib
    got = _adapter_curve(torch.device("cuda", 0), torch.bfloat16, preset_name, fmt)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    ref = _adapter_curve(torch.device("cpu"), torch.float32, preset_name, fmt)
    assert all(math.isfinite(l) for l in got) and got[-1] < got[0], got
    for i, (a, b) in enumerate(zip(got, ref)):
        assert abs(a - b) < 0.04 * abs(b) + 0.04, (preset_name, fmt, i, got, ref)


def _runner(tmp, device, preset="tiny-qwen3", **kw):
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    sa = ServerArguments(model_preset=preset, output_dir=str(tmp), device=device, sample_packing_sequence_len=256,
                         enable_mixed_precision=device != "cpu", **kw)
    return ModelRunner(Trainer(sa.to_trainer_arguments()))


def test_service_runner_on_the_gpu(tmp_path):
    from xorl_b200.ops import _lib
    from xorl_b200.parallel.state import reset_parallel_state
    data = [{"tokens": list(range(3 + i, 90 + 2 * i))} for i in range(3)]
    res = {}
    for dev in ("cuda", "cpu"):
        r = _runner(tmp_path / dev, dev, enable_lora=True, lora_rank=8, lora_alpha=16)
        base = r.forward("default", data, None)["logprobs"]
        r.create_model("a")
        for _ in range(3):
            fb = r.forward_backward("a", data, None)
            r.optim_step("a", adam_params={"learning_rate": 5e-3})
        after = r.forward("a", data, None)["logprobs"]
        ref = r.forward("a", data, None, loss_fn_config={"reference": True})["logprobs"]
        filt = r.forward("a", data, None, loss_fn_config={"top_k": 600, "temperature": 0.8})
        res[dev] = dict(base=base, after=after, ref=ref, loss=fb["loss"], filt=filt["logprobs"])
        reset_parallel_state()
    torch.cuda.synchronize()
    _lib.raise_on_status()
    g, h = res["cuda"], res["cpu"]
    flat = lambda xs: [v for x in xs for v in x]
    close = lambda a, b, tol: max(abs(p - q) for p, q in zip(flat(a), flat(b))) < tol
    assert close(g["ref"], g["base"], 1e-6)                       # the reference pass is the untouched base model
    assert not close(g["after"], g["base"], 1e-3)                 # the adapter has learned something
    assert close(g["base"], h["base"], 0.08) and close(g["after"], h["after"], 0.12)     # bf16 against fp32
    assert abs(g["loss"] - h["loss"]) < 0.03 * abs(h["loss"])
    in_support = [(p, q) for p, q in zip(flat(g["filt"]), flat(h["filt"])) if p > -1e29 and q > -1e29]
    assert len(in_support) > 50 and max(abs(p - q) for p, q in in_support) < 0.15


def test_distillation_step_on_the_gpu(tmp_path):
    """The streaming KL of the head loss through the tcgen05 GEMM (fp32 logits) against the host."""
    from xorl_b200.ops import kl_losses as K
    torch.manual_seed(0)
    N, H, V = 384, 256, 4096
    hs = (torch.randn(N, H) * 0.5)
    ht = (torch.randn(N, H) * 0.5)
    ws, wt = torch.randn(V, H) * 0.05, torch.randn(V, H) * 0.05
    lab = torch.randint(0, V, (N,))
    lab[::7] = -100
    for kind in K.KINDS:
        a = [t.cuda().bfloat16().requires_grad_() for t in (hs, ws)]
        out = K.streaming_kl(a[0], a[1], ht.cuda().bfloat16(), wt.cuda().bfloat16(), lab.cuda(), kind, vocab_chunk=1024)
        out.sum().backward()
        b = [t.bfloat16().float().requires_grad_() for t in (hs, ws)]
        ref = K.streaming_kl(b[0], b[1], ht.bfloat16().float(), wt.bfloat16().float(), lab, kind, vocab_chunk=1024)
        ref.sum().backward()
        assert torch.allclose(out.cpu(), ref, atol=2e-3, rtol=2e-2), (kind, (out.cpu() - ref).abs().max())
        assert (a[0].grad.float().cpu() - b[0].grad).abs().max() < 0.03 * b[0].grad.abs().max() + 1e-4
        assert (a[1].grad.float().cpu() - b[1].grad).abs().max() < 0.03 * b[1].grad.abs().max() + 1e-4


def _optimizer_curve(device, dtype, optimizer, lr, steps=6):
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import get_parallel_state, init_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    init_parallel_state(device_type=device.type)
    cfg = preset("tiny-qwen3", tie_word_embeddings=False)
    eng = Zero3Engine(DecoderLM(cfg, dtype=dtype, device="meta"), get_parallel_state(), compute_dtype=dtype,
                      device=device, seed=0)
    opt = build_optimizer(eng, lr=lr, weight_decay=0.01, optimizer_type=optimizer,
                          optimizer_kwargs={"muon_lr": 0.01} if optimizer == "muon" else None)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (1, 257), generator=g)
    x, y = ids[:, :-1].clone().to(device), ids[:, 1:].clone().to(device)
    cu = torch.tensor([0, 128, 256], dtype=torch.int32, device=device)
    pos = torch.cat([torch.arange(128), torch.arange(128)]).unsqueeze(0).to(device)
    out = []
    for _ in range(steps):
        opt.zero_grad()
        out.append(float(eng.forward_backward(x, y, position_ids=pos, cu_seqlens=cu, grad_scale=1.0 / 256)))
        eng.finish_grad_sync()
        _, coef = eng.grad_norm_and_clip_coef(1.0)
        opt.step(clip_coef=coef)
    reset_parallel_state()
    return out


@pytest.mark.parametrize("optimizer,lr", [("adamw", 2e-3), ("anyprecision_adamw", 2e-3), ("sgd", 0.5), ("signsgd", 2e-4),
                                          ("muon", 2e-3)])
def test_optimizers_on_the_gpu_follow_the_host_curve(optimizer, lr):
    """Every optimizer's device kernels (csrc/optim.cu, Newton-Schulz on the tcgen05 GEMM) with gradient
    clipping, against the same optimizer's tensor-op form in fp32 on the host."""
    from xorl_b200.ops import _lib
    got = _optimizer_curve(torch.device("cuda", 0), torch.bfloat16, optimizer, lr)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    ref = _optimizer_curve(torch.device("cpu"), torch.float32, optimizer, lr)
    assert all(math.isfinite(l) for l in got) and got[-1] < got[0], (optimizer, got)
    for i, (a, b) in enumerate(zip(got, ref)):
        assert abs(a - b) < 0.06 * abs(b) + 0.06, (optimizer, i, got, ref)
