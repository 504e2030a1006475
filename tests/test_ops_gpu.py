"""Each CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol, atol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).float().mean().item()
    assert bad < 1e-3, f"{what}: {bad:.4%} elements out of tolerance, max err {err.max().item():.4g}"


@pytest.mark.parametrize("T,H", [(64, 256), (1000, 4096), (33, 5120), (17, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(T, H, with_res):
    from xorl_b200.ops.norm import rmsnorm
    torch.manual_seed(0)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    gy = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    gh = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    if with_res:
        y, h = rmsnorm(x, w, 1e-6, residual=r)
        (y.float() * gy.float()).sum().add((h.float() * gh.float()).sum()).backward()
    else:
        y = rmsnorm(x, w, 1e-6)
        (y.float() * gy.float()).sum().backward()
    # fp32 reference
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    hr = xr + rr if with_res else xr
    if with_res:
        hr = hr + (hr.to(torch.bfloat16).float() - hr).detach()  # residual stream is stored in bf16
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    lossr = (yr * gy.float()).sum()
    if with_res:
        lossr = lossr + (hr * gh.float()).sum()
    lossr.backward()
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(x.grad, xr.grad, 3e-2, 3e-2, "dx")
    _close(w.grad, wr.grad, 3e-2, 0.05 * wr.grad.abs().max().item(), "dw")
    if with_res:
        _close(r.grad, rr.grad, 3e-2, 3e-2, "dres")


@pytest.mark.parametrize("T,I", [(77, 768), (512, 12288)])
def test_swiglu(T, I):
    from xorl_b200.ops.activation import swiglu
    torch.manual_seed(0)
    gu = torch.randn(T, 2 * I, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(T, I, device=DEV, dtype=torch.bfloat16)
    out = swiglu(gu)
    out.backward(go)
    gr = gu.detach().float().requires_grad_()
    ref = torch.nn.functional.silu(gr[:, :I]) * gr[:, I:]
    ref.backward(go.float())
    _close(out, ref, 2e-2, 2e-2, "out")
    _close(gu.grad, gr.grad, 2e-2, 2e-2, "dgu")


@pytest.mark.parametrize("rows,V", [(64, 1024), (130, 151936), (16, 32003)])
def test_cross_entropy_chunk(rows, V):
    from xorl_b200.ops.loss import ce_chunk_
    torch.manual_seed(0)
    ldv = (V + 7) // 8 * 8
    buf = torch.randn(rows, ldv, device=DEV, dtype=torch.bfloat16) * 3
    logits = buf[:, :V]
    labels = torch.randint(0, V, (rows,), device=DEV)
    labels[::7] = -100
    lr = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr, labels, ignore_index=-100, reduction="none")
    (ref.sum() * 0.5).backward()
    loss, lse = ce_chunk_(logits, labels, 0.5, True)
    _close(loss, ref, 1e-3, 1e-3, "loss")
    _close(logits, lr.grad, 2e-2, 1e-4, "dlogits")


def test_fused_linear_ce():
    from xorl_b200.ops.loss import fused_linear_cross_entropy
    torch.manual_seed(0)
    T, H, V = 300, 256, 5000
    h = (torch.randn(T, H, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, H, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[:5] = -100
    loss = fused_linear_cross_entropy(h, w, labels, grad_scale=1.0 / T, chunk_tokens=128)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(hr @ wr.t(), labels, ignore_index=-100, reduction="sum") / T
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    _close(h.grad, hr.grad, 5e-2, 0.03 * hr.grad.abs().max().item(), "dh")
    _close(w.grad, wr.grad, 5e-2, 0.03 * wr.grad.abs().max().item(), "dw")


def test_embedding():
    from xorl_b200.ops.embedding import embedding
    torch.manual_seed(0)
    V, H, T = 1000, 256, 513
    table = torch.randn(V, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (T,), device=DEV)
    go = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    out = embedding(ids, table)
    out.backward(go)
    tr = table.detach().float().requires_grad_()
    ref = torch.nn.functional.embedding(ids, tr)
    ref.backward(go.float())
    assert torch.equal(out.float(), ref)
    _close(table.grad, tr.grad, 2e-2, 2e-2, "dtable")


def test_adamw_and_norm():
    from xorl_b200.ops import optim
    torch.manual_seed(0)
    n = 1_000_003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 0.1
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    pr = p.clone().requires_grad_()
    opt = torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    bf = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        pr.grad = g.clone()
        opt.step()
        optim.adamw_step_(p, m, v, g, bf, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                          weight_decay=0.01, step=step)
    assert torch.allclose(p, pr.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(bf, p.to(torch.bfloat16))
    tot = torch.zeros(1, device=DEV)
    optim.sumsq_(g, tot, False)
    assert abs(tot.item() - g.double().pow(2).sum().item()) < 1e-3 * tot.item()
    norm = torch.zeros(1, device=DEV)
    coef = torch.zeros(1, device=DEV)
    optim.clip_coef_(tot, 1.0, norm, coef)
    assert abs(norm.item() - math.sqrt(tot.item())) < 1e-3
    assert abs(coef.item() - min(1.0, 1.0 / (norm.item() + 1e-6))) < 1e-5


def _make_cu(lens):
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    return torch.tensor(cu, device=DEV, dtype=torch.int32)


@pytest.fixture(params=["split", "fused"])
def bwd_mode(request):
    from xorl_b200.ops import _lib, attention
    prev = attention.set_backward_mode(request.param)
    yield request.param
    attention.set_backward_mode(prev)
    assert all(v == 0 for v in _lib.read_status()[:4])


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [
    ([128], 2, 1, True), ([256], 4, 2, True), ([200, 56, 384], 4, 1, True), ([1000], 8, 2, True),
    ([300, 100], 2, 2, False), ([4096], 8, 2, True), ([1, 63, 65, 129, 700], 4, 2, True)])
def test_flash_attention_fwd_bwd(lens, Hq, Hkv, causal, bwd_mode):
    from xorl_b200.ops.attention import attention_reference, flash_attn_varlen
    torch.manual_seed(0)
    D = 128
    T = sum(lens)
    cu = _make_cu(lens)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    out = flash_attn_varlen(q, k, v, cu, causal=causal)
    out.backward(go)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, cu, causal=causal)
    ref.backward(go.float())
    _close(out, ref, 2e-2, 2e-2, "out")
    _close(v.grad, vr.grad, 3e-2, 0.02 * vr.grad.abs().max().item(), "dv")
    _close(k.grad, kr.grad, 3e-2, 0.02 * kr.grad.abs().max().item(), "dk")
    _close(q.grad, qr.grad, 3e-2, 0.02 * qr.grad.abs().max().item(), "dq")


@pytest.mark.parametrize("lens,Hq,Hkv,D,window,sinks", [
    ([333, 691], 4, 2, 128, 128, False),      # window = one tile; documents that end inside a tile
    ([1024], 2, 2, 128, 200, False),          # window that straddles tiles
    ([700, 100], 4, 1, 128, 8, False),        # window far below the tile size
    ([515], 2, 1, 128, 4096, False),          # window longer than the document: plain causal
    ([333, 691], 4, 2, 128, 0, True),         # sink logits only
    ([300, 212, 512], 8, 2, 64, 128, True),   # gpt-oss layer: 64-wide heads, window and sinks
])
def test_flash_attention_window_sinks_head_dim(lens, Hq, Hkv, D, window, sinks):
    from xorl_b200.ops import attention as A
    torch.manual_seed(0)
    T = sum(lens)
    cu = _make_cu(lens)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    sk = (torch.randn(Hq, device=DEV) * 2).to(torch.bfloat16).requires_grad_() if sinks else None
    go = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    before = A.launch_count()
    out = A.flash_attn_varlen(q, k, v, cu, causal=True, window=window or None, sinks=sk)
    out.backward(go)
    assert A.launch_count() - before == 4, "the tcgen05 kernels must serve windows, sinks and 64-wide heads"
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    skr = sk.detach().float().requires_grad_() if sinks else None
    ref = A.attention_reference(qr, kr, vr, cu, causal=True, window=window or None, sinks=skr)
    ref.backward(go.float())
    _close(out, ref, 2e-2, 2e-2, "out")
    _close(v.grad, vr.grad, 3e-2, 0.02 * vr.grad.abs().max().item(), "dv")
    _close(k.grad, kr.grad, 3e-2, 0.02 * kr.grad.abs().max().item(), "dk")
    _close(q.grad, qr.grad, 3e-2, 0.02 * qr.grad.abs().max().item(), "dq")
    if sinks:
        _close(sk.grad, skr.grad, 3e-2, 0.03 * skr.grad.abs().max().item(), "dsinks")


@pytest.mark.parametrize("do_norm", [True, False])
def test_qk_norm_rope_attention(do_norm):
    from xorl_b200.ops.attention import (qk_norm_rope_attention,
                                         qk_norm_rope_attention_reference)
    torch.manual_seed(0)
    Hq, Hkv, D = 4, 2, 128
    lens = [300, 212]
    T = sum(lens)
    cu = _make_cu(lens)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    wq = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_() if do_norm else None
    wk = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_() if do_norm else None
    pos = torch.cat([torch.arange(l, device=DEV) for l in lens]).float()
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    go = torch.randn(T, Hq * D, device=DEV, dtype=torch.bfloat16)
    out = qk_norm_rope_attention(qkv, wq, wk, cos, sin, cu, Hq, Hkv, D)
    out.backward(go)
    qkvr = qkv.detach().float().requires_grad_()
    wqr = wq.detach().float().requires_grad_() if do_norm else None
    wkr = wk.detach().float().requires_grad_() if do_norm else None
    ref = qk_norm_rope_attention_reference(qkvr, wqr, wkr, cos, sin, cu, Hq, Hkv, D, 1e-6, True,
                                           1.0 / math.sqrt(D))
    ref.backward(go.float())
    _close(out, ref, 3e-2, 3e-2, "out")
    _close(qkv.grad, qkvr.grad, 5e-2, 0.03 * qkvr.grad.abs().max().item(), "dqkv")
    if do_norm:
        _close(wq.grad, wqr.grad, 5e-2, 0.05 * wqr.grad.abs().max().item(), "dwq")
        _close(wk.grad, wkr.grad, 5e-2, 0.05 * wkr.grad.abs().max().item(), "dwk")


def test_status_words_clean():
    from xorl_b200.ops import _lib
    assert _lib.read_status()[0] == 0


@pytest.mark.parametrize("E,K,N,counts", [(4, 256, 512, [100, 0, 300, 129]), (16, 2048, 1536, None),
                                          (8, 768, 2048, None)])
def test_grouped_linear_fwd_bwd(E, K, N, counts):
    from xorl_b200.ops import moe as moe_ops
    torch.manual_seed(0)
    if counts is None:
        counts = torch.randint(0, 700, (E,)).tolist()
    ids = torch.repeat_interleave(torch.arange(E), torch.tensor(counts)).to(DEV)
    S = ids.numel()
    dest, seg, _ = moe_ops.aligned_sort_indices(ids, E)
    rows = moe_ops.buffer_rows(S, E)
    xs = (torch.randn(S, K, device=DEV) * 0.5).to(torch.bfloat16)
    buf = torch.zeros(rows, K, device=DEV, dtype=torch.bfloat16).index_copy(0, dest, xs).requires_grad_()
    w = (torch.randn(E, K, N, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    go_s = torch.randn(S, N, device=DEV, dtype=torch.bfloat16)
    go = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16).index_copy(0, dest, go_s)
    y = moe_ops.grouped_linear(buf, w, seg)
    y.backward(go)
    # fp32 reference per expert
    xr = buf.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    s = seg.tolist()
    yr = torch.zeros(rows, N, device=DEV)
    parts = []
    for e in range(E):
        parts.append(xr[s[e]:s[e + 1]] @ wr[e])
    yr = torch.cat(parts + [torch.zeros(rows - s[E], N, device=DEV)], 0)
    yr.backward(go.float())
    _close(y, yr, 2e-2, 0.02 * yr.abs().max().item(), "y")
    _close(buf.grad, xr.grad, 3e-2, 0.02 * xr.grad.abs().max().item(), "dx")
    _close(w.grad, wr.grad, 3e-2, 0.02 * wr.grad.abs().max().item(), "dw")


def test_moe_block_gpu_matches_reference():
    from xorl_b200.models.config import preset
    from xorl_b200.models.context import StepContext
    from xorl_b200.models.moe import MoEBlock
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cuda")
    cfg = preset("qwen3-30b-a3b", hidden_size=512, num_experts=16, num_experts_per_tok=4,
                 moe_intermediate_size=256, num_hidden_layers=1)
    torch.manual_seed(0)
    blk = MoEBlock(cfg, 0, dtype=torch.bfloat16, device=DEV)
    for p in blk.parameters():
        torch.nn.init.normal_(p, 0, 0.05)
    T = 777
    x = (torch.randn(T, 512, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    ctx = StepContext(cu_seqlens=torch.tensor([0, T], device=DEV, dtype=torch.int32),
                      position_ids=torch.arange(T, device=DEV))
    out = blk(x, ctx)
    go = torch.randn_like(out)
    out.backward(go)
    w, idx, _ = blk.gate(x.detach())
    xr = x.detach().float()
    ref = torch.zeros(T, 512, device=DEV)
    gu, dn = blk.experts.gate_up_proj.detach().float(), blk.experts.down_proj.detach().float()
    for e in range(16):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xr[tok] @ gu[e]
        a = torch.nn.functional.silu(h[:, :256]) * h[:, 256:]
        ref.index_add_(0, tok, (a @ dn[e]) * w[tok, slot].unsqueeze(-1))
    _close(out, ref, 3e-2, 0.03 * ref.abs().max().item(), "moe out")
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()
    assert torch.isfinite(blk.experts.gate_up_proj.grad.float()).all()
