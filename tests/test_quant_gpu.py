"""fp8 block-scaled GEMM and quantisation kernels, token-loss head and Muon GEMM path on a B200,
each against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from xorl_b200.ops import _lib
    _lib.cuda_lib()          # fail loudly if the native library is missing on a GPU box
    yield
    assert all(v == 0 for v in _lib.read_status()[:4]), _lib.read_status()


@pytest.mark.parametrize("M,K", [(256, 512), (1000, 1024), (3, 128)])
def test_quant_rows_matches_reference(M, K):
    from xorl_b200.ops import fp8_gemm, quantize as Q
    torch.manual_seed(M + K)
    x = (torch.randn(M, K, device="cuda") * 3).bfloat16()
    q, s = fp8_gemm.quantize_rows(x)
    q_ref, s_ref = Q.block_fp8_quantize_1x128(x)
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    # a value on a rounding boundary may fall either way: compare after dequantisation
    d, d_ref = q.float() * s.repeat_interleave(128, 1), q_ref.float() * s_ref.repeat_interleave(128, 1)
    assert (d - d_ref).abs().max() <= 0.07 * x.float().abs().max()
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 3e-3
    assert (d - x.float()).abs().max() <= 0.07 * x.float().abs().max()


@pytest.mark.parametrize("N,K", [(256, 384), (300, 200)])
def test_quant_blocks_roundtrip(N, K):
    from xorl_b200.ops import fp8_gemm, quantize as Q
    torch.manual_seed(N + K)
    w = torch.randn(N, K, device="cuda").bfloat16()
    q, s = fp8_gemm.quantize_blocks(w)
    q_ref, s_ref = Q.block_fp8_quantize_128x128(w)
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    # x * (1 / scale) against x / scale: values on a rounding boundary may fall either way
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 3e-3
    back = fp8_gemm.dequantize_blocks(q, s)
    ref = Q.block_fp8_dequantize_128x128(q, s)
    torch.testing.assert_close(back.float(), ref.float(), rtol=0, atol=0)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 1024), (1000, 200, 512), (4096, 4096, 4096)])
def test_block_fp8_gemm_matches_fp32_reference(M, N, K):
    from xorl_b200.ops import fp8_gemm, quantize as Q
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").bfloat16()
    # give K blocks very different magnitudes so a wrong scale index cannot hide
    a = a * (1 + torch.arange(K // 128, device="cuda").repeat_interleave(128)).bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16() * 0.05
    aq, as_ = fp8_gemm.quantize_rows(a)
    bq, bs = fp8_gemm.quantize_blocks(b)
    out = fp8_gemm.block_fp8_gemm(aq, as_, bq, bs)
    ref = Q.block_fp8_gemm_reference(aq, as_, bq, bs, out_dtype=torch.float32)
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert err < 1e-2, err                                    # bf16 output rounding only
    dense = a.float() @ b.float().t()
    assert (out.float() - dense).norm() / dense.norm() < 0.06  # fp8 quantisation noise


@pytest.mark.parametrize("shape", [(512, 256, 384), (200, 320, 200)])
def test_fp8_linear_training_step(shape):
    """Forward and input-gradient GEMMs on e4m3 operands (cached weight codes, transposed for dgrad), weight
    gradient in bf16; sizes that are not multiples of 128 are padded."""
    from xorl_b200.adapters.fp8 import _FP8LinearFn
    from xorl_b200.ops import fp8_grouped
    M, K, N = shape
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    g = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    for fp8_backward in (True, False):
        x.grad = w.grad = None
        y = _FP8LinearFn.apply(x, w, fp8_backward)
        y.backward(g)
        ref = x.detach().float() @ w.detach().float().t()
        dx_ref = g.float() @ w.detach().float()
        dw_ref = g.float().t() @ x.detach().float()
        assert (y.float() - ref).norm() / ref.norm() < 0.06
        assert (x.grad.float() - dx_ref).norm() / dx_ref.norm() < (0.06 if fp8_backward else 0.01)
        assert (w.grad.float() - dw_ref).norm() / dw_ref.norm() < 0.01
    cache = w._xb_fp8_cache
    _FP8LinearFn.apply(x, w, True)
    assert w._xb_fp8_cache is cache                           # weights unchanged: codes reused
    fp8_grouped.invalidate_weight_cache()
    _FP8LinearFn.apply(x, w, True)
    assert w._xb_fp8_cache is not cache


def test_token_loss_head_matches_autograd():
    from xorl_b200.ops import rl_losses
    from xorl_b200.ops.loss import fused_linear_token_loss
    torch.manual_seed(0)
    T, H, V = 700, 256, 1000
    h = (torch.randn(T, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.05).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    old = torch.full((T,), -6.5, device="cuda")
    adv = torch.randn(T, device="cuda")
    fn = lambda lp, mask: rl_losses.importance_sampling(lp, mask, old_logprobs=old, advantages=adv)
    loss, lp, _ = fused_linear_token_loss(h, w, labels, fn, 1.0, chunk_tokens=256)
    loss.backward()
    h32 = h.detach().float().requires_grad_()
    w32 = w.detach().float().requires_grad_()
    logits = h32 @ w32.t()
    lp_ref = -torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100, reduction="none")
    loss_ref, _ = fn(lp_ref, (labels != -100).float())
    loss_ref.backward()
    torch.testing.assert_close(lp, lp_ref.detach(), rtol=2e-2, atol=3e-2)
    assert abs(loss.item() - loss_ref.item()) < 2e-2 * max(1.0, abs(loss_ref.item()))
    assert (h.grad.float() - h32.grad).norm() / h32.grad.norm() < 3e-2
    assert (w.grad.float() - w32.grad).norm() / w32.grad.norm() < 3e-2


def test_muon_newton_schulz_on_tcgen05_gemm():
    from xorl_b200.optim.muon import gram_newton_schulz, newton_schulz
    torch.manual_seed(0)
    G = torch.randn(256, 1024, device="cuda")
    X = newton_schulz(G).float()
    Y = gram_newton_schulz(G).float()
    Xc = newton_schulz(G.cpu()).float()
    sv = torch.linalg.svdvals(X)
    assert sv.min() > 0.5 and sv.max() < 1.3
    assert (X.cpu() - Xc).norm() / Xc.norm() < 0.05
    assert (X - Y).norm() / X.norm() < 0.06


@pytest.mark.parametrize("M,K,block,dt", [(2048, 512, 512, torch.bfloat16), (1000, 256, 256, torch.float32),
                                          (2304, 1024, 1024, torch.bfloat16)])
def test_symmetric_gemm_matches_full_product(M, K, block, dt):
    """Lower panels through the GEMM kernel + mirror kernel against the full product and fp32."""
    from xorl_b200.ops import gemm as G
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
    before = G.launch_count()
    c = G.gemm_symmetric(x, out_dtype=dt, block=block, min_rows=0)
    panels = -(-M // block)
    assert G.launch_count() == before + panels + 1
    full = G.gemm(x, x, out_dtype=dt)
    low = torch.tril(torch.ones(M, M, device="cuda", dtype=torch.bool))
    assert (c[low].float() - full[low].float()).abs().max() <= 1e-2 * full.float().abs().max()
    assert torch.equal(c, c.t())                             # exactly symmetric after the mirror
    ref = x.float() @ x.float().t()
    assert (c.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    # a product of two commuting symmetric factors
    a = full.to(torch.bfloat16)
    s2 = G.gemm_symmetric(a, a, block=block, min_rows=0).float()
    ref2 = a.float() @ a.float().t()
    assert (s2 - ref2).abs().max() <= 3e-2 * ref2.abs().max()


def test_muon_on_large_matrix_uses_symmetric_panels(monkeypatch):
    from xorl_b200.ops import gemm as G
    from xorl_b200.optim.muon import newton_schulz
    monkeypatch.setattr(G, "SYMMETRIC_MIN_ROWS", 0)          # the default keeps small matrices on the plain GEMM
    torch.manual_seed(1)
    Gm = torch.randn(2048, 2560, device="cuda")
    before = G.launch_count()
    X = newton_schulz(Gm, steps=5).float()
    # per step: 2 symmetric products (2 panels + mirror each) + 1 plain GEMM
    assert G.launch_count() - before == 5 * (2 * 3 + 1)
    sv = torch.linalg.svdvals(X)
    assert sv.min() > 0.4 and sv.max() < 1.3


@pytest.mark.parametrize("scoring,renorm,E,k,bias", [("softmax", True, 128, 8, False), ("softmax", False, 8, 2, False),
                                                     ("sigmoid", True, 256, 8, True), ("softmax_after_topk", False, 32, 4, False),
                                                     ("softmax", True, 60, 3, False)])
def test_moe_route_kernel_matches_torch(scoring, renorm, E, k, bias, monkeypatch):
    from xorl_b200.ops import moe
    torch.manual_seed(E + k)
    T = 1000
    logits = torch.randn(T, E, device="cuda")
    cb = torch.randn(E, device="cuda") * 0.3 if bias else None
    a = logits.clone().requires_grad_()
    w, idx, probs = moe.topk_route(a, k, renorm, scoring, 2.5, correction_bias=cb)           # kernel
    monkeypatch.setenv("XORL_B200_ROUTE_KERNEL", "0")
    b = logits.clone().requires_grad_()
    w2, idx2, probs2 = moe.topk_route(b, k, renorm, scoring, 2.5, correction_bias=cb)        # torch ops
    assert torch.equal(idx.sort(-1).values, idx2.sort(-1).values)
    torch.testing.assert_close(probs, probs2, rtol=1e-5, atol=1e-6)
    o1, o2 = idx.argsort(-1), idx2.argsort(-1)
    torch.testing.assert_close(w.gather(1, o1), w2.gather(1, o2), rtol=1e-5, atol=1e-6)
    gw, gp = torch.randn_like(w), torch.randn_like(probs)
    ((w.gather(1, o1) * gw).sum() + (probs * gp).sum()).backward()
    ((w2.gather(1, o2) * gw).sum() + (probs2 * gp).sum()).backward()
    torch.testing.assert_close(a.grad, b.grad, rtol=1e-4, atol=1e-5)


def test_moe_permute_combine_kernels_match_torch_path(monkeypatch):
    """The gather kernels (permute, weighted combine and their backward) against the index_select /
    index_copy formulation, forward and every gradient."""
    from xorl_b200.models.config import preset
    from xorl_b200.models.context import StepContext
    from xorl_b200.models.moe import MoEBlock
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cuda")
    cfg = preset("qwen3-30b-a3b", hidden_size=256, num_experts=8, num_experts_per_tok=3,
                 moe_intermediate_size=128, num_hidden_layers=1)
    torch.manual_seed(0)
    blk = MoEBlock(cfg, 0, dtype=torch.bfloat16, device="cuda")
    for p in blk.parameters():
        torch.nn.init.normal_(p, 0, 0.05)
    T = 515
    x0 = (torch.randn(T, 256, device="cuda") * 0.5).to(torch.bfloat16)
    go = torch.randn(T, 256, device="cuda").to(torch.bfloat16)
    ctx = StepContext(cu_seqlens=torch.tensor([0, T], device="cuda", dtype=torch.int32),
                      position_ids=torch.arange(T, device="cuda"))
    res = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("XORL_B200_MOE_KERNELS", mode)
        for p in blk.parameters():
            p.grad = None
        x = x0.clone().requires_grad_()
        out = blk(x, ctx)
        out.backward(go)
        res[mode] = (out.detach().float(), x.grad.float(), blk.gate.weight.grad.float(),
                     blk.experts.gate_up_proj.grad.float(), blk.experts.down_proj.grad.float())
    for a, b, name in zip(res["1"], res["0"], ("out", "dx", "dgate", "dgate_up", "ddown")):
        tol = 0.02 * b.abs().max().item() + 1e-4
        assert (a - b).abs().max().item() <= tol, (name, (a - b).abs().max().item(), tol)
    reset_parallel_state()


@pytest.mark.parametrize("N,rank,E,k,T", [(2, 1, 8, 2, 300), (8, 3, 128, 8, 4096), (4, 0, 16, 4, 1000)])
def test_ep_plan_kernel_matches_torch_formulation(N, rank, E, k, T):
    """Destination rank / row of every token slot and the local segment table, against the
    argsort / cumsum formulation (rows of an expert keep slot order in both)."""
    import ctypes
    from xorl_b200.ops import _lib
    torch.manual_seed(N * 100 + E)
    El = E // N
    idx = torch.randint(0, E, (T, k), device="cuda")
    flat = idx.reshape(-1)
    S = flat.numel()
    counts = torch.bincount(flat, minlength=E).to(torch.int32)
    table = torch.randint(0, 2 * S // E, (N, E), device="cuda", dtype=torch.int32)
    table[rank] = counts
    cap = (int(1.5 * S) + El * 127 + 127) // 128 * 128
    dr = torch.empty(S, device="cuda", dtype=torch.int32)
    drow = torch.empty(S, device="cuda", dtype=torch.int32)
    seg = torch.empty(El + 1, device="cuda", dtype=torch.int32)
    tot = torch.empty(El, device="cuda", dtype=torch.int32)
    ovf = torch.zeros(1, device="cuda", dtype=torch.int32)
    _lib.check(_lib.cuda_lib().xb_ep_plan(flat.data_ptr(), S, table.data_ptr(), rank, N, E, El, cap, dr.data_ptr(),
                                          drow.data_ptr(), seg.data_ptr(), tot.data_ptr(), ovf.data_ptr(),
                                          _lib.stream_ptr()), "xb_ep_plan")
    # torch formulation
    tl = table.long()
    t_all = tl.sum(0)
    padded = (t_all + 127) // 128 * 128
    pe = padded.view(N, El)
    seg_start = (pe.cumsum(1) - pe).reshape(-1)
    before = tl[:rank].sum(0) if rank > 0 else torch.zeros_like(t_all)
    base = seg_start + before
    order = torch.argsort(flat, stable=True)
    c64 = counts.long()
    starts = c64.cumsum(0) - c64
    rank_in_e = torch.empty_like(flat)
    rank_in_e[order] = torch.arange(S, device="cuda") - starts[flat[order]]
    ref_row = base[flat] + rank_in_e
    ref_rank = flat // El
    over = ref_row >= cap
    assert torch.equal(dr.long(), torch.where(over, torch.full_like(ref_rank, -1), ref_rank))
    assert torch.equal(drow.long()[~over], ref_row[~over])
    assert bool(ovf.item()) == bool(over.any().item())
    mine = slice(rank * El, (rank + 1) * El)
    ref_seg = torch.cat([padded.new_zeros(1), padded[mine].cumsum(0)]).clamp(max=cap // 128 * 128)
    assert torch.equal(seg.long(), ref_seg) and torch.equal(tot.long(), t_all[mine])


# ---- block-scaled fp8 grouped GEMM (power-of-two scales on the tensor core) ----------------------
def _mx_case(E, K, N, counts, seed=0):
    from xorl_b200.ops import moe as moe_ops
    g = torch.Generator(device="cpu").manual_seed(seed)
    ids = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)])
    dest, seg, _ = moe_ops.aligned_sort_indices(ids.cuda(), E)
    rows = moe_ops.buffer_rows(ids.numel(), E)
    x = torch.zeros(rows, K, dtype=torch.bfloat16)
    x[dest.cpu()] = (torch.randn(ids.numel(), K, generator=g) * torch.rand(ids.numel(), 1, generator=g) * 3).bfloat16()
    w = (torch.randn(E, K, N, generator=g) * 0.05 * (1 + torch.arange(E).view(E, 1, 1))).bfloat16()
    return x.cuda(), w.cuda(), seg


def test_mx_quantisers_match_the_restatement():
    from xorl_b200.ops import fp8_grouped as fg
    x, w, _ = _mx_case(3, 384, 256, [100, 0, 300])
    q, sf = fg.quantize_rows(x)
    qr, er = fg.quantize_rows_ref(x.cpu())
    assert torch.equal(sf[:, :3].cpu().int() - 127, er)
    assert torch.equal(q.cpu().view(torch.float8_e4m3fn).float(), qr.float())
    qe = fg.quantize_experts(w)
    wq, we = fg.quantize_weight_ref(w.cpu())
    assert torch.equal(qe.sf_kn[:, :, :2].cpu().int() - 127, we)
    assert torch.equal(qe.sf_nk[:, :, :3].cpu().int() - 127, we.transpose(1, 2))
    assert torch.equal(qe.q_kn.cpu().view(torch.float8_e4m3fn).float(), wq.float())
    assert torch.equal(qe.q_nk.cpu().view(torch.float8_e4m3fn).float(), wq.float().transpose(1, 2))


@pytest.mark.parametrize("E,K,N,counts", [
    (3, 384, 256, [100, 0, 300]),                       # an empty expert, N not a multiple of 192
    (4, 768, 2048, [129, 640, 1, 255]),                 # down projection of Qwen3-30B-A3B
    (16, 2048, 1536, [2048 + 37 * (i % 5) - 64 * (i % 3) for i in range(16)]),   # gate_up projection, EP 8 load
])
def test_mx_grouped_gemm_matches_dequantised_matmul(E, K, N, counts):
    from xorl_b200.ops import _lib
    from xorl_b200.ops import fp8_grouped as fg
    x, w, seg = _mx_case(E, K, N, counts, seed=E)
    xq, sfx = fg.quantize_rows(x)
    qe = fg.quantize_experts(w)
    y = fg.grouped_rows_mx(xq, sfx, qe.q_nk, qe.sf_nk, seg)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    ref = fg.grouped_rows_ref(x.cpu().float(), w.cpu().float(), seg.cpu())
    err = (y.cpu().float() - ref).abs().max() / ref.abs().max()
    assert err < 6e-3, err                               # bf16 rounding of the output only
    # against the unquantised product: the error of the fp8 scheme itself
    exact = torch.zeros_like(ref)
    s = seg.cpu().tolist()
    for e in range(E):
        exact[s[e]:s[e + 1]] = x.cpu().float()[s[e]:s[e + 1]] @ w.cpu().float()[e]
    rel = (y.cpu().float() - exact).norm() / exact.norm()
    assert rel < 0.05, rel


def test_mx_grouped_linear_gradients():
    """Forward and input gradient in fp8 against the bf16 grouped linear; weight gradient (bf16) equal."""
    from xorl_b200.ops import fp8_grouped as fg
    from xorl_b200.ops import moe as moe_ops
    x, w, seg = _mx_case(4, 256, 384, [200, 31, 0, 500], seed=5)
    outs = {}
    for mode in (None, "fp8", "bf16"):
        xi, wi = x.clone().requires_grad_(), w.clone().requires_grad_()
        y = moe_ops.grouped_linear(xi, wi, seg, mode)
        dy = torch.randn(y.shape, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
        valid = torch.zeros(y.shape[0], 1, device="cuda", dtype=torch.bfloat16)
        s = seg.tolist()
        valid[: s[-1]] = 1
        y.backward(dy * valid)
        outs[mode] = (y.float(), xi.grad.float(), wi.grad.float())
    for mode in ("fp8", "bf16"):
        for a, b, name, tol in zip(outs[mode], outs[None], ("y", "dx", "dw"), (0.05, 0.05, 1e-6)):
            if mode == "bf16" and name == "dx":
                tol = 1e-6
            rel = (a - b).norm() / b.norm()
            assert rel <= tol, (mode, name, float(rel))
