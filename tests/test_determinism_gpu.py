"""Run-to-run reproducibility of the kernels that are meant to be deterministic: each operator runs
twice on the same inputs (with other work in between, so block scheduling differs) and every output
and gradient must be bit-identical.  A kernel with a data race or an order-dependent reduction
fails this long before its numerical error becomes visible."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from xorl_b200.ops import _lib
    _lib.cuda_lib()
    yield
    assert all(v == 0 for v in _lib.read_status()[:4]), _lib.read_status()


def _disturb():
    a = torch.randn(2048, 2048, device=DEV)
    (a @ a).sum().item()


def _twice(fn):
    first = [t.clone() for t in fn()]
    _disturb()
    second = fn()
    for i, (a, b) in enumerate(zip(first, second)):
        assert torch.equal(a, b), f"output {i} differs between two runs (max diff {(a.float() - b.float()).abs().max().item():.3g})"


def test_gemm_is_reproducible():
    from xorl_b200.ops.gemm import gemm
    torch.manual_seed(0)
    a = torch.randn(1000, 520, device=DEV).bfloat16()
    b = torch.randn(1256, 520, device=DEV).bfloat16()
    _twice(lambda: [gemm(a, b), gemm(a, b, out_dtype=torch.float32)])


def test_attention_forward_and_split_backward_are_reproducible():
    from xorl_b200.ops import attention
    from xorl_b200.ops.attention import flash_attn_varlen
    torch.manual_seed(0)
    lens = [200, 56, 384, 1000]
    T, Hq, Hkv, D = sum(lens), 8, 2, 128
    cu = torch.tensor([0, 200, 256, 640, 1640], device=DEV, dtype=torch.int32)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(T, Hkv, D, device=DEV, dtype=torch.bfloat16)
    go = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    prev = attention.set_backward_mode("split")

    def run():
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        out = flash_attn_varlen(qq, kk, vv, cu, causal=True)
        out.backward(go)
        return [out.detach(), qq.grad, kk.grad, vv.grad]
    try:
        _twice(run)
    finally:
        attention.set_backward_mode(prev)


def test_rmsnorm_conv_swiglu_and_loss_are_reproducible():
    from xorl_b200.ops.activation import swiglu
    from xorl_b200.ops.loss import fused_linear_cross_entropy
    from xorl_b200.ops.norm import rmsnorm
    from xorl_b200.ops.seqmix import causal_conv1d
    torch.manual_seed(0)
    T, H, V = 1000, 1024, 3000
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    cw = torch.randn(H, 4, device=DEV).bfloat16()
    lm = (torch.randn(V, H, device=DEV) * 0.05).bfloat16()
    labels = torch.randint(0, V, (T,), device=DEV)
    cu = torch.tensor([0, 300, 301, 1000], device=DEV, dtype=torch.int32)
    gy = torch.randn(T, H, device=DEV).bfloat16()

    def run():
        xx, ww, cc, ll = (t.clone().requires_grad_() for t in (x, w, cw, lm))
        y = rmsnorm(xx, ww, 1e-6)
        z = causal_conv1d(y, cc, None, cu, silu=True)
        s = swiglu(torch.cat([z, y], dim=-1))
        loss = fused_linear_cross_entropy(s, ll, labels, grad_scale=1.0 / T, chunk_tokens=256)
        (loss + (s.float() * gy.float()).sum() * 1e-3).backward()
        return [y.detach(), z.detach(), s.detach(), loss.detach(), xx.grad, ww.grad, cc.grad, ll.grad]
    _twice(run)


def test_grouped_gemm_is_reproducible():
    from xorl_b200.ops import moe as moe_ops
    torch.manual_seed(0)
    E, K, N = 8, 256, 512
    counts = [100, 0, 300, 129, 7, 64, 250, 33]
    ids = torch.repeat_interleave(torch.arange(E), torch.tensor(counts)).to(DEV)
    S = ids.numel()
    dest, seg, _ = moe_ops.aligned_sort_indices(ids, E)
    rows = moe_ops.buffer_rows(S, E)
    xs = (torch.randn(S, K, device=DEV) * 0.5).bfloat16()
    buf = torch.zeros(rows, K, device=DEV, dtype=torch.bfloat16).index_copy(0, dest, xs)
    w = (torch.randn(E, K, N, device=DEV) * 0.05).bfloat16()
    go = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16).index_copy(
        0, dest, torch.randn(S, N, device=DEV).bfloat16())

    def run():
        bb, ww = buf.clone().requires_grad_(), w.clone().requires_grad_()
        y = moe_ops.grouped_linear(bb, ww, seg)
        y.backward(go)
        return [y.detach(), bb.grad, ww.grad]
    _twice(run)


def test_batch_invariant_gemm_rows_do_not_depend_on_the_batch():
    """In batch-invariant mode a row of x @ W^T has the same bits whether it is computed alone, in a
    batch of 300 rows or as part of 4096 rows (different tile counts, waves and tail handling)."""
    from xorl_b200.ops import gemm as G
    torch.manual_seed(0)
    x = torch.randn(4096, 1024, device="cuda").bfloat16()
    w = torch.randn(2560, 1024, device="cuda").bfloat16()
    prev = G.set_batch_invariant(True)
    try:
        full = G.gemm(x, w)
        for rows in (1, 300, 640, 2048):
            part = G.gemm(x[:rows].contiguous(), w)
            assert torch.equal(part, full[:rows]), rows
        mid = G.gemm(x[1000:1513].contiguous(), w)
        assert torch.equal(mid, full[1000:1513])
    finally:
        G.set_batch_invariant(prev)
    ref = (x.float() @ w.float().t())
    assert (full.float() - ref).abs().max() <= 0.02 * ref.abs().max()
