"""tcgen05 GEMM against an fp32 PyTorch reference, all four operand layouts."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


@pytest.fixture(params=["single", "pair"])
def variant(request):
    from xorl_b200.ops import gemm
    prev = gemm.set_variant(request.param)
    yield request.param
    gemm.set_variant(prev)
    from xorl_b200.ops import _lib
    assert all(v == 0 for v in _lib.read_status()[:4])


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (4096, 6144, 4096), (304, 200, 136),
                                   (1000, 1256, 520), (72, 88, 40), (2048, 152064, 512), (4096, 4096, 256),
                                   (1536, 2304, 192), (5000, 640, 320)])
def test_gemm_layouts(M, N, K, a_mn, b_mn, variant):
    from xorl_b200.ops import gemm
    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
    c = gemm.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn))
    torch.cuda.synchronize()
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)


def test_gemm_fp32_out_and_accumulate(variant):
    from xorl_b200.ops import gemm
    torch.manual_seed(1)
    a = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(640, 384, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    c = gemm.gemm(a, b, out_dtype=torch.float32)
    assert torch.allclose(c, ref, rtol=1e-3, atol=1e-2)
    c2 = gemm.gemm(a, b, out=c.clone(), accumulate=True)
    assert torch.allclose(c2, 2 * ref, rtol=1e-3, atol=2e-2)
    cb = gemm.gemm(a, b)
    cb2 = gemm.gemm(a, b, out=cb.clone(), accumulate=True)
    assert torch.allclose(cb2.float(), 2 * ref, rtol=2e-2, atol=0.5)
