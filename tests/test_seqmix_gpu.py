"""Causal depthwise convolution kernels and the 4-bit dequantisation kernel on a B200, each against
a plain PyTorch fp32 restatement of the same op."""
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


@pytest.mark.parametrize("T,C,K,bias,silu", [(700, 256, 4, True, True), (513, 72, 4, False, True),
                                             (64, 8, 2, True, False), (3000, 1024, 4, False, True)])
def test_causal_conv1d_forward_backward(T, C, K, bias, silu):
    from xorl_b200.ops import seqmix
    torch.manual_seed(0)
    cuts = sorted({0, 1, T // 3, T // 3 + 2, (2 * T) // 3, T - 5})
    cu = torch.tensor(cuts, dtype=torch.int32, device="cuda")          # the last 5 tokens are padding
    x = torch.randn(T, C, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(C, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    b = torch.randn(C, device="cuda").bfloat16().requires_grad_() if bias else None
    before = seqmix.launch_count()
    y = seqmix.causal_conv1d(x, w, b, cu, silu=silu)
    assert seqmix.launch_count() == before + 1
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    bf = b.detach().float().requires_grad_() if bias else None
    ref = seqmix.causal_conv1d_reference(xf, wf, bf, cu, silu)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    dy = torch.randn(T, C, device="cuda").bfloat16()
    y.backward(dy)
    ref.backward(dy.float())
    assert seqmix.launch_count() == before + 4
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=3e-2, atol=3e-2)
    scale = max(1.0, float(wf.grad.abs().max()))
    assert (w.grad.float() - wf.grad).abs().max() <= 2e-2 * scale
    if bias:
        assert (b.grad.float() - bf.grad).abs().max() <= 2e-2 * max(1.0, float(bf.grad.abs().max()))


def test_causal_conv1d_on_a_column_slice():
    """Mamba2 feeds a column block of its input projection: rows are strided."""
    from xorl_b200.ops import seqmix
    torch.manual_seed(1)
    T, C = 300, 64
    cu = torch.tensor([0, 120, 300], dtype=torch.int32, device="cuda")
    big = torch.randn(T, 3 * C, device="cuda").bfloat16()
    w = torch.randn(C, 4, device="cuda").bfloat16()
    x = big[:, C:2 * C]
    y = seqmix.causal_conv1d(x, w, None, cu, silu=True)
    ref = seqmix.causal_conv1d_reference(x.float(), w.float(), None, cu, True)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("fmt,group", [("nf4", 64), ("int4", 128), ("nvfp4", 16), ("mxfp4", 32)])
def test_dequant4_matches_codec(fmt, group):
    from xorl_b200.ops import quantize as Q, seqmix
    torch.manual_seed(0)
    shape = (192, 256)
    w = torch.randn(shape) * 0.05
    parts = Q.quantize_weight(w, fmt, group)
    ref = Q.dequantize_weight(parts, fmt, group, shape, torch.bfloat16)
    out = seqmix.dequant4({k: v.cuda() for k, v in parts.items()}, fmt, group, shape)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == shape
    assert torch.equal(out.cpu().float(), ref.float())


def test_qlora_linear_uses_the_dequant_kernel():
    from xorl_b200.adapters.qlora import QLoRALinear
    from xorl_b200.models.layers import Linear
    from xorl_b200.ops import seqmix
    torch.manual_seed(0)
    base = Linear(256, 128, dtype=torch.bfloat16, device="cuda")
    lin = QLoRALinear(base, rank=8, alpha=16, slices=[("all", 0, 128)], fmt="nf4", group=64)
    w = torch.randn(128, 256) * 0.05
    lin.load_base_weight(w)
    before = seqmix.launch_count()
    wd = lin.dequantized_weight()
    assert seqmix.launch_count() == before + 1
    assert (wd.float().cpu() - w).abs().max() < 0.04


@pytest.mark.parametrize("fmt,group", [("nf4", 64), ("int4", 128), ("nvfp4", 16), ("mxfp4", 32), ("nf4", 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quant4_kernel_matches_the_tensor_op_definitions(fmt, group, dtype):
    """The quantiser kernel gives the codes and scales of the tensor-op codecs evaluated on the host (IEEE
    division; the same tensor ops on a GPU multiply by reciprocals of scalar divisors and differ in the
    last bit of some scales), and its output decodes through the dequantiser kernel to within the
    format's step."""
    from xorl_b200.ops import quantize as Q
    from xorl_b200.ops import seqmix
    torch.manual_seed(0)
    w = (torch.randn(384, 512, device="cuda") * 0.05)
    w[0, :group] = 0                                   # an all-zero group: scale clamps
    w[1, 0] = 3.0                                      # an outlier
    w = w.to(dtype)
    ref_fn = {"nf4": Q.nf4_quantize, "int4": Q.int4_quantize, "nvfp4": Q.nvfp4_quantize, "mxfp4": Q.mxfp4_quantize}[fmt]
    ref = tuple(t.cuda() for t in ref_fn(w.cpu(), group))
    assert seqmix.quant4_supported(w, fmt, group)
    got = Q.quantize_weight(w, fmt, group)             # dispatches to the kernel on a GPU
    ref_scale = ref[1].view(torch.uint8) if fmt == "nvfp4" else ref[1]
    assert torch.equal(got["scale"], ref_scale.to(got["scale"].dtype)), fmt
    if fmt == "nvfp4":
        assert torch.equal(got["global_scale"], ref[2].float())
    # host and device libm may round log2 / exp2 differently in the last bit: allow a vanishing share of
    # codes to differ (none is expected)
    mism = (got["packed"] != ref[0]).float().mean().item()
    assert mism <= 1e-5, (fmt, mism)
    back = seqmix.dequant4(got, fmt, group, w.shape).float()
    err = (back - w.float()).abs().max().item()
    assert err < 0.3 * w.float().abs().max().item()
