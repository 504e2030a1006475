"""Weight / activation quantisation codecs: block-fp8 (e4m3, 1x128 and 128x128 scales), NVFP4
(e2m1, group 16, e4m3 block scale + fp32 global scale), MXFP4 (e2m1, group 32, e8m0 scale), NF4
and INT4 (group-wise absmax).  Every codec is ``quantize(w) -> (packed uint8, scales...)`` and
``dequantize(...) -> tensor``; 4-bit codes are packed two per byte (low nibble first).

Tensor-op implementations that run on CPU and GPU alike; the CUDA fast paths are
``csrc/quant.cu`` (block-fp8 quantise and the block-scaled tcgen05 GEMM).
Reference: src/xorl/ops/quantize/{block_fp8,nvfp4,nf4,int4,mxfp4}_quantize.py, fp4_codec.py.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

FP8_MAX = 448.0
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
NF4_VALUES = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
                           -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
                           0.07958029955625534, 0.16093020141124725, 0.24611230194568634,
                           0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                           0.7229568362236023, 1.0])


def _pack4(codes: torch.Tensor) -> torch.Tensor:
    codes = codes.reshape(-1, 2).to(torch.uint8)
    return (codes[:, 0] | (codes[:, 1] << 4)).contiguous()


def _unpack4(packed: torch.Tensor) -> torch.Tensor:
    return torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(-1)


def _nearest(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return (x.unsqueeze(-1) - table.to(x.device)).abs().argmin(-1)


# ---- block fp8 -----------------------------------------------------------------------------------
def block_fp8_quantize_1x128(x: torch.Tensor, block: int = 128):
    """Per-row blocks of 128 along the last dim (activations, row-wise weights)."""
    shp = x.shape
    K = shp[-1]
    assert K % block == 0, f"last dim {K} not a multiple of {block}"
    xb = x.float().reshape(-1, K // block, block)
    amax = xb.abs().amax(-1, keepdim=True).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (xb / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(shp), scale.squeeze(-1).reshape(*shp[:-1], K // block)


def block_fp8_dequantize_1x128(q: torch.Tensor, scale: torch.Tensor, block: int = 128, dtype=torch.bfloat16):
    K = q.shape[-1]
    xb = q.float().reshape(-1, K // block, block) * scale.reshape(-1, K // block, 1)
    return xb.reshape(q.shape).to(dtype)


def block_fp8_quantize_128x128(w: torch.Tensor, block: int = 128):
    """2-D blocks (weights [..., N, K]); scales [..., ceil(N/128), ceil(K/128)]."""
    *lead, N, K = w.shape
    nb, kb = -(-N // block), -(-K // block)
    wp = torch.zeros(*lead, nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[..., :N, :K] = w.float()
    blk = wp.reshape(*lead, nb, block, kb, block)
    amax = blk.abs().amax(dim=(-3, -1), keepdim=True).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (blk / scale).clamp(-FP8_MAX, FP8_MAX).reshape(*lead, nb * block, kb * block)[..., :N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.reshape(*lead, nb, kb)


def block_fp8_dequantize_128x128(q: torch.Tensor, scale: torch.Tensor, block: int = 128, dtype=torch.bfloat16):
    *lead, N, K = q.shape
    s = scale.repeat_interleave(block, -2).repeat_interleave(block, -1)[..., :N, :K]
    return (q.float() * s).to(dtype)


def block_fp8_gemm_reference(a_q, a_s, b_q, b_s, block: int = 128, out_dtype=torch.bfloat16):
    """C = sum_kb (A_kb B_kb^T) a_s[m,kb] b_s[n/128,kb]  — the 1x128 activation / 128x128 weight
    scheme (src/xorl/ops/quantize/block_fp8_quantize.py:155-203)."""
    a = block_fp8_dequantize_1x128(a_q, a_s, block, torch.float32)
    b = block_fp8_dequantize_128x128(b_q, b_s, block, torch.float32)
    return (a @ b.t()).to(out_dtype)


# ---- 4-bit codecs -----------------------------------------------------------------------------------
def _group(x: torch.Tensor, g: int) -> torch.Tensor:
    assert x.numel() % g == 0, f"{x.numel()} elements not divisible by group size {g}"
    return x.float().reshape(-1, g)


def nf4_quantize(w: torch.Tensor, group: int = 64):
    xg = _group(w, group)
    absmax = xg.abs().amax(-1, keepdim=True).clamp_min(1e-12)
    codes = _nearest(xg / absmax, NF4_VALUES)
    return _pack4(codes), absmax.squeeze(-1)


def nf4_dequantize(packed, absmax, shape, group: int = 64, dtype=torch.bfloat16):
    vals = NF4_VALUES.to(packed.device)[_unpack4(packed).long()].reshape(-1, group)
    return (vals * absmax.reshape(-1, 1)).reshape(shape).to(dtype)


def int4_quantize(w: torch.Tensor, group: int = 128):
    xg = _group(w, group)
    scale = xg.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 7.0
    codes = (xg / scale).round().clamp(-8, 7) + 8
    return _pack4(codes), scale.squeeze(-1)


def int4_dequantize(packed, scale, shape, group: int = 128, dtype=torch.bfloat16):
    vals = _unpack4(packed).float().reshape(-1, group) - 8.0
    return (vals * scale.reshape(-1, 1)).reshape(shape).to(dtype)


def _e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    mag = _nearest(x.abs(), E2M1_VALUES)
    return mag | ((x < 0).long() << 3)


def _e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    mag = E2M1_VALUES.to(codes.device)[(codes & 7).long()]
    return torch.where((codes & 8) > 0, -mag, mag)


def nvfp4_quantize(w: torch.Tensor, group: int = 16, global_scale: Optional[torch.Tensor] = None):
    """e2m1 values, one e4m3 scale per 16 elements, one fp32 global scale per tensor (``global_scale``
    forces a given one: matrices that a consumer fuses into one GEMM must share it)."""
    xg = _group(w, group)
    if global_scale is None:
        gmax = xg.abs().max().clamp_min(1e-12)
        global_scale = gmax / (6.0 * FP8_MAX)
    else:
        global_scale = torch.as_tensor(global_scale, dtype=torch.float32, device=w.device).reshape(())
    bs = (xg.abs().amax(-1, keepdim=True) / 6.0 / global_scale).clamp(1e-12, FP8_MAX)
    bs8 = bs.to(torch.float8_e4m3fn)
    denom = (bs8.float() * global_scale).clamp_min(1e-30)
    codes = _e2m1_encode(xg / denom)
    return _pack4(codes), bs8.squeeze(-1), global_scale.reshape(1)


def nvfp4_dequantize(packed, block_scale, global_scale, shape, group: int = 16, dtype=torch.bfloat16):
    vals = _e2m1_decode(_unpack4(packed)).reshape(-1, group)
    return (vals * block_scale.float().reshape(-1, 1) * global_scale.float()).reshape(shape).to(dtype)


def mxfp4_quantize(w: torch.Tensor, group: int = 32):
    """e2m1 values with a power-of-two (e8m0) scale per 32 elements."""
    xg = _group(w, group)
    amax = xg.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    codes = _e2m1_encode(xg / torch.exp2(exp))
    return _pack4(codes), (exp.squeeze(-1) + 127).to(torch.uint8)


def mxfp4_dequantize(packed, exp_biased, shape, group: int = 32, dtype=torch.bfloat16):
    vals = _e2m1_decode(_unpack4(packed)).reshape(-1, group)
    return (vals * torch.exp2(exp_biased.float().reshape(-1, 1) - 127.0)).reshape(shape).to(dtype)


# ---- uniform interface used by QLoRA ------------------------------------------------------------------
def quantize_weight(w: torch.Tensor, fmt: str, group: int) -> Dict[str, torch.Tensor]:
    if w.is_cuda and fmt in ("nf4", "int4", "nvfp4", "mxfp4"):
        from . import seqmix
        if seqmix.quant4_supported(w, fmt, group):
            return seqmix.quant4(w, fmt, group)          # quantiser kernel (csrc/seqmix.cu)
    if fmt == "nf4":
        p, s = nf4_quantize(w, group)
        return {"packed": p, "scale": s}
    if fmt == "int4":
        p, s = int4_quantize(w, group)
        return {"packed": p, "scale": s}
    if fmt == "nvfp4":
        p, s, g = nvfp4_quantize(w, group)
        return {"packed": p, "scale": s.view(torch.uint8), "global_scale": g}
    if fmt == "mxfp4":
        p, s = mxfp4_quantize(w, group)
        return {"packed": p, "scale": s}
    if fmt == "block_fp8":
        q, s = block_fp8_quantize_128x128(w)
        return {"packed": q.view(torch.uint8).reshape(-1), "scale": s.reshape(-1)}
    raise ValueError(f"unknown quant_format {fmt!r}")


def dequantize_weight(parts: Dict[str, torch.Tensor], fmt: str, group: int, shape, dtype=torch.bfloat16):
    if fmt == "nf4":
        return nf4_dequantize(parts["packed"], parts["scale"], shape, group, dtype)
    if fmt == "int4":
        return int4_dequantize(parts["packed"], parts["scale"], shape, group, dtype)
    if fmt == "nvfp4":
        return nvfp4_dequantize(parts["packed"], parts["scale"].view(torch.float8_e4m3fn),
                                parts["global_scale"], shape, group, dtype)
    if fmt == "mxfp4":
        return mxfp4_dequantize(parts["packed"], parts["scale"], shape, group, dtype)
    if fmt == "block_fp8":
        N, K = shape
        q = parts["packed"].view(torch.float8_e4m3fn).reshape(N, K)
        return block_fp8_dequantize_128x128(q, parts["scale"].reshape(-(-N // 128), -(-K // 128)), 128, dtype)
    raise ValueError(f"unknown quant_format {fmt!r}")
