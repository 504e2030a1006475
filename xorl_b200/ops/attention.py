"""Variable-length flash attention (``csrc/attn_fwd.cu`` / ``csrc/attn_bwd.cu``) and the fused
qk-RMSNorm + RoPE + attention block used by the decoder layers.

Layout is the packed one of the reference's varlen path
(src/xorl/models/layers/attention/backend/flash_attention.py:295-532): tokens of all sequences
concatenated, ``cu_seqlens`` int32 prefix sums, q ``[T, Hq, D]``, k/v ``[T, Hkv, D]``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib
from .grad_sink import deliver_param_grad

_launches = 0


def launch_count() -> int:
    return _launches


# --------------------------------------------------------------------------------------------
# Reference implementations (CPU lane and test oracle)
# --------------------------------------------------------------------------------------------
def attention_reference(q, k, v, cu_seqlens, causal=True, scale=None, window=None, sinks=None):
    """Plain fp32 attention over packed sequences. q [T,Hq,D], k [T,Hkv,D], v [T,Hkv,Dv].
    ``window``: a query sees only the last ``window`` keys (itself included).  ``sinks`` fp32 [Hq]:
    one extra logit per head that joins the softmax denominator but contributes no value
    (attention sinks of gpt-oss)."""
    T, Hq, D = q.shape
    Hkv, Dv = k.shape[1], v.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((T, Hq, Dv), dtype=q.dtype, device=q.device)
    cu = cu_seqlens.tolist()
    g = Hq // Hkv
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e <= s:
            continue
        L = e - s
        qb = q[s:e].float().transpose(0, 1)                      # [Hq, L, D]
        kb = k[s:e].float().transpose(0, 1).repeat_interleave(g, 0)
        vb = v[s:e].float().transpose(0, 1).repeat_interleave(g, 0)
        sc = torch.matmul(qb, kb.transpose(1, 2)) * scale
        if causal or window:
            i = torch.arange(L, device=q.device)
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device)
            if causal:
                mask &= i[:, None] >= i[None, :]
            if window:
                mask &= (i[:, None] - i[None, :]) < window
            sc = sc.masked_fill(~mask, float("-inf"))
        if sinks is not None:
            sink = sinks.float().view(Hq, 1, 1).expand(Hq, L, 1)
            p = torch.softmax(torch.cat([sc, sink], -1), dim=-1)[..., :L]
        else:
            p = torch.softmax(sc, dim=-1)
        out[s:e] = torch.matmul(p, vb).transpose(0, 1).to(q.dtype)
    return out


def rope_reference(x, cos, sin):
    """Rotate-half RoPE. x [T, H, D]; cos/sin [T, D/2]."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def _head_rmsnorm_ref(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def qk_norm_rope_attention_reference(qkv, wq, wk, cos, sin, cu_seqlens, Hq, Hkv, D, eps, causal,
                                     scale):
    T = qkv.shape[0]
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q = q.reshape(T, Hq, D)
    k = k.reshape(T, Hkv, D)
    v = v.reshape(T, Hkv, D)
    if wq is not None:
        q = _head_rmsnorm_ref(q, wq, eps)
        k = _head_rmsnorm_ref(k, wk, eps)
    q = rope_reference(q, cos, sin)
    k = rope_reference(k, cos, sin)
    return attention_reference(q, k, v, cu_seqlens, causal, scale).reshape(T, Hq * D)


# --------------------------------------------------------------------------------------------
# CUDA path
# --------------------------------------------------------------------------------------------
def _mask_arg(causal: bool, window) -> int:
    """The kernels' mask word: bit 0 causal, the bits above it a sliding-window length (0: none)."""
    return int(bool(causal)) | (int(window or 0) << 1)


def _attn_fwd(q, k, v, cu_seqlens, causal, scale, window=0, sinks=None):
    global _launches
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    out = torch.empty((T, Hq, D), device=q.device, dtype=q.dtype)
    lse = torch.empty((Hq, T), device=q.device, dtype=torch.float32)
    nseq = cu_seqlens.numel() - 1
    rc = _lib.cuda_lib().xb_attn_fwd_sink(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                          lse.data_ptr(), cu_seqlens.data_ptr(), None, _lib.ptr(sinks), q.stride(0),
                                          k.stride(0), v.stride(0), out.stride(0), nseq, T, T, Hq, Hkv, D,
                                          _mask_arg(causal, window), float(scale), 0, _lib.stream_ptr())
    _lib.check(rc, "xb_attn_fwd_sink")
    _launches += 1
    return out, lse


def _attn_bwd(q, k, v, out, dout, lse, cu_seqlens, causal, scale, dv_out, window=0, want_delta=False):
    """Returns dq fp32 [T,Hq,D], dk fp32 [T,Hkv,D]; writes dv (bf16) into ``dv_out``.  With
    ``want_delta`` also the per-row sums of dO o O (fp32 [Hq, T])."""
    global _launches
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    delta = torch.empty((Hq, T), device=q.device, dtype=torch.float32)
    dq = torch.empty((T, Hq, D), device=q.device, dtype=torch.float32)
    dk = torch.empty((T, Hkv, D), device=q.device, dtype=torch.float32)
    nseq = cu_seqlens.numel() - 1
    rc = _lib.cuda_lib().xb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                     dout.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                                     dq.data_ptr(), dk.data_ptr(), dv_out.data_ptr(),
                                     cu_seqlens.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                                     out.stride(0), dout.stride(0), dv_out.stride(0), nseq, T, Hq,
                                     Hkv, D, _mask_arg(causal, window), float(scale), 0, _lib.stream_ptr())
    _lib.check(rc, "xb_attn_bwd")
    _launches += 3
    return (dq, dk, delta) if want_delta else (dq, dk)


def set_backward_mode(mode: str) -> str:
    """"split": dK/dV kernel + query-stationary dQ kernel without atomics (default); "fused": one
    kernel that reduces dQ partials into global memory.  Returns the previous mode."""
    assert mode in ("split", "fused")
    prev = _lib.cuda_lib().xb_attn_bwd_set_split(1 if mode == "split" else 0)
    return "split" if prev else "fused"


def _kernel_ok(t: torch.Tensor, D: int) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and D == 128


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, causal, scale, window, sinks):
        def fix(t):
            if t.stride(2) != 1 or t.stride(1) != t.shape[2] or t.stride(0) % 8 or t.data_ptr() % 16:
                return t.contiguous()
            return t
        q, k, v = fix(q), fix(k), fix(v)
        sinks_f = sinks.detach().float().contiguous() if sinks is not None else None
        out, lse = _attn_fwd(q, k, v, cu_seqlens, causal, scale, window, sinks_f)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens, sinks_f)
        ctx.causal, ctx.scale, ctx.window = causal, scale, window
        ctx.sinks_dtype = sinks.dtype if sinks is not None else None
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu, sinks_f = ctx.saved_tensors
        dout = dout.contiguous()
        dv = torch.empty_like(v.contiguous())
        dq, dk, delta = _attn_bwd(q, k, v, out, dout, lse, cu, ctx.causal, ctx.scale, dv, ctx.window, True)
        dsinks = None
        if sinks_f is not None:
            # d/d sink = -sum over rows of p_sink * delta, p_sink = exp(sink - lse); rows outside
            # every sequence have lse = 0 written by nobody, so they are masked by position
            pos = torch.arange(lse.shape[1], device=lse.device)
            valid = ((pos >= cu[0]) & (pos < cu[-1])).view(1, -1)
            contrib = torch.where(valid, torch.exp(sinks_f.view(-1, 1) - lse) * delta, torch.zeros_like(lse))
            dsinks = (-contrib.sum(1)).to(ctx.sinks_dtype)
        return dq.to(q.dtype), dk.to(k.dtype), dv, None, None, None, None, dsinks


def flash_attn_varlen(q, k, v, cu_seqlens, causal=True, scale=None, window=None, sinks=None):
    """Packed varlen attention. q [T,Hq,D], k/v [T,Hkv,D], cu_seqlens int32 [B+1].  ``window``: a
    query sees only the last ``window`` keys (itself included); ``sinks`` [Hq]: per-head sink logits.
    Head dims below 128 run on the 128-wide kernel with zero-padded heads (the products are unchanged)."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    window = int(window or 0)
    if q.is_cuda and q.dtype == torch.bfloat16 and v.shape[-1] == D and D < 128 and D % 8 == 0:
        pad = (0, 128 - D)
        out = _FlashAttn.apply(F.pad(q, pad), F.pad(k, pad), F.pad(v, pad), cu_seqlens, causal, scale, window, sinks)
        return out[..., :D]
    if _kernel_ok(q, D) and v.shape[-1] == D:
        return _FlashAttn.apply(q, k, v, cu_seqlens, causal, scale, window, sinks)
    return attention_reference(q, k, v, cu_seqlens, causal, scale, window=window or None, sinks=sinks)


class _QKNormRopeAttn(torch.autograd.Function):
    """qkv [T, (Hq+2Hkv)*D] -> attention output [T, Hq*D]: per-head RMSNorm on q and k (optional),
    rotate-half RoPE, causal varlen attention.  The v slice is consumed in place through a strided
    view, and backward writes dq/dk/dv straight into one dqkv buffer."""

    @staticmethod
    def forward(ctx, qkv, wq, wk, cos, sin, cu_seqlens, Hq, Hkv, D, eps, causal, scale):
        global _launches
        T = qkv.shape[0]
        if not qkv.is_contiguous():
            qkv = qkv.contiguous()
        do_norm = wq is not None
        lib = _lib.cuda_lib()
        qk = torch.empty((T, (Hq + Hkv) * D), device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty((T, Hq + Hkv), device=qkv.device, dtype=torch.float32) if do_norm else None
        _lib.check(lib.xb_qk_norm_rope_fwd(qkv.data_ptr(), qkv.stride(0), _lib.ptr(wq), _lib.ptr(wk),
                                           cos.data_ptr(), sin.data_ptr(), qk.data_ptr(),
                                           qk.stride(0), _lib.ptr(rstd), T, Hq, Hkv, D, float(eps),
                                           int(do_norm), _lib.stream_ptr()), "xb_qk_norm_rope_fwd")
        _launches += 1
        q = qk[:, :Hq * D].view(T, Hq, D)
        k = qk[:, Hq * D:].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        out, lse = _attn_fwd(q, k, v, cu_seqlens, causal, scale)
        ctx.save_for_backward(qkv, qk, out, lse, cos, sin, cu_seqlens, rstd)
        ctx.wq, ctx.wk = wq, wk
        ctx.cfg = (Hq, Hkv, D, eps, causal, scale)
        return out.view(T, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        global _launches
        qkv, qk, out, lse, cos, sin, cu, rstd = ctx.saved_tensors
        Hq, Hkv, D, eps, causal, scale = ctx.cfg
        wq, wk = ctx.wq, ctx.wk
        do_norm = wq is not None
        T = qkv.shape[0]
        dout = dout.reshape(T, Hq, D)
        if not dout.is_contiguous():
            dout = dout.contiguous()
        q = qk[:, :Hq * D].view(T, Hq, D)
        k = qk[:, Hq * D:].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        dqkv = torch.empty_like(qkv)
        dv = dqkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        dq, dk = _attn_bwd(q, k, v, out, dout, lse, cu, causal, scale, dv)
        lib = _lib.cuda_lib()
        partial = dwq = dwk = None
        if do_norm:
            rows = lib.xb_qk_norm_rope_bwd_partial_rows()
            partial = torch.empty(rows * 2 * D, device=qkv.device, dtype=torch.float32)
            dwq = torch.zeros(D, device=qkv.device, dtype=torch.bfloat16)
            dwk = torch.zeros(D, device=qkv.device, dtype=torch.bfloat16)
        _lib.check(lib.xb_qk_norm_rope_bwd(None, dq.data_ptr(), dk.data_ptr(), 0, qkv.data_ptr(),
                                           qkv.stride(0), _lib.ptr(wq), _lib.ptr(wk), cos.data_ptr(),
                                           sin.data_ptr(), _lib.ptr(rstd), dqkv.data_ptr(),
                                           dqkv.stride(0), _lib.ptr(partial), _lib.ptr(dwq),
                                           _lib.ptr(dwk), 0, T, Hq, Hkv, D, int(do_norm),
                                           _lib.stream_ptr()), "xb_qk_norm_rope_bwd")
        _launches += 4 if do_norm else 1
        gq = gk = None
        if do_norm:
            gq = deliver_param_grad(wq, dwq)
            gk = deliver_param_grad(wk, dwk)
        return dqkv, gq, gk, None, None, None, None, None, None, None, None, None


class _QKNormRope(torch.autograd.Function):
    """The first half of ``_QKNormRopeAttn`` on its own: qkv [T, (Hq+2Hkv)*D] -> normalised, rotated
    q [T,Hq,D], k [T,Hkv,D] and the v view, for callers that run attention themselves (context
    parallelism moves q/k/v between ranks first)."""

    @staticmethod
    def forward(ctx, qkv, wq, wk, cos, sin, Hq, Hkv, D, eps):
        global _launches
        T = qkv.shape[0]
        if not qkv.is_contiguous():
            qkv = qkv.contiguous()
        do_norm = wq is not None
        qk = torch.empty((T, (Hq + Hkv) * D), device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty((T, Hq + Hkv), device=qkv.device, dtype=torch.float32) if do_norm else None
        _lib.check(_lib.cuda_lib().xb_qk_norm_rope_fwd(
            qkv.data_ptr(), qkv.stride(0), _lib.ptr(wq), _lib.ptr(wk), cos.data_ptr(), sin.data_ptr(), qk.data_ptr(),
            qk.stride(0), _lib.ptr(rstd), T, Hq, Hkv, D, float(eps), int(do_norm), _lib.stream_ptr()),
            "xb_qk_norm_rope_fwd")
        _launches += 1
        ctx.save_for_backward(qkv, cos, sin, rstd)
        ctx.wq, ctx.wk, ctx.cfg = wq, wk, (Hq, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
        return qk[:, :Hq * D].view(T, Hq, D), qk[:, Hq * D:].view(T, Hkv, D), v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        global _launches
        qkv, cos, sin, rstd = ctx.saved_tensors
        Hq, Hkv, D = ctx.cfg
        wq, wk = ctx.wq, ctx.wk
        do_norm = wq is not None
        T = qkv.shape[0]
        dqk = torch.cat([dq.reshape(T, Hq * D), dk.reshape(T, Hkv * D)], 1).to(qkv.dtype).contiguous()
        dqkv = torch.empty_like(qkv)
        dqkv[:, (Hq + Hkv) * D:] = dv.reshape(T, Hkv * D)
        lib = _lib.cuda_lib()
        partial = dwq = dwk = None
        if do_norm:
            rows = lib.xb_qk_norm_rope_bwd_partial_rows()
            partial = torch.empty(rows * 2 * D, device=qkv.device, dtype=torch.float32)
            dwq = torch.zeros(D, device=qkv.device, dtype=torch.bfloat16)
            dwk = torch.zeros(D, device=qkv.device, dtype=torch.bfloat16)
        _lib.check(lib.xb_qk_norm_rope_bwd(dqk.data_ptr(), None, None, dqk.stride(0), qkv.data_ptr(), qkv.stride(0),
                                           _lib.ptr(wq), _lib.ptr(wk), cos.data_ptr(), sin.data_ptr(), _lib.ptr(rstd),
                                           dqkv.data_ptr(), dqkv.stride(0), _lib.ptr(partial), _lib.ptr(dwq),
                                           _lib.ptr(dwk), 0, T, Hq, Hkv, D, int(do_norm), _lib.stream_ptr()),
                   "xb_qk_norm_rope_bwd")
        _launches += 4 if do_norm else 1
        gq = deliver_param_grad(wq, dwq) if do_norm else None
        gk = deliver_param_grad(wk, dwk) if do_norm else None
        return dqkv, gq, gk, None, None, None, None, None, None


def qk_norm_rope(qkv, wq, wk, cos, sin, Hq, Hkv, D, eps=1e-6):
    """qkv [T, (Hq+2Hkv)*D] -> (q [T,Hq,D], k [T,Hkv,D], v [T,Hkv,D]) with per-head RMSNorm (when
    ``wq``/``wk`` are given) and rotate-half RoPE applied to q and k."""
    T = qkv.shape[0]
    if _kernel_ok(qkv, D):
        return _QKNormRope.apply(qkv, wq, wk, cos, sin, Hq, Hkv, D, eps)
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q, k, v = q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D)
    if wq is not None:
        q, k = _head_rmsnorm_ref(q, wq, eps), _head_rmsnorm_ref(k, wk, eps)
    return rope_reference(q, cos, sin), rope_reference(k, cos, sin), v


def qk_norm_rope_attention(qkv, wq, wk, cos, sin, cu_seqlens, Hq, Hkv, D, eps=1e-6, causal=True,
                           scale=None):
    """Fused attention block over a packed qkv activation.

    qkv: [T, (Hq + 2*Hkv) * D]; wq/wk: per-head RMSNorm weights [D] or None (no qk-norm);
    cos/sin: fp32 [T, D/2] gathered at each token's position.  Returns [T, Hq*D].
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _kernel_ok(qkv, D):
        return _QKNormRopeAttn.apply(qkv, wq, wk, cos, sin, cu_seqlens, Hq, Hkv, D, eps, causal,
                                     scale)
    return qk_norm_rope_attention_reference(qkv, wq, wk, cos, sin, cu_seqlens, Hq, Hkv, D, eps,
                                            causal, scale)
