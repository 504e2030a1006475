"""MoE operators: top-k routing, load-balancing loss, token permutation, grouped expert MLP.

CUDA path: ``csrc/moe.cu`` (routing / histogram / aligned sort indices / gather / weighted
scatter, no host synchronisation) and ``csrc/grouped_gemm.cu`` (tcgen05 grouped GEMM over
128-row-aligned expert segments).  CPU path: plain PyTorch with identical semantics.
Reference counterparts: src/xorl/models/layers/moe/router.py:232-259,
src/xorl/ops/group_gemm/kernel/group_gemm.py:80-377, src/xorl/ops/group_gemm/kernel/moe.py:45-433.
"""
from __future__ import annotations

import os

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .activation import swiglu
from .grad_sink import deliver_param_grad, grad_target, mark_written

SEG_ALIGN = 128  # expert segments of the sorted token buffer start at multiples of 128 rows
_launches = 0


def launch_count() -> int:
    return _launches


# --------------------------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------------------------
_SCORING_ID = {"softmax": 0, "sigmoid": 1, "softmax_after_topk": 2}


class _RouteKernel(torch.autograd.Function):
    """Forward: one fused kernel (csrc/moe_route.cu).  Backward: closed forms on the saved
    probabilities / choices (a few [T, E] elementwise ops)."""

    @staticmethod
    def forward(ctx, logits, bias, k, renorm, scoring, scale):
        global _launches
        T, E = logits.shape
        logits = logits.contiguous()
        w = torch.empty((T, k), device=logits.device, dtype=torch.float32)
        idx = torch.empty((T, k), device=logits.device, dtype=torch.int64)
        probs = torch.empty((T, E), device=logits.device, dtype=torch.float32)
        _lib.check(_lib.cuda_lib().xb_moe_route(
            logits.data_ptr(), logits.stride(0), _lib.ptr(bias), w.data_ptr(), idx.data_ptr(), probs.data_ptr(),
            None, T, E, k, _SCORING_ID[scoring], int(renorm), float(scale), _lib.stream_ptr()), "xb_moe_route")
        _launches += 1
        ctx.save_for_backward(probs, idx, w)
        ctx.cfg = (renorm, scoring, scale)
        ctx.mark_non_differentiable(idx)
        return w, idx, probs

    @staticmethod
    def backward(ctx, dw, _didx, dprobs):
        probs, idx, w = ctx.saved_tensors
        renorm, scoring, scale = ctx.cfg
        dp = dprobs.clone() if dprobs is not None else torch.zeros_like(probs)
        dlogits = None
        if dw is not None:
            if scoring == "softmax_after_topk":
                s = w / scale
                dl_sel = scale * s * (dw - (dw * s).sum(-1, keepdim=True))
                dlogits = torch.zeros_like(probs).scatter_add_(1, idx, dl_sel)
            else:
                if renorm:
                    u = w / scale
                    S = probs.gather(1, idx).sum(-1, keepdim=True).clamp_min(1e-20)
                    dp_sel = scale / S * (dw - (dw * u).sum(-1, keepdim=True))
                else:
                    dp_sel = scale * dw
                dp.scatter_add_(1, idx, dp_sel)
        if scoring == "sigmoid":
            g = dp * probs * (1 - probs)
        else:
            g = probs * (dp - (dp * probs).sum(-1, keepdim=True))
        dlogits = g if dlogits is None else dlogits + g
        return dlogits, None, None, None, None, None


def topk_route(logits: torch.Tensor, k: int, renorm: bool = True, scoring: str = "softmax",
               scale: float = 1.0, n_group: int = 1, topk_group: int = 1,
               correction_bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 logits [T, E] -> (weights [T, k], indices [T, k], probs [T, E]).

    ``scoring`` "softmax" (Qwen/Mixtral style), "sigmoid" (DeepSeek-V3 / GLM-4.5 style),
    "sqrtsoftplus" (DeepSeek-V4: sqrt(softplus(logit)), otherwise like sigmoid) or
    "softmax_after_topk" (gpt-oss: softmax over the k selected logits).  With ``correction_bias``
    the *selection* uses ``probs + bias`` while the weights stay the unbiased scores (auxiliary-loss
    free balancing); with ``n_group > 1`` experts are chosen only inside the ``topk_group`` groups
    with the best sum of their two best biased scores (src/xorl/models/layers/moe/router.py)."""
    if (logits.is_cuda and logits.dtype == torch.float32 and n_group <= 1 and logits.shape[1] <= 512 and k <= 32
            and scoring in ("softmax", "sigmoid", "softmax_after_topk") and _lib.have_cuda_lib() and os.environ.get("XORL_B200_ROUTE_KERNEL", "1") == "1"):
        return _RouteKernel.apply(logits, correction_bias, k, bool(renorm), scoring, float(scale))
    if scoring == "softmax_after_topk":
        top, indices = torch.topk(logits, k, dim=-1)
        weights = torch.softmax(top, dim=-1, dtype=torch.float32)
        probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
        return weights * scale if scale != 1.0 else weights, indices, probs
    if scoring == "sigmoid":
        probs = torch.sigmoid(logits)
    elif scoring == "sqrtsoftplus":             # DeepSeek-V4
        probs = torch.sqrt(torch.nn.functional.softplus(logits.float()))
    else:
        probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    choice = probs if correction_bias is None else probs + correction_bias.float().unsqueeze(0)
    if n_group > 1:
        T, E = choice.shape
        grouped = choice.view(T, n_group, E // n_group)
        gscore = grouped.topk(min(2, E // n_group), dim=-1)[0].sum(-1)          # [T, n_group]
        keep = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, gscore.topk(topk_group, dim=-1)[1], True)
        choice = grouped.masked_fill(~keep.unsqueeze(-1), float("-inf")).view(T, E)
    _, indices = torch.topk(choice, k, dim=-1)
    weights = probs.gather(1, indices)
    if renorm:
        weights = weights / weights.sum(-1, keepdim=True).clamp_min(1e-20)
    if scale != 1.0:
        weights = weights * scale
    return weights, indices, probs


def expert_histogram(indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    """int32 [E]: number of (token, slot) pairs routed to every expert (one kernel on CUDA)."""
    global _launches
    flat = indices.reshape(-1)
    if flat.is_cuda and flat.dtype == torch.int64 and _lib.have_cuda_lib():
        flat = flat.contiguous()
        counts = torch.empty(num_experts, device=flat.device, dtype=torch.int32)
        _lib.check(_lib.cuda_lib().xb_moe_histogram(flat.data_ptr(), flat.numel(), counts.data_ptr(), num_experts,
                                                    _lib.stream_ptr()), "xb_moe_histogram")
        _launches += 1
        return counts
    return torch.bincount(flat, minlength=num_experts).to(torch.int32)


def load_balancing_loss(probs: torch.Tensor, indices: torch.Tensor, num_experts: int,
                        global_group=None, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``E * sum_e f_e * P_e`` with f_e the fraction of routed slots sent to expert e and P_e the
    mean router probability.  With ``global_group`` the counts are summed over that group.
    ``counts``: the per-expert histogram of ``indices`` when the caller already has it."""
    T, k = indices.shape
    if counts is None:
        counts = expert_histogram(indices, num_experts)
    counts = counts.float()
    if global_group is not None:
        total = torch.tensor(float(T), device=probs.device)
        dist.all_reduce(counts, group=global_group)
        dist.all_reduce(total, group=global_group)
        f = counts / (total * k)
    else:
        f = counts * (1.0 / (T * k))
    return num_experts * torch.dot(f, probs.mean(0))


# --------------------------------------------------------------------------------------------
# permutation helpers (aligned segments)
# --------------------------------------------------------------------------------------------
def aligned_sort_indices(expert_ids: torch.Tensor, num_experts: int, align: int = SEG_ALIGN):
    """For a flat list of expert ids [S] returns
       dest   int64 [S]   row of every slot in the sorted, segment-aligned buffer,
       seg    int32 [E+1] aligned start row of each expert segment (seg[E] = total rows),
       counts int64 [E]   real rows per expert.
    Stable (slots of one expert keep their order), no host sync; the buffer size bound
    ``S + E*(align-1)`` rounded up to ``align`` is what callers allocate."""
    S = expert_ids.numel()
    counts = torch.bincount(expert_ids, minlength=num_experts)
    padded = (counts + align - 1) // align * align
    seg = torch.zeros(num_experts + 1, device=expert_ids.device, dtype=torch.int64)
    seg[1:] = torch.cumsum(padded, 0)
    order = torch.argsort(expert_ids, stable=True)
    starts_unpadded = torch.cumsum(counts, 0) - counts
    sorted_e = expert_ids[order]
    rank_in_e = torch.arange(S, device=expert_ids.device) - starts_unpadded[sorted_e]
    dest_sorted = seg[:-1][sorted_e] + rank_in_e
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    return dest, seg.to(torch.int32), counts


def buffer_rows(num_slots: int, num_experts: int, align: int = SEG_ALIGN) -> int:
    return (num_slots + num_experts * (align - 1) + align - 1) // align * align


# --------------------------------------------------------------------------------------------
# grouped GEMM
# --------------------------------------------------------------------------------------------
def _grouped_rows_cuda(a, b, seg, out, b_kmajor: bool):
    """out[rows of e] = a[rows of e] @ op(b[e]); b [E, K, N] (b_kmajor False) or [E, N, K]."""
    global _launches
    E = b.shape[0]
    if b_kmajor:
        N, K = b.shape[1], b.shape[2]
    else:
        K, N = b.shape[1], b.shape[2]
    rc = _lib.cuda_lib().xb_grouped_gemm_rows(a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                              seg.data_ptr(), E, a.shape[0], N, K, a.stride(0),
                                              out.stride(0), int(not b_kmajor), _lib.stream_ptr())
    _lib.check(rc, "xb_grouped_gemm_rows")
    _launches += 1
    return out


def _grouped_wgrad_cuda(a, b, seg, out, accumulate: bool):
    """out[e] (+)= a[rows of e]^T @ b[rows of e]; a [R, M], b [R, N], out [E, M, N]."""
    global _launches
    E, M, N = out.shape
    rc = _lib.cuda_lib().xb_grouped_gemm_wgrad(a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                               seg.data_ptr(), E, a.shape[0], M, N, a.stride(0),
                                               b.stride(0), int(out.dtype == torch.float32),
                                               int(accumulate), _lib.stream_ptr())
    _lib.check(rc, "xb_grouped_gemm_wgrad")
    _launches += 1
    return out


def _grouped_rows_ref(a, b, seg, b_kmajor: bool):
    E = b.shape[0]
    N = b.shape[1] if b_kmajor else b.shape[2]
    out = a.new_zeros((a.shape[0], N))
    s = seg.tolist()
    for e in range(E):
        if s[e + 1] > s[e]:
            w = b[e].t() if b_kmajor else b[e]
            out[s[e]:s[e + 1]] = (a[s[e]:s[e + 1]].float() @ w.float()).to(a.dtype)
    return out


class _GroupedLinear(torch.autograd.Function):
    """y[rows of e] = x[rows of e] @ w[e]  with w [E, K, N]; padding rows of x must be zero."""

    @staticmethod
    def forward(ctx, x, w, seg):
        ctx.save_for_backward(x, seg)
        ctx.w = w
        out = torch.zeros((x.shape[0], w.shape[2]), device=x.device, dtype=x.dtype)
        return _grouped_rows_cuda(x, w, seg, out, b_kmajor=False)

    @staticmethod
    def backward(ctx, dy):
        x, seg = ctx.saved_tensors
        w = ctx.w
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros_like(x)
            _grouped_rows_cuda(dy, w, seg, dx, b_kmajor=True)   # dx = dy @ w[e]^T
        dw = None
        if ctx.needs_input_grad[1]:
            tgt, fresh = grad_target(w)
            if tgt is not None:
                _grouped_wgrad_cuda(x, dy, seg, tgt, accumulate=not fresh)
                mark_written(w)
            else:
                dw = torch.empty_like(w)
                _grouped_wgrad_cuda(x, dy, seg, dw, accumulate=False)
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, seg: torch.Tensor, fp8: Optional[str] = None) -> torch.Tensor:
    """``fp8``: None (bf16 GEMMs), "fp8" (block-scaled fp8 forward and input gradient) or "bf16"
    (fp8 forward, bf16 input gradient) -- ``train.fp8_training_backward``."""
    if fp8 is not None:
        from .fp8_grouped import grouped_linear_fp8
        return grouped_linear_fp8(x, w, seg, backward=fp8)
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 \
            and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0:
        return _GroupedLinear.apply(x, w, seg)
    # CPU lane: differentiable loop over experts
    outs = []
    s = seg.tolist()
    for e in range(w.shape[0]):
        outs.append(x[s[e]:s[e + 1]] @ w[e])
    return torch.cat(outs, 0) if outs else x.new_zeros((0, w.shape[2]))


def _rows_to_expert(seg: torch.Tensor, rows: int) -> torch.Tensor:
    """Expert index of every row of a segment-aligned buffer (rows past the last segment -> last)."""
    r = torch.arange(rows, device=seg.device)
    return (torch.bucketize(r, seg[1:].long(), right=True)).clamp_max(seg.numel() - 2)


def clamped_swiglu(h: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
    """gpt-oss activation on a fused [gate | up] tensor: (up.clamp(+-limit) + 1) * gate' * sigmoid(alpha gate')
    with gate' = gate.clamp(max=limit)."""
    gate, up = h.float().chunk(2, dim=-1)
    gate = gate.clamp(max=limit)
    up = up.clamp(min=-limit, max=limit)
    return ((up + 1.0) * gate * torch.sigmoid(alpha * gate)).to(h.dtype)


def expert_mlp_aligned(x_buf: torch.Tensor, seg: torch.Tensor, gate_up: torch.Tensor,
                       down: torch.Tensor, gate_up_bias: Optional[torch.Tensor] = None,
                       down_bias: Optional[torch.Tensor] = None,
                       swiglu_limit: Optional[float] = None, activation: Optional[str] = None,
                       fp8: Optional[str] = None, lora: Optional[dict] = None) -> torch.Tensor:
    """SwiGLU expert MLP over a segment-aligned token buffer (optional per-expert biases and the
    clamped activation of gpt-oss); ``activation="relu2"``: non-gated ``relu(up(x))^2`` experts.
    ``fp8``: run both grouped GEMMs in block-scaled fp8 (see ``grouped_linear``).
    ``lora``: per-expert low-rank adapters ``{"scaling": s, "gate_proj": (A [E,H,r], B [E,r,I]),
    "up_proj": ..., "down_proj": (A [E,I,r], B [E,r,H])}``; each projection present adds
    ``s * (x @ A[e]) @ B[e]`` through two more grouped GEMMs
    (src/xorl/models/layers/moe/lora.py:13-15)."""
    if lora is not None:
        return _expert_mlp_lora(x_buf, seg, gate_up, down, lora, fp8)
    h = grouped_linear(x_buf, gate_up, seg, fp8)
    if activation == "relu2":
        return grouped_linear(torch.relu(h).square(), down, seg, fp8)
    if gate_up_bias is None and swiglu_limit is None:
        return grouped_linear(swiglu(h), down, seg, fp8)
    eid = _rows_to_expert(seg, h.shape[0])
    if gate_up_bias is not None:
        h = h + gate_up_bias.index_select(0, eid).to(h.dtype)
    a = clamped_swiglu(h, swiglu_limit) if swiglu_limit is not None else swiglu(h)
    y = grouped_linear(a, down, seg, fp8)
    if down_bias is not None:
        y = y + down_bias.index_select(0, eid[: y.shape[0]]).to(y.dtype)
    return y


def _lora_factor(x, W, seg, n_experts: int):
    """``x`` through one adapter factor ``W [E, in, out]``: grouped by expert, or -- a factor shared by all
    experts, ``W [1, in, out]`` -- one dense GEMM over all rows."""
    if W.shape[0] == 1 and n_experts > 1:
        from .gemm import linear
        return linear(x, W[0].t().contiguous())
    return grouped_linear(x, W, seg)


def _expert_mlp_lora(x_buf, seg, gate_up, down, lora: dict, fp8) -> torch.Tensor:
    s = float(lora["scaling"])
    I = down.shape[1]
    E = gate_up.shape[0]
    h = grouped_linear(x_buf, gate_up, seg, fp8)
    parts = []
    for name in ("gate_proj", "up_proj"):
        ab = lora.get(name)
        if ab is None:
            parts.append(None)
            continue
        A, B = ab
        parts.append(_lora_factor(_lora_factor(x_buf, A, seg, E), B, seg, E) * s)
    if parts[0] is not None or parts[1] is not None:
        zero = None
        cols = []
        for d in parts:
            if d is None:
                zero = h.new_zeros((h.shape[0], I)) if zero is None else zero
                d = zero
            cols.append(d)
        h = h + torch.cat(cols, dim=-1)
    a = swiglu(h)
    y = grouped_linear(a, down, seg, fp8)
    ab = lora.get("down_proj")
    if ab is not None:
        y = y + _lora_factor(_lora_factor(a, ab[0], seg, E), ab[1], seg, E) * s
    return y


def experts_mlp_kwargs(experts) -> dict:
    """Bias / activation options of an experts holder (plain holders without them -> {})."""
    fn = getattr(experts, "mlp_kwargs", None)
    return fn() if callable(fn) else {}


def expert_mlp(x_sorted: torch.Tensor, tokens_per_expert: torch.Tensor, gate_up: torch.Tensor,
               down: torch.Tensor, **kw) -> torch.Tensor:
    """Unaligned variant (rows exactly grouped by expert): pads to aligned segments internally."""
    E = gate_up.shape[0]
    ids = torch.repeat_interleave(torch.arange(E, device=x_sorted.device), tokens_per_expert)
    dest, seg, _ = aligned_sort_indices(ids, E)
    buf = x_sorted.new_zeros((buffer_rows(x_sorted.shape[0], E), x_sorted.shape[1]))
    buf = buf.index_copy(0, dest, x_sorted)
    out = expert_mlp_aligned(buf, seg, gate_up, down, **kw)
    return out.index_select(0, dest)


# --------------------------------------------------------------------------------------------
# permutation / combine kernels (csrc/moe_permute.cu)
# --------------------------------------------------------------------------------------------
def _permute_kernels_ok(x: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and _lib.have_cuda_lib()
            and os.environ.get("XORL_B200_MOE_KERNELS", "1") == "1")


def _gather_rows(inp, src_row, rows, scale=None):
    global _launches
    out = torch.empty((rows, inp.shape[1]), device=inp.device, dtype=inp.dtype)
    inp = inp.contiguous()
    _lib.check(_lib.cuda_lib().xb_moe_gather_rows(out.data_ptr(), out.stride(0), inp.data_ptr(), inp.stride(0),
                                                  src_row.data_ptr(), _lib.ptr(scale), rows, inp.shape[1],
                                                  _lib.stream_ptr()), "xb_moe_gather_rows")
    _launches += 1
    return out


def _gather_sum(inp, idx, w):
    global _launches
    T, k = idx.shape
    inp = inp.contiguous()
    out = torch.empty((T, inp.shape[1]), device=inp.device, dtype=inp.dtype)
    _lib.check(_lib.cuda_lib().xb_moe_gather_sum(out.data_ptr(), out.stride(0), inp.data_ptr(), inp.stride(0),
                                                 idx.data_ptr(), _lib.ptr(w), T, k, inp.shape[1],
                                                 _lib.stream_ptr()), "xb_moe_gather_sum")
    _launches += 1
    return out


class _Permute(torch.autograd.Function):
    """x [T,H] -> buffer [rows,H]: row dest[t,j] holds x[t]; rows nobody owns are zero."""

    @staticmethod
    def forward(ctx, x, dest, tok_of_row):
        ctx.save_for_backward(dest)
        return _gather_rows(x, tok_of_row, tok_of_row.numel())

    @staticmethod
    def backward(ctx, dbuf):
        (dest,) = ctx.saved_tensors
        return _gather_sum(dbuf, dest, None), None, None


class _Combine(torch.autograd.Function):
    """out[t] = sum_j w[t,j] * y[dest[t,j]] (fp32 accumulation, bf16 result)."""

    @staticmethod
    def forward(ctx, y, w, dest, tok_of_row):
        w = w.float().contiguous()
        ctx.save_for_backward(y, w, dest, tok_of_row)
        return _gather_sum(y, dest, w)

    @staticmethod
    def backward(ctx, dout):
        global _launches
        y, w, dest, tok_of_row = ctx.saved_tensors
        dout = dout.contiguous()
        rows = y.shape[0]
        T, k = dest.shape
        scale_row = torch.zeros(rows, device=y.device, dtype=torch.float32)
        scale_row[dest.reshape(-1)] = w.reshape(-1)
        dy = _gather_rows(dout, tok_of_row, rows, scale_row)
        dw = torch.empty((T, k), device=y.device, dtype=torch.float32)
        _lib.check(_lib.cuda_lib().xb_moe_slot_dots(dw.data_ptr(), dout.data_ptr(), dout.stride(0), y.data_ptr(),
                                                    y.stride(0), dest.data_ptr(), T, k, y.shape[1],
                                                    _lib.stream_ptr()), "xb_moe_slot_dots")
        _launches += 1
        return dy, dw, None, None


def canonical_combine(y_slots: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Bit-reproducible weighted sum over the k expert outputs of every token: products and sums in
    fp64, added as a fixed balanced binary tree over the slot axis (slot order = the router's
    order), one final rounding to the output dtype.  The result does not depend on how slots were
    permuted, exchanged or which rank computed which expert -- the parity lane between training and
    serving (src/xorl/distributed/canonical_moe.py, canonical_combine.py:315)."""
    T, k, H = y_slots.shape
    terms = y_slots.double() * weights.double().unsqueeze(-1)
    parts = [terms[:, j] for j in range(k)]
    while len(parts) > 1:
        nxt = [parts[i] + parts[i + 1] for i in range(0, len(parts) - 1, 2)]
        if len(parts) % 2:
            nxt.append(parts[-1])
        parts = nxt
    return parts[0].to(y_slots.dtype)


def token_of_row(dest: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Inverse of ``dest`` [T*k]: token index stored in every buffer row, -1 for padding rows."""
    tok = torch.full((rows,), -1, device=dest.device, dtype=torch.int32)
    tok[dest] = (torch.arange(dest.numel(), device=dest.device) // k).to(torch.int32)
    return tok


def local_moe_forward(x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, experts,
                      num_experts: int, canonical: bool = False) -> torch.Tensor:
    """All experts local: gather tokens into expert-sorted aligned segments, run the grouped MLP,
    combine the k expert outputs of every token with its routing weights (fp32 accumulation)."""
    T, H = x.shape
    k = indices.shape[1]
    dest, seg, _ = aligned_sort_indices(indices.reshape(-1), num_experts)
    rows = buffer_rows(T * k, num_experts)
    if _permute_kernels_ok(x) and not canonical:
        tok = token_of_row(dest, rows, k)
        dest2 = dest.view(T, k)
        buf = _Permute.apply(x, dest2, tok)
        y = expert_mlp_aligned(buf, seg, experts.gate_up_proj, experts.down_proj, **experts_mlp_kwargs(experts))
        return _Combine.apply(y, weights, dest2, tok)
    token_of_slot = torch.arange(T, device=x.device).repeat_interleave(k)
    buf = x.new_zeros((rows, H)).index_copy(0, dest, x.index_select(0, token_of_slot))
    y = expert_mlp_aligned(buf, seg, experts.gate_up_proj, experts.down_proj, **experts_mlp_kwargs(experts))
    y_slots = y.index_select(0, dest).reshape(T, k, H)
    if canonical:
        return canonical_combine(y_slots, weights)
    out = (y_slots.float() * weights.unsqueeze(-1).float()).sum(1)
    return out.to(x.dtype)
