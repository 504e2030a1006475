"""Cross-entropy and the fused lm-head + cross-entropy (``csrc/loss.cu`` + tcgen05 GEMMs).

``fused_linear_cross_entropy`` never materialises ``[tokens, vocab]`` logits beyond one token
chunk (bf16) and computes the gradients of hidden states and lm-head weight in the same pass, in
the spirit of the reference's chunked lm-head loss (src/xorl/ops/loss/causallm_loss.py:445-864).
Loss reduction is a **sum** over valid tokens (labels != ignore_index); callers divide by the
global token count (src/xorl/distributed/gradient_accumulate_loss.py:7-64).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import gemm
from .grad_sink import deliver_param_grad, grad_target, mark_written

IGNORE_INDEX = -100
_launches = 0


def launch_count() -> int:
    return _launches


def cross_entropy_sum_reference(logits: torch.Tensor, labels: torch.Tensor,
                                ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    return F.cross_entropy(logits.float(), labels, ignore_index=ignore_index, reduction="sum")


def ce_chunk_(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float, write_grad: bool,
              ignore_index: int = IGNORE_INDEX, z_loss: float = 0.0):
    """Per-row losses and LSE of a bf16 logits chunk; rewrites ``logits`` with d(loss)/d(logits)
    times ``grad_scale`` when ``write_grad``."""
    global _launches
    rows, V = logits.shape
    loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
    lse = torch.empty(rows, device=logits.device, dtype=torch.float32)
    _lib.check(_lib.cuda_lib().xb_cross_entropy(logits.data_ptr(), logits.stride(0),
                                                labels.data_ptr(), loss.data_ptr(), lse.data_ptr(),
                                                rows, V, ignore_index, float(grad_scale),
                                                int(write_grad), float(z_loss), _lib.stream_ptr()),
               "xb_cross_entropy")
    _launches += 1
    return loss, lse


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, grad_scale, chunk_tokens, ignore_index, z_loss,
                want_logprobs):
        T, H = hidden.shape
        V = weight.shape[0]
        need_dh = hidden.requires_grad
        need_dw = weight.requires_grad
        dh = torch.empty_like(hidden) if need_dh else None
        tgt, fresh = grad_target(weight) if need_dw else (None, False)
        dw_local = None
        if need_dw and tgt is None:
            dw_local = torch.zeros((V, H), device=hidden.device, dtype=torch.float32)
        losses = torch.empty(T, device=hidden.device, dtype=torch.float32)
        ldv = (V + 7) // 8 * 8
        buf = torch.empty((min(chunk_tokens, T), ldv), device=hidden.device, dtype=torch.bfloat16)
        first = True
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            h = hidden[s:e]
            logits = buf[: e - s, :V]
            gemm(h, weight, out=logits)
            l, _ = ce_chunk_(logits, labels[s:e], grad_scale, need_dh or need_dw, ignore_index,
                             z_loss)
            losses[s:e] = l
            if need_dh:
                gemm(logits, weight, b_mn=True, out=dh[s:e])
            if need_dw:
                if tgt is not None:
                    gemm(logits, h, a_mn=True, b_mn=True, out=tgt, accumulate=not (fresh and first))
                else:
                    gemm(logits, h, a_mn=True, b_mn=True, out=dw_local, accumulate=True)
            first = False
        if need_dw and tgt is not None:
            mark_written(weight)
        ctx.dh = dh
        ctx.dw_local = dw_local
        ctx.weight = weight
        loss_sum = losses.sum()
        if want_logprobs:
            ctx.mark_non_differentiable(losses)
            return loss_sum * grad_scale, losses
        return loss_sum * grad_scale, None

    @staticmethod
    def backward(ctx, g, _g2):
        dh = ctx.dh
        if dh is not None:
            dh = dh * g.to(dh.dtype)
        dw = None
        if ctx.dw_local is not None:
            dw = deliver_param_grad(ctx.weight, ctx.dw_local * g)
        ctx.dh = ctx.dw_local = None
        return dh, dw, None, None, None, None, None, None


def fused_linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               grad_scale: float = 1.0, chunk_tokens: int = 1024,
                               ignore_index: int = IGNORE_INDEX, z_loss: float = 0.0,
                               return_token_losses: bool = False):
    """``grad_scale * sum_t CE(hidden[t] @ weight.T, labels[t])``.

    The lm-head weight gradient is produced during the forward call with the scale folded in, so
    the returned scalar must be back-propagated with an upstream gradient of 1 (``loss.backward()``
    directly on it or on a sum it is part of).
    """
    if hidden.is_cuda and hidden.dtype == torch.bfloat16 and hidden.shape[-1] % 8 == 0:
        loss, tl = _FusedLinearCE.apply(hidden.reshape(-1, hidden.shape[-1]), weight,
                                        labels.reshape(-1), float(grad_scale), int(chunk_tokens),
                                        int(ignore_index), float(z_loss), bool(return_token_losses))
        return (loss, tl) if return_token_losses else loss
    # CPU / fp32 lane: chunked plain torch, same reduction
    h2 = hidden.reshape(-1, hidden.shape[-1])
    lab = labels.reshape(-1)
    total = hidden.new_zeros((), dtype=torch.float32)
    tls = []
    for s in range(0, h2.shape[0], chunk_tokens):
        logits = F.linear(h2[s:s + chunk_tokens], weight).float()
        tl = F.cross_entropy(logits, lab[s:s + chunk_tokens], ignore_index=ignore_index,
                             reduction="none")
        if z_loss:
            lse = torch.logsumexp(logits, dim=-1)
            tl = tl + z_loss * lse.pow(2) * (lab[s:s + chunk_tokens] != ignore_index)
        total = total + tl.sum()
        tls.append(tl.detach())
    loss = total * grad_scale
    return (loss, torch.cat(tls)) if return_token_losses else loss


# --------------------------------------------------------------------------------------------
# losses that are functions of per-token log-probabilities (RL, distillation)
# --------------------------------------------------------------------------------------------
def fused_linear_token_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                            loss_fn, grad_scale: float = 1.0, chunk_tokens: int = 1024,
                            ignore_index: int = IGNORE_INDEX):
    """``loss_fn(logprobs [T], mask [T]) -> (scalar, metrics)`` evaluated on the log-probabilities of
    the label tokens, without materialising the logits: pass 1 computes the log-probs chunk by
    chunk, the loss function runs on that small vector, pass 2 recomputes each logits chunk and
    back-propagates d(loss)/d(logprob) through the lm-head.  Returns (grad_scale * loss, logprobs,
    metrics); the hidden-state and lm-head gradients are produced like in
    ``fused_linear_cross_entropy`` (back-propagate the returned scalar with gradient 1)."""
    global _launches
    h2 = hidden.reshape(-1, hidden.shape[-1])
    lab = labels.reshape(-1)
    mask = (lab != ignore_index).float()
    if not (h2.is_cuda and h2.dtype == torch.bfloat16):
        lps = []
        for s in range(0, h2.shape[0], chunk_tokens):
            logits = F.linear(h2[s:s + chunk_tokens], weight).float()
            lps.append(-F.cross_entropy(logits, lab[s:s + chunk_tokens], ignore_index=ignore_index,
                                        reduction="none"))
        lp = torch.cat(lps)
        loss, metrics = loss_fn(lp, mask)
        return loss * grad_scale, lp.detach(), metrics
    T, H = h2.shape
    V = weight.shape[0]
    ldv = (V + 7) // 8 * 8
    buf = torch.empty((min(chunk_tokens, T), ldv), device=h2.device, dtype=torch.bfloat16)
    lp = torch.empty(T, device=h2.device, dtype=torch.float32)
    with torch.no_grad():
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            logits = buf[: e - s, :V]
            gemm(h2[s:e], weight, out=logits)
            l, _ = ce_chunk_(logits, lab[s:e], 0.0, False, ignore_index)
            lp[s:e] = -l
    if not torch.is_grad_enabled():
        # evaluation (log-probabilities only): there is nothing to differentiate
        loss, metrics = loss_fn(lp, mask)
        return loss * grad_scale, lp, metrics
    lp_leaf = lp.clone().requires_grad_()
    loss, metrics = loss_fn(lp_leaf, mask)
    (coef,) = torch.autograd.grad(loss, lp_leaf)
    return _TokenLossBackward.apply(h2, weight, lab, (-coef).contiguous(), float(grad_scale),
                                    int(chunk_tokens), int(ignore_index), loss.detach()), lp, metrics


class _TokenLossBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, row_scale, grad_scale, chunk_tokens, ignore_index, loss_value):
        global _launches
        T, H = hidden.shape
        V = weight.shape[0]
        need_dh, need_dw = hidden.requires_grad, weight.requires_grad
        dh = torch.empty_like(hidden) if need_dh else None
        tgt, fresh = grad_target(weight) if need_dw else (None, False)
        dw_local = torch.zeros((V, H), device=hidden.device, dtype=torch.float32) \
            if (need_dw and tgt is None) else None
        ldv = (V + 7) // 8 * 8
        buf = torch.empty((min(chunk_tokens, T), ldv), device=hidden.device, dtype=torch.bfloat16)
        lib = _lib.cuda_lib()
        scratch = torch.empty(min(chunk_tokens, T), device=hidden.device, dtype=torch.float32)
        first = True
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            logits = buf[: e - s, :V]
            gemm(hidden[s:e], weight, out=logits)
            _lib.check(lib.xb_cross_entropy_rows(logits.data_ptr(), logits.stride(0),
                                                 labels[s:e].data_ptr(), scratch.data_ptr(), None,
                                                 row_scale[s:e].data_ptr(), e - s, V, ignore_index,
                                                 grad_scale, 1, _lib.stream_ptr()),
                       "xb_cross_entropy_rows")
            _launches += 1
            if need_dh:
                gemm(logits, weight, b_mn=True, out=dh[s:e])
            if need_dw:
                if tgt is not None:
                    gemm(logits, hidden[s:e], a_mn=True, b_mn=True, out=tgt, accumulate=not (fresh and first))
                else:
                    gemm(logits, hidden[s:e], a_mn=True, b_mn=True, out=dw_local, accumulate=True)
            first = False
        if need_dw and tgt is not None:
            mark_written(weight)
        ctx.dh, ctx.dw_local, ctx.weight = dh, dw_local, weight
        return loss_value * grad_scale

    @staticmethod
    def backward(ctx, g):
        dh = ctx.dh * g.to(ctx.dh.dtype) if ctx.dh is not None else None
        dw = deliver_param_grad(ctx.weight, ctx.dw_local * g) if ctx.dw_local is not None else None
        ctx.dh = ctx.dw_local = None
        return dh, dw, None, None, None, None, None, None


# --------------------------------------------------------------------------------------------
# vocab-parallel head (tensor-parallel lm-head)
# --------------------------------------------------------------------------------------------
class _VocabParallelLinearCE(torch.autograd.Function):
    """Every rank of ``group`` holds rows [vocab_start, vocab_start + V_local) of the lm-head and
    the same hidden states.  Per chunk: local logits -> (max, sum-exp, target logit) -> three small
    all-reduces give the global log-sum-exp -> local gradient of the logits -> partial hidden
    gradient (all-reduced over the group at the end) and this rank's rows of the weight gradient.
    The full [T, V] logits never exist on any rank (src/xorl/ops/loss/vocab_parallel_cross_entropy.py)."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, group, vocab_start, grad_scale, chunk_tokens, ignore_index, pooled=False):
        import torch.distributed as dist
        global _launches
        T, H = hidden.shape
        Vl = weight.shape[0]
        cuda = hidden.is_cuda and hidden.dtype == torch.bfloat16
        need_dh, need_dw = hidden.requires_grad, weight.requires_grad
        # pooled: every rank of the group brings T tokens of its own.  Chunk by chunk the group's tokens are
        # gathered (rank order), taken through this rank's vocabulary rows, and the hidden gradient of the
        # chunk is reduce-scattered back so that each rank keeps the summed gradient of its own tokens: the
        # gathered hidden states and their gradient exist one chunk at a time
        # (src/xorl/ops/loss/causallm_loss.py:46-192 streams the same way and all-reduces the gradient)
        L = dist.get_world_size(group) if pooled else 1
        nccl = pooled and dist.get_backend(group) == "nccl"
        if pooled:
            chunk_tokens = max(8, chunk_tokens // L // 8 * 8)

        def pool(x):
            out = x.new_empty((L * x.shape[0],) + tuple(x.shape[1:]))
            dist.all_gather_into_tensor(out, x.contiguous(), group=group)
            return out
        dh = torch.zeros_like(hidden, dtype=torch.float32 if not cuda else hidden.dtype) if need_dh else None
        tgt, fresh = grad_target(weight) if (need_dw and cuda) else (None, False)
        dw_local = torch.zeros((Vl, H), device=hidden.device, dtype=torch.float32) if (need_dw and tgt is None) else None
        total = torch.zeros((), device=hidden.device, dtype=torch.float32)
        ldv = (Vl + 7) // 8 * 8
        buf = torch.empty((min(chunk_tokens, T) * L, ldv), device=hidden.device, dtype=torch.bfloat16) if cuda else None
        first = True
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            h, lab = hidden[s:e], labels[s:e]
            if pooled:
                h, lab = pool(h), pool(lab)
                s0, s, e = s, 0, h.shape[0]             # the body below indexes the pooled chunk
            valid = lab != ignore_index
            if cuda:
                logits = buf[: e - s, :Vl]
                gemm(h, weight, out=logits)
                stats = torch.empty((e - s, 3), device=h.device, dtype=torch.float32)
                _lib.check(_lib.cuda_lib().xb_cross_entropy_vp_stats(
                    logits.data_ptr(), logits.stride(0), lab.data_ptr(), stats.data_ptr(), e - s, Vl,
                    int(vocab_start), ignore_index, _lib.stream_ptr()), "xb_cross_entropy_vp_stats")
                _launches += 1
                m, se, tl = stats[:, 0].contiguous(), stats[:, 1].contiguous(), stats[:, 2].contiguous()
            else:
                logits = F.linear(h, weight).float()
                m = logits.max(-1).values
                se = torch.exp(logits - m[:, None]).sum(-1)
                lt = lab - vocab_start
                mine = valid & (lt >= 0) & (lt < Vl)
                tl = torch.where(mine, logits.gather(1, lt.clamp(0, Vl - 1)[:, None])[:, 0], torch.zeros_like(m))
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
            se = se * torch.exp(m - gm)
            packed = torch.stack([se, tl])
            dist.all_reduce(packed, group=group)
            lse = gm + torch.log(packed[0])
            total = total + torch.where(valid, lse - packed[1], torch.zeros_like(lse)).sum()
            if not (need_dh or need_dw):
                continue
            if cuda:
                _lib.check(_lib.cuda_lib().xb_cross_entropy_vp_grad(
                    logits.data_ptr(), logits.stride(0), lab.data_ptr(), lse.contiguous().data_ptr(), e - s, Vl,
                    int(vocab_start), ignore_index, float(grad_scale), _lib.stream_ptr()), "xb_cross_entropy_vp_grad")
                _launches += 1
                g = logits
                if need_dh and pooled:
                    part = torch.empty((e, H), device=h.device, dtype=dh.dtype)
                    gemm(g, weight, b_mn=True, out=part)
                    dist.reduce_scatter_tensor(dh[s0:s0 + e // L], part, group=group)
                elif need_dh:
                    gemm(g, weight, b_mn=True, out=dh[s:e])
                if need_dw:
                    if tgt is not None:
                        gemm(g, h, a_mn=True, b_mn=True, out=tgt, accumulate=not (fresh and first))
                    else:
                        gemm(g, h, a_mn=True, b_mn=True, out=dw_local, accumulate=True)
            else:
                g = torch.exp(logits - lse[:, None])
                lt = lab - vocab_start
                mine = valid & (lt >= 0) & (lt < Vl)
                rows = torch.nonzero(mine)[:, 0]
                g[rows, lt[rows]] -= 1.0
                g = g * (valid[:, None] * grad_scale)
                if need_dh and pooled:
                    part = g @ weight.float()
                    if nccl:
                        dist.reduce_scatter_tensor(dh[s0:s0 + e // L], part, group=group)
                    else:
                        dist.all_reduce(part, group=group)
                        r = dist.get_rank(group)
                        dh[s0:s0 + e // L] = part[r * (e // L):(r + 1) * (e // L)]
                elif need_dh:
                    dh[s:e] = g @ weight.float()
                if need_dw:
                    dw_local += g.t() @ h.float()
            first = False
        if need_dh and not pooled:
            dist.all_reduce(dh, group=group)
        if need_dw and tgt is not None:
            mark_written(weight)
        ctx.dh, ctx.dw_local, ctx.weight = dh, dw_local, weight
        ctx.h_dtype = hidden.dtype
        return total * grad_scale

    @staticmethod
    def backward(ctx, g):
        dh = (ctx.dh * g).to(ctx.h_dtype) if ctx.dh is not None else None
        dw = None
        if ctx.dw_local is not None:
            dw = deliver_param_grad(ctx.weight, ctx.dw_local * g)
        ctx.dh = ctx.dw_local = None
        return dh, dw, None, None, None, None, None, None, None


def vocab_parallel_linear_cross_entropy(hidden, weight_shard, labels, group, vocab_start: int,
                                        grad_scale: float = 1.0, chunk_tokens: int = 1024,
                                        ignore_index: int = IGNORE_INDEX, pooled: bool = False):
    """``grad_scale * sum_t CE`` with the lm-head sharded by vocabulary rows over ``group``.  The hidden
    states (and labels) are replicated over the group, or, with ``pooled``, every rank brings the same
    number of tokens of its own and the result is the loss of the whole group's tokens (the same value on
    every rank; the hidden gradient is that of this rank's tokens).  Back-propagate the result with an
    upstream gradient of 1, as for ``fused_linear_cross_entropy``."""
    return _VocabParallelLinearCE.apply(hidden.reshape(-1, hidden.shape[-1]), weight_shard, labels.reshape(-1),
                                        group, int(vocab_start), float(grad_scale), int(chunk_tokens),
                                        int(ignore_index), bool(pooled))


def distillation_kl(hidden_s: torch.Tensor, w_s: torch.Tensor, hidden_t: torch.Tensor, w_t: torch.Tensor,
                    labels: torch.Tensor, kind: str = "forward_kl", chunk_tokens: int = 1024,
                    ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """Sum over supervised tokens of the KL divergence between the teacher's and the student's
    next-token distributions: ``forward_kl`` = KL(teacher || student), ``reverse_kl`` =
    KL(student || teacher).  Logits are formed chunk by chunk from the final hidden states and the two
    lm-head weights (the student's through the differentiable linear, so its gradients reach the
    hidden states and the lm-head like any other loss term); the teacher's side carries no gradient.
    Keys: ``distill.distillation_loss_type`` (src/xorl/arguments.py:1846-1849)."""
    from .gemm import linear
    if kind not in ("forward_kl", "reverse_kl"):
        raise ValueError(f"distillation_loss_type must be forward_kl or reverse_kl, got {kind!r}")
    hs = hidden_s.reshape(-1, hidden_s.shape[-1])
    ht = hidden_t.reshape(-1, hidden_t.shape[-1])
    lab = labels.reshape(-1)
    if w_s.shape[0] != w_t.shape[0]:
        raise ValueError(f"teacher and student vocabularies differ: {w_t.shape[0]} vs {w_s.shape[0]}")
    total = hs.new_zeros((), dtype=torch.float32)
    for s in range(0, hs.shape[0], chunk_tokens):
        e = min(hs.shape[0], s + chunk_tokens)
        mask = (lab[s:e] != ignore_index).float()
        logp_s = torch.log_softmax(linear(hs[s:e], w_s).float(), dim=-1)
        with torch.no_grad():
            logp_t = torch.log_softmax(linear(ht[s:e], w_t).float(), dim=-1)
        if kind == "forward_kl":
            kl = (logp_t.exp() * (logp_t - logp_s)).sum(-1)
        else:
            kl = (logp_s.exp() * (logp_s - logp_t)).sum(-1)
        total = total + (kl * mask).sum()
    return total
