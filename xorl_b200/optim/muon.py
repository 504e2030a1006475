"""Muon on ZeRO flat shards.

Matrices (2-D weights of the decoder layers, and every expert slice of stacked 3-D expert weights)
are updated with the orthogonalised momentum; everything else (embeddings, lm-head, norms, biases,
router gates) falls back to AdamW on the same shards (src/xorl/optim/muon.py:51-728).

A flat shard does not hold whole matrices, so a step does, per parameter group:
  1. momentum on the fp32 gradient shard (nesterov optional),
  2. one all-gather of the bf16 update direction over the shard group,
  3. Newton-Schulz on every matrix that overlaps this rank's shard (ranks whose shards miss a
     matrix skip it), either the classic quintic iteration on X or the Gram form that iterates on
     the small m x m Gram matrix and touches the m x n matrix only at the start, at restarts and
     at the end (src/xorl/optim/gram_newton_schulz.py),
  4. the update of the local slice of the fp32 master weights and their compute-dtype copy.
The result is the full-matrix update whatever the shard boundaries are, so ``shard_local`` and
``full_matrix`` distributed modes coincide here.  GEMMs run on the tcgen05 kernel when on GPU.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops.gemm import gemm, gemm_symmetric
from .optimizer import ShardedOptimizer

NS_COEFFS = (3.4445, -4.7750, 2.0315)
_FALLBACK_PATTERNS = ("embed_tokens", "lm_head", "norm", ".bias", ".gate.weight", "lora_")


def _mm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M,K] @ b[N,K]^T in bf16 with fp32 accumulation."""
    if a.is_cuda and a.shape[1] % 8 == 0:
        return gemm(a, b)
    return (a.float() @ b.float().t()).to(a.dtype)


def _mm_sym(a: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a @ b^T where the product is symmetric (b omitted: a @ a^T): block-lower panels + mirror."""
    if a.is_cuda and a.shape[1] % 8 == 0:
        return gemm_symmetric(a, b)
    b = a if b is None else b
    return (a.float() @ b.float().t()).to(a.dtype)


def _mm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M,K] @ b[K,N]."""
    if a.is_cuda and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
        return gemm(a, b, b_mn=True)
    return (a.float() @ b.float()).to(a.dtype)


def newton_schulz(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal polar factor of ``G`` [m, n]."""
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16)
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t().contiguous()
    X = X / (X.float().norm() + eps).to(X.dtype)
    for _ in range(steps):
        A = _mm_sym(X)                         # X X^T  (symmetric: lower panels + mirror)
        B = (b * A.float() + c * _mm_sym(A).float()).to(X.dtype)     # A symmetric: A A^T = A A
        X = (a * X.float() + _mm_nn(B, X).float()).to(X.dtype)
    return X.t().contiguous() if transposed else X


def gram_newton_schulz(G: torch.Tensor, steps: int = 5, restart_iterations: Sequence[int] = (2,),
                       eps: float = 1e-7) -> torch.Tensor:
    """The same iteration carried on the Gram matrix.  With A = X X^T and P = aI + bA + cA^2,
    X <- P X implies A <- P A P and the accumulated left factor Q <- P Q, all m x m; X itself is
    rebuilt as Q X0 only at ``restart_iterations`` (to stop rounding errors in A from drifting)
    and at the end.  Costs O(m^3) per step instead of O(m^2 n)."""
    a, b, c = NS_COEFFS
    X0 = G.to(torch.bfloat16)
    transposed = X0.shape[0] > X0.shape[1]
    if transposed:
        X0 = X0.t().contiguous()
    X0 = X0 / (X0.float().norm() + eps).to(X0.dtype)
    m = X0.shape[0]
    eye = torch.eye(m, device=X0.device, dtype=torch.float32)
    A = _mm_sym(X0).float()
    Q: Optional[torch.Tensor] = None
    for it in range(steps):
        if it in restart_iterations and Q is not None:
            X0 = _mm_nn(Q.to(torch.bfloat16), X0)
            A = _mm_sym(X0).float()
            Q = None
        A16 = A.to(torch.bfloat16)
        A2 = _mm_sym(A16).float()
        P = a * eye + b * A + c * A2
        P16 = P.to(torch.bfloat16)
        Q = P if Q is None else _mm_nt(P16, Q.t().contiguous().to(torch.bfloat16)).float()
        PA = _mm_nt(P16, A16).float()                     # P A      (A symmetric)
        A = _mm_nt(PA.to(torch.bfloat16), P16).float()    # P A P    (P symmetric)
        A = 0.5 * (A + A.t())
    X = _mm_nn(Q.to(torch.bfloat16), X0)
    return X.t().contiguous() if transposed else X


def adjusted_lr(lr: float, shape, fn: Optional[str]) -> float:
    rows, cols = shape[-2], shape[-1]
    if fn in (None, "original"):
        return lr * math.sqrt(max(1.0, rows / cols))
    if fn == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(rows, cols))
    raise ValueError(f"unknown muon_adjust_lr_fn {fn!r}")


class ShardedMuon(ShardedOptimizer):
    kind = "muon"

    def __init__(self, engine, lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, muon_lr: float = 0.02,
                 muon_momentum: float = 0.95, muon_nesterov: bool = True, muon_ns_steps: int = 5,
                 muon_adjust_lr_fn: Optional[str] = None, muon_ns_algorithm: str = "gram_newton_schulz",
                 muon_gram_ns_restart_iterations: Optional[List[int]] = None,
                 muon_gram_ns_num_restarts: int = 1, **kw):
        super().__init__(engine, lr, weight_decay, kw.get("no_decay_modules", ()), kw.get("no_decay_params", ()))
        self.betas, self.eps = betas, eps
        self.muon_lr, self.mu, self.nesterov = muon_lr, muon_momentum, muon_nesterov
        self.ns_steps, self.adjust = muon_ns_steps, muon_adjust_lr_fn
        self.algorithm = muon_ns_algorithm
        if muon_gram_ns_restart_iterations is None:
            n = max(0, muon_gram_ns_num_restarts)
            muon_gram_ns_restart_iterations = [round((i + 1) * muon_ns_steps / (n + 1)) for i in range(n)]
        self.restarts = tuple(muon_gram_ns_restart_iterations)
        self._base_lr = lr
        self.momentum = self._new_state("momentum_buffer")
        self.exp_avg = self._new_state("exp_avg")
        self.exp_avg_sq = self._new_state("exp_avg_sq")

    def set_lr(self, lr: float) -> None:
        """The scheduler drives the AdamW rate; the Muon rate follows it proportionally."""
        self.lr = lr

    def _muon_rate(self) -> float:
        return self.muon_lr * (self.lr / self._base_lr if self._base_lr else 1.0)

    def is_matrix_param(self, name: str, shape) -> bool:
        return len(shape) >= 2 and not any(p in name for p in _FALLBACK_PATTERNS)

    def _orthogonalise(self, M: torch.Tensor) -> torch.Tensor:
        if self.algorithm == "newton_schulz":
            return newton_schulz(M, self.ns_steps)
        return gram_newton_schulz(M, self.ns_steps, self.restarts)

    @torch.no_grad()
    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        mlr = self._muon_rate()
        for g in self.engine.all_groups():
            if getattr(g, "frozen", False) or not g.grad_ready:
                continue
            grad = g.grad_shard * grad_scale
            if clip_coef is not None:
                grad = grad * clip_coef
            mom = self.momentum[id(g)]
            segs = g.param_segments_in_shard()
            muon_segs = [(i, a, b) for i, a, b in segs if self.is_matrix_param(g.named_params[i][0], g.shapes[i])]
            any_muon = any(self.is_matrix_param(n, s) for (n, _), s in zip(g.named_params, g.shapes))
            # ---- AdamW fallback on everything that is not a matrix --------------------------------
            m, v = self.exp_avg[id(g)], self.exp_avg_sq[id(g)]
            for i, a, b in segs:
                name = g.named_params[i][0]
                if self.is_matrix_param(name, g.shapes[i]):
                    continue
                gs = grad[a:b]
                m[a:b].mul_(b1).add_(gs, alpha=1 - b1)
                v[a:b].mul_(b2).addcmul_(gs, gs, value=1 - b2)
                w = g.master[a:b]
                w.mul_(1 - self.lr * self._decay[name])
                w.addcdiv_(m[a:b] / bc1, (v[a:b] / bc2).sqrt_().add_(self.eps), value=-self.lr)
            if any_muon:
                # ---- momentum, gather of the update direction, orthogonalisation ------------------
                mom.mul_(self.mu).add_(grad)
                upd = (grad + self.mu * mom) if self.nesterov else mom
                upd16 = upd.to(torch.bfloat16)
                if g.world > 1:
                    full = torch.empty(g.padded, device=upd16.device, dtype=torch.bfloat16)
                    dist.all_gather_into_tensor(full, upd16.contiguous(), group=g.pg)
                else:
                    full = upd16
                s0, _ = g.shard_range()
                for i, a, b in muon_segs:
                    name, shape = g.named_params[i][0], g.shapes[i]
                    o, n = g.offsets[i], math.prod(shape)
                    M = full[o:o + n].view(shape)
                    lo, hi = s0 + a - o, s0 + b - o            # this rank's element range inside the param
                    w = g.master[a:b]
                    w.mul_(1 - mlr * self._decay[name])
                    rate = adjusted_lr(mlr, shape, self.adjust)
                    if len(shape) == 2:
                        O = self._orthogonalise(M).reshape(-1)
                        w.add_(O[lo:hi].float(), alpha=-rate)
                    else:
                        per = math.prod(shape[1:])
                        mats = M.reshape(-1, shape[-2], shape[-1])
                        for e in range(lo // per, (hi - 1) // per + 1):
                            O = self._orthogonalise(mats[e]).reshape(-1)
                            ea, eb = max(lo, e * per), min(hi, (e + 1) * per)
                            w[ea - lo:eb - lo].add_(O[ea - e * per:eb - e * per].float(), alpha=-rate)
            if g.shard_lp is not g.master:
                g.shard_lp.copy_(g.master)
