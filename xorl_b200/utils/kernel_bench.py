"""Micro-benchmarks of the native kernels against their library counterparts.

    python -m xorl_b200.utils.kernel_bench gemm --m 4096 --n 6144 --k 4096
    python -m xorl_b200.utils.kernel_bench fp8_gemm --m 4096 --n 4096 --k 4096
    python -m xorl_b200.utils.kernel_bench attn --tokens 4096 --heads 32 --kv-heads 8
    python -m xorl_b200.utils.kernel_bench adamw --numel 268435456
    python -m xorl_b200.utils.kernel_bench rmsnorm --tokens 16384 --hidden 4096
    python -m xorl_b200.utils.kernel_bench conv1d --tokens 32768 --hidden 8192 --doc-len 4096
    python -m xorl_b200.utils.kernel_bench dequant4 --n 12288 --k 4096
    python -m xorl_b200.utils.kernel_bench symgemm --m 4096 --k 12288 --block 1024
    python -m xorl_b200.utils.kernel_bench grouped --experts 16 --m 32768 --k 2048 --n 1536

Timing: CUDA events on the launching stream around each run, ``--warmup`` untimed runs, the median
of ``--iters`` runs, and a buffer larger than L2 written between runs.  ``--no-lib`` skips the
library comparison (useful under a profiler, where only the native kernel is of interest).
One JSON line per case on stdout.
"""
from __future__ import annotations

import argparse
import json
import statistics
from typing import Callable, Dict

import torch


def _time(fn: Callable[[], None], warmup: int, iters: int, flush: torch.Tensor) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def bench_gemm(a) -> Dict:
    from ..ops import gemm as gemm_mod
    from ..ops.gemm import gemm
    gemm_mod.set_variant(a.variant)
    A = torch.randn(a.k, a.m, device="cuda").bfloat16() if a.a_mn else torch.randn(a.m, a.k, device="cuda").bfloat16()
    B = torch.randn(a.k, a.n, device="cuda").bfloat16() if a.b_mn else torch.randn(a.n, a.k, device="cuda").bfloat16()
    C = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: gemm(A, B, a_mn=a.a_mn, b_mn=a.b_mn, out=C), a.warmup, a.iters, a.flush)
    flops = 2.0 * a.m * a.n * a.k
    r = {"kernel": "gemm_bf16", "variant": a.variant, "m": a.m, "n": a.n, "k": a.k, "a_mn": a.a_mn, "b_mn": a.b_mn, "ms": ms,
         "tflops": flops / ms / 1e9}
    if not a.no_lib:
        Am = A.t() if a.a_mn else A
        Bm = B if a.b_mn else B.t()
        ms2 = _time(lambda: torch.matmul(Am, Bm, out=C), a.warmup, a.iters, a.flush)
        r.update(lib_ms=ms2, lib_tflops=flops / ms2 / 1e9, ratio=ms2 / ms)
    return r


def bench_fp8_gemm(a) -> Dict:
    from ..ops import fp8_gemm
    A = torch.randn(a.m, a.k, device="cuda").bfloat16()
    B = torch.randn(a.n, a.k, device="cuda").bfloat16()
    aq, as_ = fp8_gemm.quantize_rows(A)
    bq, bs = fp8_gemm.quantize_blocks(B)
    ms = _time(lambda: fp8_gemm.block_fp8_gemm(aq, as_, bq, bs), a.warmup, a.iters, a.flush)
    msq = _time(lambda: fp8_gemm.quantize_rows(A), a.warmup, a.iters, a.flush)
    flops = 2.0 * a.m * a.n * a.k
    r = {"kernel": "block_fp8_gemm", "m": a.m, "n": a.n, "k": a.k, "ms": ms, "tflops": flops / ms / 1e9,
         "quant_rows_ms": msq, "quant_rows_gbs": (a.m * a.k * 3 + a.m * a.k / 32) / msq / 1e6}
    if not a.no_lib:
        C = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        ms2 = _time(lambda: torch.matmul(A, B.t(), out=C), a.warmup, a.iters, a.flush)
        r.update(lib_bf16_ms=ms2, lib_bf16_tflops=flops / ms2 / 1e9)
    return r


def bench_attn(a) -> Dict:
    from ..ops import attention as attn_mod
    from ..ops.attention import flash_attn_varlen
    attn_mod.set_backward_mode(a.attn_bwd)
    T, Hq, Hkv, D = a.tokens, a.heads, a.kv_heads, 128
    q = torch.randn(T, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(T, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(T, Hkv, D, device="cuda").bfloat16().requires_grad_()
    lens = [a.doc_len] * (T // a.doc_len) if a.doc_len else [T]
    if sum(lens) < T:
        lens.append(T - sum(lens))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    do = torch.randn(T, Hq, D, device="cuda").bfloat16()
    fl = sum(2.0 * 2 * L * L * Hq * D / 2 for L in lens)           # causal: half of QK^T and PV
    holder = {}

    def fwd():
        holder["o"] = flash_attn_varlen(q, k, v, cu, causal=True)

    ms_f = _time(fwd, a.warmup, a.iters, a.flush)

    def bwd():
        holder["o"].backward(do, retain_graph=True)

    fwd()
    ms_b = _time(bwd, a.warmup, a.iters, a.flush)
    r = {"kernel": "flash_attn", "bwd_mode": a.attn_bwd, "tokens": T, "heads": Hq, "kv_heads": Hkv, "docs": len(lens), "fwd_ms": ms_f,
         "fwd_tflops": fl / ms_f / 1e9, "bwd_ms": ms_b, "bwd_tflops": 2.5 * fl / ms_b / 1e9}
    if not a.no_lib:
        try:
            from flash_attn import flash_attn_varlen_func
            qq, kk, vv = (t.detach().clone().requires_grad_() for t in (q, k, v))

            def lf():
                holder["lo"] = flash_attn_varlen_func(qq, kk, vv, cu, cu, max(lens), max(lens), causal=True)

            ms_lf = _time(lf, a.warmup, a.iters, a.flush)
            lf()
            ms_lb = _time(lambda: holder["lo"].backward(do, retain_graph=True), a.warmup, a.iters, a.flush)
            r.update(lib="flash_attn2", lib_fwd_ms=ms_lf, lib_bwd_ms=ms_lb)
        except Exception as e:  # noqa: BLE001
            r["lib_error"] = str(e)[:100]
        # torch SDPA on the cuDNN backend (the library's Blackwell attention); equal-length documents only:
        # they become the batch dimension
        if len(set(lens)) == 1:
            try:
                from torch.nn.attention import SDPBackend, sdpa_kernel
                B, L = len(lens), lens[0]
                q4, k4, v4 = (t.detach().view(B, L, -1, D).transpose(1, 2).contiguous().requires_grad_()
                              for t in (q, k, v))
                do4 = do.view(B, L, Hq, D).transpose(1, 2).contiguous()

                def cf():
                    with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                        holder["co"] = torch.nn.functional.scaled_dot_product_attention(
                            q4, k4, v4, is_causal=True, enable_gqa=Hq != Hkv)

                ms_cf = _time(cf, a.warmup, a.iters, a.flush)
                cf()
                ms_cb = _time(lambda: holder["co"].backward(do4, retain_graph=True), a.warmup, a.iters, a.flush)
                r.update(cudnn_fwd_ms=ms_cf, cudnn_fwd_tflops=fl / ms_cf / 1e9, cudnn_bwd_ms=ms_cb,
                         cudnn_bwd_tflops=2.5 * fl / ms_cb / 1e9)
            except Exception as e:  # noqa: BLE001
                r["cudnn_error"] = str(e)[:160]
    return r


def bench_fused_gemm(a) -> Dict:
    """The collective GEMM kernel on one device (``--ranks`` local buffers stand in for the peers):
    what the gather warps, the rotated raster and the completion counters cost next to the plain
    CTA-pair GEMM, without any NVLink traffic."""
    from ..ops.fused_gemm import Peers, ag_gemm, gemm_rs
    from ..ops.gemm import gemm
    R = a.ranks
    A = torch.randn(a.m, a.k, device="cuda").bfloat16()
    B = torch.randn(a.n, a.k, device="cuda").bfloat16()
    C = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    shards = [A[r * (a.m // R):(r + 1) * (a.m // R)].clone() for r in range(R)]
    full = torch.empty_like(A)
    ptrs = [s_.data_ptr() for s_ in shards]
    peers = Peers(R // 2, R)
    partial = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    ms_plain = _time(lambda: gemm(A, B, out=C), a.warmup, a.iters, a.flush)
    ms_ag = _time(lambda: ag_gemm(full, ptrs, a.m // R, B, peers, gathered="a", out=C), a.warmup, a.iters, a.flush)
    ms_rs = _time(lambda: gemm_rs(A, B, partial, [partial.data_ptr()] * R, a.m // R, peers), a.warmup, a.iters, a.flush)
    flops = 2.0 * a.m * a.n * a.k
    return {"kernel": "gemm_fused_one_device", "m": a.m, "n": a.n, "k": a.k, "ranks": R, "plain_ms": ms_plain,
            "gather_ms": ms_ag, "partial_ms": ms_rs, "plain_tflops": flops / ms_plain / 1e9,
            "gather_tflops": flops / ms_ag / 1e9, "partial_tflops": flops / ms_rs / 1e9}


def bench_adamw(a) -> Dict:
    from ..ops import optim as optim_ops
    n = a.numel
    w = torch.randn(n, device="cuda")
    m, v, g = torch.zeros_like(w), torch.zeros_like(w), torch.randn(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: optim_ops.adamw_step_(w, m, v, g, lp, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                             weight_decay=0.01, step=3, grad_scale=1.0, clip_coef=None),
               a.warmup, a.iters, a.flush)
    nbytes = n * (4 * 4 + 3 * 4 + 2)          # read w,m,v,g; write w,m,v and the bf16 copy
    return {"kernel": "adamw", "numel": n, "ms": ms, "gbs": nbytes / ms / 1e6}


def bench_rmsnorm(a) -> Dict:
    from ..ops.norm import rmsnorm
    x = torch.randn(a.tokens, a.hidden, device="cuda").bfloat16()
    w = torch.ones(a.hidden, device="cuda").bfloat16()
    ms = _time(lambda: rmsnorm(x, w, 1e-6), a.warmup, a.iters, a.flush)
    return {"kernel": "rmsnorm_fwd", "tokens": a.tokens, "hidden": a.hidden, "ms": ms,
            "gbs": a.tokens * a.hidden * 4 / ms / 1e6}


def bench_conv1d(a) -> Dict:
    """Short causal convolution + SiLU over a packed batch (forward, and forward + backward)."""
    from ..ops import seqmix
    T, C, K = a.tokens, a.hidden, 4
    x = torch.randn(T, C, device="cuda").bfloat16().requires_grad_()
    w = torch.randn(C, K, device="cuda").bfloat16().requires_grad_()
    doc = a.doc_len or T
    cu = torch.arange(0, T + 1, doc, device="cuda", dtype=torch.int32)
    start = seqmix.document_starts(cu, T)
    dy = torch.randn(T, C, device="cuda").bfloat16()
    with torch.no_grad():
        ms_f = _time(lambda: seqmix.causal_conv1d(x, w, None, cu, True, doc_start=start), a.warmup, a.iters, a.flush)

    def fb():
        x.grad = w.grad = None
        seqmix.causal_conv1d(x, w, None, cu, True, doc_start=start).backward(dy)
    ms_fb = _time(fb, a.warmup, a.iters, a.flush)
    r = {"kernel": "causal_conv1d_silu", "tokens": T, "channels": C, "taps": K, "fwd_ms": ms_f,
         "fwd_gbs": T * C * 4 / ms_f / 1e6, "fwd_bwd_ms": ms_fb}
    if not a.no_lib:
        import torch.nn.functional as F
        xt = x.detach().t().unsqueeze(0).contiguous()

        def lib():
            F.silu(F.conv1d(F.pad(xt, (K - 1, 0)), w.detach().unsqueeze(1), groups=C))
        ms2 = _time(lib, a.warmup, a.iters, a.flush)
        r.update(lib_fwd_ms=ms2, ratio=ms2 / ms_f)
    return r


def bench_dequant4(a) -> Dict:
    from ..ops import quantize as Q, seqmix
    shape = (a.n, a.k)
    out = {}
    for fmt, group in (("nf4", 64), ("nvfp4", 16)):
        parts = {k: v.cuda() for k, v in Q.quantize_weight(torch.randn(64, a.k) * 0.05, fmt, group).items()}
        reps = a.n // 64                       # quantise a slab on the host, tile it on the device
        for key in ("packed", "scale"):
            parts[key] = parts[key].repeat(reps)
        ms = _time(lambda: seqmix.dequant4(parts, fmt, group, shape), a.warmup, a.iters, a.flush)
        out[fmt + "_ms"] = ms
        out[fmt + "_out_gbs"] = a.n * a.k * 2 / ms / 1e6
    return {"kernel": "dequant4", "n": a.n, "k": a.k, **out}


def bench_symgemm(a) -> Dict:
    """X X^T (the Gram product of Muon's Newton-Schulz step): full GEMM against lower panels + mirror."""
    from ..ops.gemm import gemm, gemm_symmetric
    X = (torch.randn(a.m, a.k, device="cuda") * 0.05).bfloat16()
    ms_full = _time(lambda: gemm(X, X), a.warmup, a.iters, a.flush)
    ms_sym = _time(lambda: gemm_symmetric(X, block=a.block, min_rows=0), a.warmup, a.iters, a.flush)
    flops = 2.0 * a.m * a.m * a.k
    r = {"kernel": "gemm_symmetric", "m": a.m, "k": a.k, "block": a.block, "full_ms": ms_full, "sym_ms": ms_sym,
         "full_tflops": flops / ms_full / 1e9, "sym_effective_tflops": flops / ms_sym / 1e9,
         "speedup": ms_full / ms_sym}
    if not a.no_lib:
        C = torch.empty(a.m, a.m, device="cuda", dtype=torch.bfloat16)
        ms2 = _time(lambda: torch.matmul(X, X.t(), out=C), a.warmup, a.iters, a.flush)
        r.update(lib_ms=ms2, lib_tflops=flops / ms2 / 1e9)
    return r


BENCHES = {"symgemm": bench_symgemm, "conv1d": bench_conv1d, "dequant4": bench_dequant4, "gemm": bench_gemm, "fp8_gemm": bench_fp8_gemm, "attn": bench_attn, "adamw": bench_adamw,
           "rmsnorm": bench_rmsnorm, "fused_gemm": bench_fused_gemm}


def bench_grouped(a) -> Dict:
    """Grouped expert GEMM (rows mode): bf16 tcgen05 kernel, block-scaled fp8 kernel (operands
    quantised beforehand; the row quantiser is timed separately) and ``torch._grouped_mm``.
    ``--m`` rows are spread over ``--experts`` experts with an uneven load (+-12 %)."""
    from ..ops import fp8_grouped as fg
    from ..ops import moe as moe_ops
    E, K, N = a.experts, a.k, a.n
    base = a.m // E
    counts = [base + (base // 8) * ((i % 3) - 1) for i in range(E)]
    ids = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)]).cuda()
    dest, seg, _ = moe_ops.aligned_sort_indices(ids, E)
    rows = moe_ops.buffer_rows(ids.numel(), E)
    x = torch.zeros(rows, K, device="cuda", dtype=torch.bfloat16)
    x[dest] = torch.randn(ids.numel(), K, device="cuda").bfloat16()
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16()
    out = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * sum(counts) * K * N
    ms_bf16 = _time(lambda: moe_ops._grouped_rows_cuda(x, w, seg, out, b_kmajor=False), a.warmup, a.iters, a.flush)
    xq, sfx = fg.quantize_rows(x)
    qe = fg.quantize_experts(w)
    ms_fp8 = _time(lambda: fg.grouped_rows_mx(xq, sfx, qe.q_nk, qe.sf_nk, seg, out), a.warmup, a.iters, a.flush)
    ms_q = _time(lambda: fg.quantize_rows(x), a.warmup, a.iters, a.flush)
    ms_wq = _time(lambda: fg.quantize_experts(w), a.warmup, a.iters, a.flush)
    r = {"kernel": "grouped_gemm_rows", "experts": E, "rows": sum(counts), "k": K, "n": N,
         "bf16_ms": ms_bf16, "bf16_tflops": flops / ms_bf16 / 1e9, "fp8_ms": ms_fp8, "fp8_tflops": flops / ms_fp8 / 1e9,
         "fp8_over_bf16": ms_bf16 / ms_fp8, "row_quant_ms": ms_q, "weight_quant_ms": ms_wq}
    if not a.no_lib and hasattr(torch, "_grouped_mm"):
        xs = torch.randn(sum(counts), K, device="cuda").bfloat16()
        offs = torch.tensor(counts, device="cuda").cumsum(0).to(torch.int32)
        try:
            ms_lib = _time(lambda: torch._grouped_mm(xs, w, offs=offs), a.warmup, a.iters, a.flush)
            r.update(lib_ms=ms_lib, lib_tflops=flops / ms_lib / 1e9)
        except Exception as e:  # noqa: BLE001
            r["lib_error"] = str(e)[:120]
    return r


def bench_ce(a) -> Dict:
    """Cross-entropy over one chunk of logits (fp32 statistics, gradient written in place)."""
    from ..ops.loss import ce_chunk_
    V = a.n
    logits = torch.randn(a.tokens, V, device="cuda").bfloat16()
    labels = torch.randint(0, V, (a.tokens,), device="cuda")
    ms = _time(lambda: ce_chunk_(logits, labels, 1.0 / a.tokens, True), a.warmup, a.iters, a.flush)
    return {"kernel": "cross_entropy", "tokens": a.tokens, "vocab": V, "ms": ms,
            "gbs": a.tokens * V * 2 * 2 / ms / 1e6}          # logits read once, gradient written once


def bench_route(a) -> Dict:
    """Router: fp32 logits -> softmax, top-k, renormalised weights."""
    from ..ops.moe import expert_histogram, topk_route
    logits = torch.randn(a.tokens, a.experts, device="cuda")
    ms = _time(lambda: topk_route(logits, 8, True), a.warmup, a.iters, a.flush)
    idx = topk_route(logits, 8, True)[1]
    ms_h = _time(lambda: expert_histogram(idx, a.experts), a.warmup, a.iters, a.flush)
    return {"kernel": "moe_route", "tokens": a.tokens, "experts": a.experts, "k": 8, "ms": ms,
            "gbs": a.tokens * a.experts * 4 * 2 / ms / 1e6, "histogram_ms": ms_h}


def bench_qk_norm_rope(a) -> Dict:
    """Per-head qk RMSNorm + rotary embedding on the fused projection output, forward only."""
    from ..ops import _lib
    Hq, Hkv, D = a.heads, a.kv_heads, 128
    T = a.tokens
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    wq, wk = torch.ones(D, device="cuda").bfloat16(), torch.ones(D, device="cuda").bfloat16()
    pos = torch.arange(T, device="cuda")
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = pos[:, None].float() * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    qk = torch.empty(T, (Hq + Hkv) * D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.empty(T, Hq + Hkv, device="cuda", dtype=torch.float32)
    lib = _lib.cuda_lib()

    def run():
        _lib.check(lib.xb_qk_norm_rope_fwd(qkv.data_ptr(), qkv.stride(0), wq.data_ptr(), wk.data_ptr(), cos.data_ptr(),
                                           sin.data_ptr(), qk.data_ptr(), qk.stride(0), rstd.data_ptr(), T, Hq, Hkv, D,
                                           1e-6, 1, _lib.stream_ptr()), "xb_qk_norm_rope_fwd")
    try:
        ms = _time(run, a.warmup, a.iters, a.flush)
    except Exception as e:  # noqa: BLE001
        return {"kernel": "qk_norm_rope_fwd", "error": str(e)[:200]}
    return {"kernel": "qk_norm_rope_fwd", "tokens": T, "heads": Hq, "kv_heads": Hkv, "ms": ms,
            "gbs": T * (Hq + Hkv) * D * 2 * 2 / ms / 1e6}


def bench_permute(a) -> Dict:
    """MoE row gather (token -> expert-sorted buffer) and weighted combine (k rows -> token)."""
    from ..ops import moe as moe_ops
    T, k, H, E = a.tokens, 8, a.hidden, a.experts
    x = torch.randn(T, H, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(64)]).repeat(T // 64 + 1, 1)[:T]
    dest, seg, _ = moe_ops.aligned_sort_indices(idx.reshape(-1), E)
    rows = moe_ops.buffer_rows(T * k, E)
    tok = moe_ops.token_of_row(dest, rows, k)
    w = torch.rand(T, k, device="cuda")
    ms_g = _time(lambda: moe_ops._gather_rows(x, tok, rows), a.warmup, a.iters, a.flush)
    buf = moe_ops._gather_rows(x, tok, rows)
    d2 = dest.view(T, k)
    ms_c = _time(lambda: moe_ops._gather_sum(buf, d2, w), a.warmup, a.iters, a.flush)
    return {"kernel": "moe_permute", "tokens": T, "k": k, "hidden": H, "gather_ms": ms_g,
            "gather_gbs": (T * k * H * 2 * 2) / ms_g / 1e6, "combine_ms": ms_c,
            "combine_gbs": (T * k * H * 2 + T * H * 2) / ms_c / 1e6}


def bench_mx_quant(a) -> Dict:
    """Row quantiser of the block-scaled fp8 path (bf16 -> e4m3 + UE8M0 1 x 128 scales)."""
    from ..ops import fp8_grouped as fg
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    ms = _time(lambda: fg.quantize_rows(x), a.warmup, a.iters, a.flush)
    return {"kernel": "quant_mx_rows", "m": a.m, "k": a.k, "ms": ms, "gbs": a.m * a.k * 3 / ms / 1e6}


BENCHES["grouped"] = bench_grouped
BENCHES.update(ce=bench_ce, route=bench_route, qk_norm_rope=bench_qk_norm_rope, permute=bench_permute,
               mx_quant=bench_mx_quant)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=sorted(BENCHES))
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--variant", choices=["single", "pair"], default="pair")
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--doc-len", type=int, default=0)
    ap.add_argument("--attn-bwd", choices=["split", "fused"], default="split")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-lib", action="store_true")
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--block", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=16)
    a = ap.parse_args(argv)
    a.flush = torch.zeros(256 << 20, device="cuda", dtype=torch.uint8)
    print(json.dumps(BENCHES[a.kernel](a)))


if __name__ == "__main__":
    main()
