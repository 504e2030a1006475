"""Fused collective GEMMs (csrc/gemm_fused.cu) on one device: every "rank" is a buffer of the same
GPU and the kernel runs without handshakes, so gather order, chunk counters, staging stores and the
reduction are checked against plain fp32 PyTorch.  The two-GPU run with real peers is in
test_comm_gpu.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K,R,rank,gathered", [
    (2048, 1024, 512, 4, 1, "a"),
    (1536, 768, 256, 4, 3, "a"),       # 384 rows per rank: chunks straddle two shards
    (4096, 6144, 4096, 8, 5, "a"),
    (1024, 2048, 512, 4, 2, "b"),
    (4096, 4096, 1024, 8, 7, "b"),
    (640, 1536, 320, 2, 1, "b"),       # 768 rows per rank, partial M tile
])
def test_ag_gemm_one_device(M, N, K, R, rank, gathered):
    from xorl_b200.ops import _lib
    from xorl_b200.ops.fused_gemm import Peers, ag_gemm
    torch.manual_seed(0)
    rows = M if gathered == "a" else N
    assert rows % R == 0
    per = rows // R
    shards = [_rand(per, K) for _ in range(R)]
    other = _rand(N, K) if gathered == "a" else _rand(M, K)
    full = torch.full((rows, K), float("nan"), device="cuda", dtype=torch.bfloat16)
    peers = Peers(rank=rank, nranks=R)
    for _ in range(2):           # the second call exercises the monotonic chunk counters
        full.fill_(float("nan"))
        out = ag_gemm(full, [s.data_ptr() for s in shards], per, other, peers, gathered=gathered)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    ref_full = torch.cat(shards, 0)
    assert torch.equal(full, ref_full)
    a, b = (ref_full, other) if gathered == "a" else (other, ref_full)
    ref = a.float() @ b.float().t()
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err


def test_ag_gemm_transposed_weight():
    """dX = all_gather(dY) @ W with W stored [N_in, K_out] (b_mn)."""
    from xorl_b200.ops import _lib
    from xorl_b200.ops.fused_gemm import Peers, ag_gemm
    torch.manual_seed(1)
    M, Kc, N, R = 2048, 512, 1024, 4
    shards = [_rand(M // R, Kc) for _ in range(R)]
    w = _rand(Kc, N)                        # [contraction, N]
    full = torch.empty(M, Kc, device="cuda", dtype=torch.bfloat16)
    out = ag_gemm(full, [s.data_ptr() for s in shards], M // R, w, Peers(0, R), gathered="a", b_mn=True)
    torch.cuda.synchronize()
    _lib.raise_on_status()
    ref = torch.cat(shards, 0).float() @ w.float()
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,K,R", [(2048, 1024, 256, 4), (1024, 768, 512, 2), (4096, 4096, 512, 8),
                                     (1920, 512, 256, 2)])      # 960 rows per rank: blocks straddle tiles
def test_gemm_rs_one_device(M, N, K, R):
    """Partial results with the rotated block order and the per-owner completion counters (which
    must be back at zero after every launch), then the reduction over the ranks' blocks."""
    from xorl_b200.ops import _lib
    from xorl_b200.ops.fused_gemm import Peers, _shape_state, gemm_rs, rs_reduce
    torch.manual_seed(2)
    per = M // R
    As = [_rand(M, K) for _ in range(R)]
    Bs = [_rand(N, K) for _ in range(R)]
    parts = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(R)]
    ptrs = [s.data_ptr() for s in parts]
    for _ in range(2):
        for r in range(R):
            gemm_rs(As[r], Bs[r], parts[r], ptrs, per, Peers(r, R))
    resid = _rand(per, N)
    outs = [rs_reduce([parts[r][o * per:(o + 1) * per] for r in range(R)],
                      torch.empty(per, N, device="cuda", dtype=torch.bfloat16),
                      residual=resid if o == 0 else None) for o in range(R)]
    torch.cuda.synchronize()
    _lib.raise_on_status()
    counters = _shape_state(torch.device("cuda", torch.cuda.current_device()), ("rs", M, N, K), 1)["counters"]
    assert int(counters.abs().sum()) == 0
    partial = [a.float() @ b.float().t() for a, b in zip(As, Bs)]
    for r in range(R):
        assert (parts[r].float() - partial[r]).abs().max().item() <= 2e-2 * partial[r].abs().max().item() + 1e-2
    for o in range(R):
        ref = sum(p[o * per:(o + 1) * per].to(torch.bfloat16).float() for p in partial)
        if o == 0:
            ref = ref + resid.float()
        assert (outs[o].float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
