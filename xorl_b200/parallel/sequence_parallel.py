"""Context parallelism: Ulysses (head-scatter all-to-all), zigzag ring attention, and the hybrid.

Token layout (see ``data.collators.SequenceShardCollator``): every document is padded to a multiple
of ``2 * ring * ulysses``; ring rank ``r`` owns chunks ``r`` and ``2R-1-r`` of every document
(zigzag, balanced causal work) and inside a ring rank the Ulysses ranks own contiguous slices.

* Ulysses: q/k/v ``[T_loc, H, D] -> [T_ring, H/U, D]`` in one exchange before attention and back
  after (src/xorl/distributed/sequence_parallel/ulysses.py:49-152, strategy.py:164-247).  On GPUs the
  exchange is ``_PeerExchange``: strided copy-engine writes into the peers' symmetric receive slots;
  elsewhere all_to_all_single.
* Ring: every rank attends its queries to the K/V of every ring rank.  For source rank ``j`` the
  zigzag layout reduces the causal structure to whole-block pairs of equal length — (q_a,k_a) and
  (q_b,k_b) causal plus (q_b,k_a) full when ``j == r``; (q_a,k_a),(q_b,k_a) full when ``j < r``;
  (q_b,k_a),(q_b,k_b) full when ``j > r`` — each one call of the block-pair attention kernel, merged
  by log-sum-exp (src/xorl/distributed/sequence_parallel/ring_attention.py:28-77,202-253,331-843).
  On GPUs every rank publishes its K/V in a symmetric slot and the attention kernels load the peers'
  tiles in place (``_RingPeerKV``); elsewhere K/V blocks rotate peer to peer with the next hop in flight
  under the current block's kernels.  Backward reads K/V the same way; the dK/dV accumulator of each
  block travels rank to rank; dQ accumulates locally.
* Hybrid: Ulysses inside each ring rank group, ring across groups (strategy.py:428-477).
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import attention as attn_ops


# --------------------------------------------------------------------------------------------
# block-pair attention primitive
# --------------------------------------------------------------------------------------------
def _block_ref(q, k, v, cu, k_starts, causal, scale):
    T, Hq, D = q.shape
    g = Hq // k.shape[1]
    out = torch.zeros_like(q, dtype=torch.float32)
    lse = torch.full((Hq, T), float("-inf"), device=q.device, dtype=torch.float32)
    cu_l, ks = cu.tolist(), k_starts.tolist()
    for b in range(len(ks)):
        if ks[b] < 0:
            continue
        s, e = cu_l[b], cu_l[b + 1]
        L = e - s
        qb = q[s:e].float().transpose(0, 1)
        kb = k[ks[b]:ks[b] + L].float().transpose(0, 1).repeat_interleave(g, 0)
        vb = v[ks[b]:ks[b] + L].float().transpose(0, 1).repeat_interleave(g, 0)
        sc = torch.matmul(qb, kb.transpose(1, 2)) * scale
        if causal:
            sc = sc.masked_fill(~torch.ones(L, L, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        l = torch.logsumexp(sc, dim=-1)
        out[s:e] = torch.matmul(torch.softmax(sc, -1), vb).transpose(0, 1)
        lse[:, s:e] = l
    return out, lse


def block_attention(q, k, v, cu, k_starts, causal: bool, scale: float):
    """Attention of query blocks (tiling given by ``cu``) against key blocks starting at
    ``k_starts`` (-1 = skip).  Returns (out fp32 [T,Hq,D] zero where skipped, lse [Hq,T] -inf there)."""
    T, Hq, D = q.shape
    if q.is_cuda and q.dtype == torch.bfloat16 and D == 128:
        out = torch.zeros((T, Hq, D), device=q.device, dtype=q.dtype)
        lse = torch.full((Hq, T), float("-inf"), device=q.device, dtype=torch.float32)
        k, v = k.contiguous(), v.contiguous()
        rc = _lib.cuda_lib().xb_attn_fwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            lse.data_ptr(), cu.data_ptr(), k_starts.data_ptr(),
                                            q.stride(0), k.stride(0), v.stride(0), out.stride(0),
                                            k_starts.numel(), T, k.shape[0], Hq, k.shape[1], D,
                                            int(causal), float(scale), 0, _lib.stream_ptr())
        _lib.check(rc, "xb_attn_fwd_ex")
        return out.float(), lse
    return _block_ref(q, k, v, cu, k_starts, causal, scale)


def block_attention_bwd(q, k, v, out, dout, lse, delta, dq_acc, cu, k_starts, causal, scale,
                        first: bool):
    """Gradients of one block-pair call given the *final* (merged) out / lse.  dq is accumulated
    into ``dq_acc`` (fp32); returns (dk fp32, dv fp32) for the K/V tensor (zeros where untouched)."""
    T, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    if q.is_cuda and q.dtype == torch.bfloat16 and D == 128:
        dk = torch.zeros((Tk, Hkv, D), device=q.device, dtype=torch.float32)
        dv = torch.zeros((Tk, Hkv, D), device=q.device, dtype=torch.bfloat16)
        flags = (0 if first else 1) | (0 if first else 2)
        rc = _lib.cuda_lib().xb_attn_bwd_ex(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            delta.data_ptr(), dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr(),
            k_starts.data_ptr(), q.stride(0), k.stride(0), v.stride(0), out.stride(0), dout.stride(0),
            dv.stride(0), k_starts.numel(), T, Tk, Hq, Hkv, D, int(causal), float(scale), flags, 0,
            _lib.stream_ptr())
        _lib.check(rc, "xb_attn_bwd_ex")
        return dk, dv.float()
    # reference math
    g = Hq // Hkv
    dk = torch.zeros((Tk, Hkv, D), device=q.device, dtype=torch.float32)
    dv = torch.zeros_like(dk)
    cu_l, ks = cu.tolist(), k_starts.tolist()
    if first:
        dq_acc.zero_()
        delta.copy_((out.float() * dout.float()).sum(-1).transpose(0, 1))
    for b in range(len(ks)):
        if ks[b] < 0:
            continue
        s, e = cu_l[b], cu_l[b + 1]
        L = e - s
        qb = q[s:e].float().transpose(0, 1)
        kb = k[ks[b]:ks[b] + L].float().transpose(0, 1).repeat_interleave(g, 0)
        vb = v[ks[b]:ks[b] + L].float().transpose(0, 1).repeat_interleave(g, 0)
        do = dout[s:e].float().transpose(0, 1)
        sc = torch.matmul(qb, kb.transpose(1, 2)) * scale
        if causal:
            sc = sc.masked_fill(~torch.ones(L, L, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        p = torch.exp(sc - lse[:, s:e].unsqueeze(-1))
        dp = torch.matmul(do, vb.transpose(1, 2))
        ds = p * (dp - delta[:, s:e].unsqueeze(-1)) * scale
        dq_acc[s:e] += torch.matmul(ds, kb).transpose(0, 1)
        dkb = torch.matmul(ds.transpose(1, 2), qb)          # [Hq, L, D]
        dvb = torch.matmul(p.transpose(1, 2), do)
        dk[ks[b]:ks[b] + L] += dkb.reshape(Hkv, g, L, D).sum(1).transpose(0, 1)
        dv[ks[b]:ks[b] + L] += dvb.reshape(Hkv, g, L, D).sum(1).transpose(0, 1)
    return dk, dv


def _merge(out_acc, lse_acc, out_p, lse_p):
    """Log-sum-exp merge of partial attention results; tensors are [T,Hq,D] fp32 and [Hq,T]."""
    new = torch.logaddexp(lse_acc, lse_p)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    wa = torch.exp(lse_acc - safe).transpose(0, 1).unsqueeze(-1)
    wp = torch.exp(lse_p - safe).transpose(0, 1).unsqueeze(-1)
    return out_acc * wa + out_p * wp, new


# --------------------------------------------------------------------------------------------
# ring attention
# --------------------------------------------------------------------------------------------
def _ring_calls(cu_blocks: torch.Tensor, r: int, j: int) -> List[Tuple[torch.Tensor, bool]]:
    """k_starts (per query block) and causal flag of every kernel call for source rank j.
    ``cu_blocks`` tiles the local tokens into blocks a0,b0,a1,b1,... (two per document)."""
    starts = cu_blocks[:-1].clone()
    nb = starts.numel()
    is_a = torch.arange(nb, device=starts.device) % 2 == 0
    a_start = starts.clone()
    a_start[~is_a] = starts[is_a]                 # start of the document's a-block
    b_start = starts.clone()
    b_start[is_a] = starts[~is_a]
    neg = torch.full_like(starts, -1)
    i32 = lambda t: t.to(torch.int32)
    if j == r:
        return [(i32(starts), True),                               # (q_a,k_a), (q_b,k_b) causal
                (i32(torch.where(is_a, neg, a_start)), False)]    # (q_b,k_a) full
    if j < r:
        # two calls: the backward kernel writes dK/dV per key block, so a key block may appear
        # only once per call
        return [(i32(torch.where(is_a, a_start, neg)), False),    # (q_a,k_a) full
                (i32(torch.where(is_a, neg, a_start)), False)]    # (q_b,k_a) full
    return [(i32(torch.where(is_a, neg, a_start)), False),        # (q_b,k_a)
            (i32(torch.where(is_a, neg, b_start)), False)]        # (q_b,k_b)


def _ring_exchange(send: torch.Tensor, recv: torch.Tensor, group, rank: int, world: int):
    """Posts ``send`` to the next ring rank and ``recv`` from the previous one; returns the requests.
    Nothing waits here: the caller computes on the block it already holds and waits afterwards."""
    nxt = dist.get_global_rank(group, (rank + 1) % world)
    prv = dist.get_global_rank(group, (rank - 1) % world)
    return dist.batch_isend_irecv([dist.P2POp(dist.isend, send, nxt, group),
                                   dist.P2POp(dist.irecv, recv, prv, group)])


def _wait_all(reqs) -> None:
    for r in reqs:
        r.wait()


# how often the peer-memory forms ran in this process (the trainer writes them to training_metrics.json)
PEER_PATH_CALLS = {"ring_kv_published": 0, "ulysses_exchanges": 0}


class _RingPeerKV:
    """K/V of every ring rank published in symmetric memory and pulled by the copy engines.

    One symmetric heap per (ring group, size): a flag area for the bounded barrier of ``csrc/comm.cu`` and
    two K/V slots.  A call writes this rank's K/V into slot ``n % 2`` and runs the barrier (all ranks have
    written; since a rank reaches the barrier of call ``n`` only after its work of call ``n - 1`` is queued
    on the same stream, passing the barrier of call ``n - 1`` also means that nobody still reads the slot of
    call ``n - 2``: two slots and one barrier per call are enough).  The block of the rank whose turn comes
    next is then copied from its owner's slot into one of two local buffers by a copy engine on a side
    stream, under the attention kernels of the current block, and the kernels read local memory: every
    remote block crosses NVLink exactly once, straight from its owner (no hop-by-hop rotation), without a
    collective library and without an SM.  (Letting the attention kernels load the peers' tiles in place
    was measured first: every query tile re-reads the remote K/V over NVLink, which does not pass through
    the local L2, and a 65 536-token step took twice as long.)
    (src/xorl/distributed/sequence_parallel/ring_attention.py:168-191 does the hop with batched isend / irecv.)"""
    FLAG_BYTES = 16 * 1024
    WAIT_MS = 2000
    _cache: dict = {}

    @classmethod
    def get(cls, group, world: int, rank: int, numel: int, dtype, device) -> "Optional[_RingPeerKV]":
        if os.environ.get("XORL_B200_RING_PEER_KV", "1") == "0" or device.type != "cuda" or dtype != torch.bfloat16:
            return None
        key = (id(group), device.index)
        ws = cls._cache.get(key)
        if ws is None or ws.capacity < numel:
            try:
                ws = cls(group, world, rank, numel, dtype, device)
            except Exception as e:  # noqa: BLE001  (no symmetric memory on this system: rotate through NCCL)
                from ..utils.logging import info_rank0
                info_rank0(f"ring attention: peer-memory K/V unavailable ({type(e).__name__}: {e}); using send/recv")
                os.environ["XORL_B200_RING_PEER_KV"] = "0"
                return None
            cls._cache[key] = ws
        return ws

    def __init__(self, group, world, rank, numel, dtype, device):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank, self.dtype = world, rank, dtype
        self.capacity = numel
        es = torch.empty(0, dtype=dtype).element_size()
        self.slot_bytes = (numel * es + 255) // 256 * 256
        self.heap = symm_mem.empty(self.FLAG_BYTES + 2 * self.slot_bytes, dtype=torch.uint8, device=device)
        self.heap[:self.FLAG_BYTES].zero_()
        self.hdl = symm_mem.rendezvous(self.heap, group)
        self.base = [int(p) for p in self.hdl.buffer_ptrs]
        self.flag_ptrs = (ctypes.c_ulonglong * world)(*self.base)
        self.epoch = 0
        self.calls = 0
        self._bufs = None
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def publish(self, kv: torch.Tensor) -> "_RingFetch":
        """Writes ``kv`` into the next slot, runs the barrier, returns the fetcher of the peers' blocks."""
        es = kv.element_size()
        slot = self.calls % 2
        self.calls += 1
        PEER_PATH_CALLS["ring_kv_published"] += 1
        off = self.FLAG_BYTES + slot * self.slot_bytes
        self.heap[off:off + kv.numel() * es].view(kv.dtype).view(kv.shape).copy_(kv)
        self.epoch += 1
        _lib.check(_lib.cuda_lib().xb_symm_barrier(self.flag_ptrs, 0, self.rank, self.world, self.epoch, self.WAIT_MS,
                                                   _lib.stream_ptr()), "xb_symm_barrier")
        return _RingFetch(self, kv, off)


class _RingFetch:
    """Double-buffered copy-engine pulls of the peers' K/V blocks for one ring pass.  ``prefetch(j)`` starts
    the copy of rank ``j``'s block on the side stream (after the compute stream has released the buffer it
    lands in); ``take(j)`` makes the compute stream wait for it and returns the local tensor."""

    def __init__(self, ws: _RingPeerKV, kv: torch.Tensor, off: int):
        self.ws, self.kv, self.off = ws, kv, off
        self.nbytes = kv.numel() * kv.element_size()
        if getattr(ws, "_bufs", None) is None or ws._bufs[0].numel() < kv.numel() or ws._bufs[0].dtype != kv.dtype:
            ws._bufs = [torch.empty(kv.numel(), dtype=kv.dtype, device=kv.device) for _ in range(2)]
            ws._copy_stream = torch.cuda.Stream(device=kv.device)
            ws._free = [None, None]                 # event: the compute stream is done with the buffer
        self.n = 0
        self.pending = {}

    def prefetch(self, j: int) -> None:
        ws = self.ws
        b = self.n % 2
        self.n += 1
        cs = ws._copy_stream
        cs.wait_stream(torch.cuda.current_stream())          # the barrier (peers have written) precedes the copy
        if ws._free[b] is not None:
            cs.wait_event(ws._free[b])
        _lib.check(_lib.cuda_lib().xb_peer_copy_2d(ws._bufs[b].data_ptr(), self.nbytes, ws.base[j] + self.off,
                                                   self.nbytes, self.nbytes, 1, cs.cuda_stream), "xb_peer_copy_2d")
        ev = torch.cuda.Event()
        ev.record(cs)
        self.pending[j] = (b, ev)

    def take(self, j: int) -> torch.Tensor:
        b, ev = self.pending.pop(j)
        torch.cuda.current_stream().wait_event(ev)
        self._held = b
        return self.ws._bufs[b][:self.kv.numel()].view(self.kv.shape)

    def release(self) -> None:
        """The kernels that read the buffer returned by the last ``take`` have been queued."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.ws._free[self._held] = ev


def _ring_blocks(fetch: Optional["_RingFetch"], kv: torch.Tensor, rank: int, world: int):
    """Yields (source rank, its K/V) in ring order with the next block's copy in flight."""
    order = [(rank - s) % world for s in range(world)]
    if world > 1:
        fetch.prefetch(order[1])
    for s, j in enumerate(order):
        if j == rank:
            yield j, kv
            continue
        cur = fetch.take(j)
        if s + 1 < world:
            fetch.prefetch(order[s + 1])
        yield j, cur
        fetch.release()


class _RingAttention(torch.autograd.Function):
    """K/V blocks travel round the ring one hop per step (two receive buffers: the hop for step
    ``s+1`` is in flight while step ``s`` computes), so a rank never holds more than its own block
    plus two in transit, and only its own block is kept for backward
    (src/xorl/distributed/sequence_parallel/ring_attention.py:168-191).  In backward the blocks make
    the same trip again and the fp32 dK/dV accumulator of a block travels with it, picking up one
    contribution per rank; one last hop brings it home (ring_attention.py:612-843)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_blocks, group, rank, world, scale):
        T, Hq, D = q.shape
        kv = torch.stack([k.contiguous(), v.contiguous()])            # [2, T, Hkv, D]
        out = torch.zeros((T, Hq, D), device=q.device, dtype=torch.float32)
        lse = torch.full((Hq, T), float("-inf"), device=q.device, dtype=torch.float32)
        qc = q.contiguous()
        peers = _RingPeerKV.get(group, world, rank, kv.numel(), kv.dtype, kv.device)
        if peers is not None:
            # every peer's block is pulled from its owner's slot by a copy engine, one block ahead
            for j, cur in _ring_blocks(peers.publish(kv), kv, rank, world):
                for k_starts, causal in _ring_calls(cu_blocks, rank, j):
                    o_p, l_p = block_attention(qc, cur[0], cur[1], cu_blocks, k_starts, causal, scale)
                    out, lse = _merge(out, lse, o_p, l_p)
            out_lp = out.to(q.dtype)
            ctx.save_for_backward(qc, kv, out_lp, lse, cu_blocks)
            ctx.cfg = (group, rank, world, scale)
            return out_lp
        bufs = [torch.empty_like(kv), torch.empty_like(kv)]
        cur = kv
        for s in range(world):
            j = (rank - s) % world
            reqs = _ring_exchange(cur, bufs[s % 2], group, rank, world) if s < world - 1 else ()
            for k_starts, causal in _ring_calls(cu_blocks, rank, j):
                o_p, l_p = block_attention(qc, cur[0], cur[1], cu_blocks, k_starts, causal, scale)
                out, lse = _merge(out, lse, o_p, l_p)
            if s < world - 1:
                _wait_all(reqs)
                cur = bufs[s % 2]
        out_lp = out.to(q.dtype)
        ctx.save_for_backward(qc, kv, out_lp, lse, cu_blocks)
        ctx.cfg = (group, rank, world, scale)
        return out_lp

    @staticmethod
    def backward(ctx, dout):
        qc, kv, out, lse, cu_blocks = ctx.saved_tensors
        group, rank, world, scale = ctx.cfg
        T, Hq, D = qc.shape
        dout = dout.contiguous()
        dq = torch.zeros((T, Hq, D), device=qc.device, dtype=torch.float32)
        delta = torch.empty((Hq, T), device=qc.device, dtype=torch.float32)
        peers = _RingPeerKV.get(group, world, rank, kv.numel(), kv.dtype, kv.device)
        fetch = peers.publish(kv) if peers is not None else None      # the peers' blocks are pulled again, one ahead
        order = [(rank - s) % world for s in range(world)]
        if fetch is not None and world > 1:
            fetch.prefetch(order[1])
        bufs = [torch.empty_like(kv), torch.empty_like(kv)] if peers is None else None
        acc_bufs = [torch.empty(kv.shape, device=kv.device, dtype=torch.float32) for _ in range(2)]
        cur, acc, acc_reqs = kv, None, ()
        first = True
        for s in range(world):
            j = order[s]
            if fetch is not None:
                if j == rank:
                    cur = kv
                else:
                    cur = fetch.take(j)
                    if s + 1 < world:
                        fetch.prefetch(order[s + 1])
            reqs = _ring_exchange(cur, bufs[s % 2], group, rank, world) if (peers is None and s < world - 1) else ()
            part = None
            for k_starts, causal in _ring_calls(cu_blocks, rank, j):
                dk, dv = block_attention_bwd(qc, cur[0], cur[1], out, dout, lse, delta, dq, cu_blocks,
                                             k_starts, causal, scale, first)
                first = False
                both = torch.stack([dk, dv])
                part = both if part is None else part + both
            if fetch is not None and j != rank:
                fetch.release()
            if s > 0:
                _wait_all(acc_reqs)                                  # block j's accumulator so far
                part = part + acc_bufs[(s - 1) % 2]
            acc = part
            acc_reqs = _ring_exchange(acc, acc_bufs[s % 2], group, rank, world)
            if peers is None and s < world - 1:
                _wait_all(reqs)
                cur = bufs[s % 2]
        _wait_all(acc_reqs)                                          # the hop home: this rank's own block
        mine = acc_bufs[(world - 1) % 2]
        return dq.to(qc.dtype), mine[0].to(qc.dtype), mine[1].to(qc.dtype), None, None, None, None, None


# --------------------------------------------------------------------------------------------
# Ulysses all-to-all
# --------------------------------------------------------------------------------------------
class _SeqToHead(torch.autograd.Function):
    """[T_loc, H, D] (all heads, local tokens) -> [U*T_loc, H/U, D] (local heads, group tokens)."""

    @staticmethod
    def forward(ctx, x, group, world):
        ctx.group, ctx.world = group, world
        T, H, D = x.shape
        send = x.reshape(T, world, H // world, D).permute(1, 0, 2, 3).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.reshape(world * T, H // world, D)

    @staticmethod
    def backward(ctx, g):
        world = ctx.world
        TT, Hl, D = g.shape
        T = TT // world
        send = g.reshape(world, T, Hl, D).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=ctx.group)
        return recv.permute(1, 0, 2, 3).reshape(T, world * Hl, D), None, None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world):
        ctx.group, ctx.world = group, world
        TT, Hl, D = x.shape
        T = TT // world
        send = x.reshape(world, T, Hl, D).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 0, 2, 3).reshape(T, world * Hl, D)

    @staticmethod
    def backward(ctx, g):
        world = ctx.world
        T, H, D = g.shape
        send = g.reshape(T, world, H // world, D).permute(1, 0, 2, 3).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=ctx.group)
        return recv.reshape(world * T, H // world, D), None, None


class _PeerExchange:
    """Head / sequence exchange of Ulysses without a collective library: every rank writes its slice for
    rank ``u`` straight into ``u``'s receive slot (symmetric memory, one strided copy-engine transfer per
    destination, no SM and no pack / unpack pass), then the bounded barrier of ``csrc/comm.cu`` tells
    everybody that its slot is complete.  Two slots alternate, for the reason given in ``_RingPeerKV``
    (src/xorl/distributed/sequence_parallel/ulysses.py:49-152 does this with all_to_all_single on packed
    copies)."""
    FLAG_BYTES = 16 * 1024
    WAIT_MS = 2000
    _cache: dict = {}

    @classmethod
    def get(cls, group, world, rank, nbytes, device) -> "Optional[_PeerExchange]":
        if os.environ.get("XORL_B200_ULYSSES_PEER", "1") == "0" or device.type != "cuda":
            return None
        key = (id(group), device.index)
        ws = cls._cache.get(key)
        if ws is None or ws.slot_bytes < nbytes:
            try:
                ws = cls(group, world, rank, nbytes, device)
            except Exception as e:  # noqa: BLE001
                from ..utils.logging import info_rank0
                info_rank0(f"ulysses: peer-memory exchange unavailable ({type(e).__name__}: {e}); using all_to_all")
                os.environ["XORL_B200_ULYSSES_PEER"] = "0"
                return None
            cls._cache[key] = ws
        return ws

    def __init__(self, group, world, rank, nbytes, device):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = world, rank
        self.slot_bytes = (nbytes + 255) // 256 * 256
        self.heap = symm_mem.empty(self.FLAG_BYTES + 2 * self.slot_bytes, dtype=torch.uint8, device=device)
        self.heap[:self.FLAG_BYTES].zero_()
        self.hdl = symm_mem.rendezvous(self.heap, group)
        self.base = [int(p) for p in self.hdl.buffer_ptrs]
        self.flag_ptrs = (ctypes.c_ulonglong * world)(*self.base)
        self.epoch = 0
        self.calls = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _exchange(self, pieces, out_shape, dtype) -> torch.Tensor:
        """``pieces``: per destination rank (dst byte offset inside the slot, dst pitch, src pointer, src pitch,
        width, height).  Returns this rank's slot viewed as ``out_shape`` (valid until two calls later)."""
        lib = _lib.cuda_lib()
        slot = self.calls % 2
        self.calls += 1
        PEER_PATH_CALLS["ulysses_exchanges"] += 1
        off = self.FLAG_BYTES + slot * self.slot_bytes
        st = _lib.stream_ptr()
        for u, (doff, dpitch, sptr, spitch, width, height) in enumerate(pieces):
            _lib.check(lib.xb_peer_copy_2d(self.base[u] + off + doff, dpitch, sptr, spitch, width, height, st),
                       "xb_peer_copy_2d")
        self.epoch += 1
        _lib.check(lib.xb_symm_barrier(self.flag_ptrs, 0, self.rank, self.world, self.epoch, self.WAIT_MS, st),
                   "xb_symm_barrier")
        n = 1
        for d in out_shape:
            n *= d
        es = torch.empty(0, dtype=dtype).element_size()
        return self.heap[off:off + n * es].view(dtype).view(out_shape)

    @staticmethod
    def seq_to_head_pieces(rank: int, T: int, H: int, D: int, U: int, es: int):
        """Per destination rank: (dst byte offset in its slot, dst pitch, src byte offset, src pitch, width, rows)."""
        row = (H // U) * D * es
        return [(rank * T * row, row, u * row, H * D * es, row, T) for u in range(U)]

    @staticmethod
    def head_to_seq_pieces(rank: int, T: int, h: int, D: int, U: int, es: int):
        row = h * D * es
        return [(rank * row, U * row, u * T * row, row, row, T) for u in range(U)]

    def _with_base(self, pieces, base_ptr: int):
        return [(doff, dp, base_ptr + soff, sp, w, n) for doff, dp, soff, sp, w, n in pieces]

    def seq_to_head(self, x: torch.Tensor) -> torch.Tensor:
        """[T, U*h, D] (all heads, local tokens) -> [U*T, h, D] (local heads, the group's tokens)."""
        T, H, D = x.shape
        pieces = self.seq_to_head_pieces(self.rank, T, H, D, self.world, x.element_size())
        return self._exchange(self._with_base(pieces, x.data_ptr()), (self.world * T, H // self.world, D), x.dtype)

    def head_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        """[U*T, h, D] -> [T, U*h, D]."""
        TT, h, D = x.shape
        T = TT // self.world
        pieces = self.head_to_seq_pieces(self.rank, T, h, D, self.world, x.element_size())
        return self._exchange(self._with_base(pieces, x.data_ptr()), (T, self.world * h, D), x.dtype)


def _peer_exchange_for(x: torch.Tensor, group, world):
    if not x.is_cuda:
        return None
    return _PeerExchange.get(group, world, dist.get_rank(group), x.numel() * x.element_size(), x.device)


class _SeqToHeadPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world, ex):
        ctx.group, ctx.world, ctx.ex = group, world, ex
        return ex.seq_to_head(x.contiguous())          # a view of the receive slot: consume before two more exchanges

    @staticmethod
    def backward(ctx, g):
        return ctx.ex.head_to_seq(g.contiguous()).clone(), None, None, None


class _HeadToSeqPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world, ex):
        ctx.group, ctx.world, ctx.ex = group, world, ex
        return ex.head_to_seq(x.contiguous()).clone()

    @staticmethod
    def backward(ctx, g):
        return ctx.ex.seq_to_head(g.contiguous()).clone(), None, None, None


# --------------------------------------------------------------------------------------------
# strategy object used by the attention layers
# --------------------------------------------------------------------------------------------
class ContextParallelStrategy:
    def __init__(self, ps):
        self.ps = ps
        self.U, self.R = ps.ulysses_size, ps.ringattn_size
        self.u_group, self.r_group = ps.group("ulysses"), ps.group("ringattn")
        self.u_rank, self.r_rank = ps.ulysses_rank, ps.ringattn_rank

    def prepare(self, model, ctx) -> None:
        """cos/sin for the local tokens' global positions; block tilings for the attention calls."""
        ctx.cos, ctx.sin = model.rotary(ctx.position_ids)
        local_cu = ctx.aux.get("local_cu_seqlens")
        if local_cu is None:
            raise ValueError("context parallelism needs batches from SequenceShardCollator "
                             "(local_cu_seqlens missing)")
        local_cu = local_cu.cpu()
        lens = (local_cu[1:] - local_cu[:-1]).to(torch.int64)      # this rank's tokens per document
        dev = ctx.position_ids.device
        U = self.U
        ring_lens = lens * U                                       # tokens per document per ring rank
        if self.R > 1:
            half = ring_lens // 2
            blocks = torch.stack([half, half], 1).reshape(-1)      # a, b per document
            ctx.aux["cp_blocks"] = torch.cat([blocks.new_zeros(1), blocks.cumsum(0)]).to(torch.int32).to(dev)
        ctx.aux["cp_ring_cu"] = torch.cat([ring_lens.new_zeros(1), ring_lens.cumsum(0)]).to(torch.int32).to(dev)
        if U > 1:
            # after the all-to-all tokens are ordered (ulysses rank, document, offset); attention wants
            # (document, ulysses rank, offset)
            T_loc = int(lens.sum())
            doc_of = torch.repeat_interleave(torch.arange(lens.numel()), lens)
            off = torch.arange(T_loc) - torch.repeat_interleave(local_cu[:-1].to(torch.int64), lens)
            ring_start = ctx.aux["cp_ring_cu"][:-1].to("cpu", torch.int64)
            idx = torch.empty(U * T_loc, dtype=torch.int64)
            for u in range(U):
                dst = ring_start[doc_of] + u * lens[doc_of] + off
                idx[dst] = u * T_loc + torch.arange(T_loc)
            ctx.aux["cp_gather_idx"] = idx.to(dev)
            inv = torch.empty_like(idx)
            inv[idx] = torch.arange(idx.numel())
            ctx.aux["cp_scatter_idx"] = inv.to(dev)

    def attention(self, attn, qkv, ctx) -> torch.Tensor:
        """qkv: local tokens, all (tensor-parallel-local) heads.  Returns [T_loc, Hq*D]."""
        Hq, Hkv, D = attn.Hq, attn.Hkv, attn.D
        T = qkv.shape[0]
        if hasattr(attn, "_qkv_heads"):
            # the layer's own norm / rotary variants (whole-projection or per-head norms, partial
            # rotary, no positional embedding) on this rank's tokens at their global positions
            q, k, v = attn._qkv_heads(qkv, ctx)
        else:
            wq = attn.q_norm.weight if attn.use_qk_norm else None
            wk = attn.k_norm.weight if attn.use_qk_norm else None
            # per-head RMSNorm + rotary at the tokens' global positions: the fused kernel on a GPU
            q, k, v = attn_ops.qk_norm_rope(qkv, wq, wk, ctx.cos, ctx.sin, Hq, Hkv, D, attn.cfg.rms_norm_eps)
        U = self.U
        if U > 1:
            if Hkv % U:
                rep = U // math.gcd(Hkv, U)
                k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
            # one all-to-all for q, k and v: heads are laid out (ulysses rank, [q | k | v] heads of that rank)
            hq, hk = Hq // U, k.shape[1] // U
            packed = torch.cat([q.reshape(T, U, hq, D), k.reshape(T, U, hk, D), v.reshape(T, U, hk, D)], 2)
            packed = packed.reshape(T, U * (hq + 2 * hk), D)
            ex = _peer_exchange_for(packed, self.u_group, U)
            if ex is not None:
                # the receive slot is read once, by the gather that puts tokens into document order
                packed = _SeqToHeadPeer.apply(packed, self.u_group, U, ex)
            else:
                packed = _SeqToHead.apply(packed, self.u_group, U)
            packed = packed.index_select(0, ctx.aux["cp_gather_idx"])
            q, k, v = packed.split([hq, hk, hk], dim=1)
        if self.R > 1:
            out = _RingAttention.apply(q, k, v, ctx.aux["cp_blocks"], self.r_group, self.r_rank,
                                       self.R, attn.scale)
        else:
            out = attn_ops.flash_attn_varlen(q, k, v, ctx.aux["cp_ring_cu"], ctx.causal, attn.scale)
        if U > 1:
            out = out.index_select(0, ctx.aux["cp_scatter_idx"])
            ex = _peer_exchange_for(out, self.u_group, U)
            out = _HeadToSeqPeer.apply(out, self.u_group, U, ex) if ex is not None \
                else _HeadToSeq.apply(out, self.u_group, U)
        return out.reshape(T, Hq * D)


def build_cp_strategy(model, ps) -> ContextParallelStrategy:
    return ContextParallelStrategy(ps)
