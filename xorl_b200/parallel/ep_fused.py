"""Fused expert-parallel dispatch / combine over peer memory (``csrc/ep.cu``).

Per MoE layer: exchange per-expert counts through peer stores -> every rank derives, on the
device, the exact row of each of its token slots in the owners' segment-aligned receive buffers
-> push rows straight into the owners' buffers -> grouped expert MLP on the receive buffer ->
push expert outputs straight back into the sources' slot buffers -> weighted sum over the k
experts of a token.  No NCCL call and no host synchronisation on the path; every wait on a peer
is bounded.  Backward runs the same two pushes in the opposite roles on a second set of buffers.

The receive buffer holds ``XORL_B200_EP_CAPACITY`` (default 2.0) times the balanced load; a
routing so skewed that a rank would receive more rows than that is reported through the status
words (rows beyond the capacity are dropped, never written out of bounds).  Workspace tensors
are reused by every layer, which is safe because layers are recomputed right before their
backward; without recomputation the all-to-all path is used instead.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe as moe_ops
from .state import get_parallel_state

FLAG_BYTES = 4096
S_COUNTS, S_DISP, S_RET, S_BDISP, S_BRET = 0, 16, 32, 48, 64
C_DISP, C_RET, C_BDISP, C_BRET = 96, 97, 98, 99
WAIT_MS = 2000
_WS: Dict = {}
_SRC_ROW: Dict = {}


def fused_ep_available() -> bool:
    ps = get_parallel_state()
    return ps.ep_size > 1 and torch.cuda.is_available() and ps.group("ep") is not None \
        and os.environ.get("XORL_B200_EP_FUSED", "1") == "1"


class _Workspace:
    def __init__(self, H: int, slots: int, num_experts: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        ps = get_parallel_state()
        self.N, self.rank = ps.ep_size, ps.ep_rank
        self.El = num_experts // self.N
        self.E, self.H, self.slots = num_experts, H, slots
        factor = float(os.environ.get("XORL_B200_EP_CAPACITY", "2.0"))
        self.cap = moe_ops.buffer_rows(int(min(self.N, factor) * slots), self.El)
        a = lambda x: (x + 255) // 256 * 256
        off = FLAG_BYTES
        self.o_table = off; off = a(off + self.N * self.E * 4)
        self.o = {}
        for name, rows, width in (("recv_f", self.cap, H * 2), ("meta_f", self.cap, 4),
                                  ("ret_f", slots, H * 2), ("recv_b", self.cap, H * 2),
                                  ("meta_b", self.cap, 4), ("ret_b", slots, H * 2)):
            self.o[name] = off
            off = a(off + rows * width)
        self.heap = symm_mem.empty(off, dtype=torch.uint8, device=device)
        self.heap.zero_()
        self.hdl = symm_mem.rendezvous(self.heap, ps.group("ep"))
        self.base = [int(p) for p in self.hdl.buffer_ptrs]
        self.epoch = {k: 0 for k in ("counts", "disp", "ret", "bdisp", "bret")}
        self.lib = _lib.cuda_lib()
        self._ptr_cache: Dict[int, object] = {}
        torch.cuda.synchronize()
        dist.barrier(group=ps.group("ep"))

    def ptrs(self, off: int):
        arr = self._ptr_cache.get(off)
        if arr is None:
            arr = self._ptr_cache[off] = (ctypes.c_ulonglong * self.N)(*[b + off for b in self.base])
        return arr

    def view(self, name: str, rows: int, dtype, width_elems: int):
        es = torch.empty(0, dtype=dtype).element_size()
        o = self.o[name]
        return self.heap[o:o + rows * width_elems * es].view(dtype).view(rows, width_elems) \
            if width_elems > 1 else self.heap[o:o + rows * es].view(dtype)

    def local_flags(self, slot: int) -> int:
        return self.base[self.rank] + 4 * slot

    def wait(self, slot: int, epoch: int) -> None:
        _lib.check(self.lib.xb_symm_wait(ctypes.c_void_p(self.local_flags(slot)), self.N, self.rank,
                                         epoch, WAIT_MS, _lib.stream_ptr()), "xb_symm_wait")

    def push(self, src, src_row, dest_rank, dest_row, tag, dst_name, meta_name, slot, counter, key,
             row_bytes: int = 0):
        """``row_bytes`` (default: one bf16 row of width H) is the payload of a row and the row pitch of both
        the source and the destination when given (quantised rows: e4m3 values followed by their scales)."""
        self.epoch[key] += 1
        n_items = dest_rank.numel()
        rb = row_bytes or self.H * 2
        src_ld = row_bytes or src.stride(0) * src.element_size()
        _lib.check(self.lib.xb_ep_push_rows(
            src.data_ptr(), src_ld, _lib.ptr(src_row), dest_rank.data_ptr(),
            dest_row.data_ptr(), _lib.ptr(tag), 24, n_items, rb, self.ptrs(self.o[dst_name]),
            rb, None if meta_name is None else self.ptrs(self.o[meta_name]), self.ptrs(0),
            slot, counter, self.rank, self.N, self.epoch[key], _lib.stream_ptr()), "xb_ep_push_rows")
        self.wait(slot, self.epoch[key])


def _workspace(H, slots, E, device) -> _Workspace:
    key = (H, slots, E)
    if key not in _WS:
        _WS[key] = _Workspace(H, slots, E, device)
    return _WS[key]


class _Plan:
    """Everything both directions need, computed once per layer call on the device."""
    pass


def _make_plan(ws: _Workspace, indices: torch.Tensor) -> _Plan:
    dev = indices.device
    T, k = indices.shape
    flat = indices.reshape(-1)
    counts = torch.bincount(flat, minlength=ws.E).to(torch.int32)
    ws.epoch["counts"] += 1
    _lib.check(ws.lib.xb_ep_exchange_counts(counts.data_ptr(), ws.ptrs(ws.o_table), ws.ptrs(0), S_COUNTS,
                                            ws.rank, ws.N, ws.E, ws.epoch["counts"], WAIT_MS,
                                            _lib.stream_ptr()), "xb_ep_exchange_counts")
    if os.environ.get("XORL_B200_EP_PLAN_KERNEL", "1") == "1":
        # one kernel: per-slot destination (rank, row), local segment table, overflow flag
        S = flat.numel()
        p = _Plan()
        p.T, p.k = T, k
        p.dest_rank = torch.empty(S, device=dev, dtype=torch.int32)
        p.dest_row = torch.empty(S, device=dev, dtype=torch.int32)
        p.seg = torch.empty(ws.El + 1, device=dev, dtype=torch.int32)
        p.tot = torch.empty(ws.El, device=dev, dtype=torch.int32)
        p.overflow = torch.zeros(1, device=dev, dtype=torch.int32)
        table_ptr = ws.heap.data_ptr() + ws.o_table
        _lib.check(ws.lib.xb_ep_plan(flat.contiguous().data_ptr(), S, ctypes.c_void_p(table_ptr), ws.rank, ws.N, ws.E,
                                     ws.El, ws.cap, p.dest_rank.data_ptr(), p.dest_row.data_ptr(),
                                     p.seg.data_ptr(), p.tot.data_ptr(), p.overflow.data_ptr(),
                                     _lib.stream_ptr()), "xb_ep_plan")
        key = (S, k, dev)
        if key not in _SRC_ROW:
            _SRC_ROW[key] = (torch.arange(S, device=dev) // k).to(torch.int32)
        p.src_row = _SRC_ROW[key]
        return p
    table = ws.heap[ws.o_table:ws.o_table + ws.N * ws.E * 4].view(torch.int32).view(ws.N, ws.E).long()
    tot = table.sum(0)                                              # [E] rows per expert (all sources)
    padded = (tot + moe_ops.SEG_ALIGN - 1) // moe_ops.SEG_ALIGN * moe_ops.SEG_ALIGN
    pe = padded.view(ws.N, ws.El)
    seg_start = (pe.cumsum(1) - pe).reshape(-1)                     # start row of expert e on its owner
    before_me = table[:ws.rank].sum(0) if ws.rank > 0 else torch.zeros_like(tot)
    base = seg_start + before_me
    order = torch.argsort(flat, stable=True)
    c64 = counts.long()
    starts = c64.cumsum(0) - c64
    sorted_e = flat[order]
    rank_in_e = torch.empty_like(flat)
    rank_in_e[order] = torch.arange(flat.numel(), device=dev) - starts[sorted_e]
    p = _Plan()
    p.T, p.k = T, k
    p.dest_rank = (flat // ws.El).to(torch.int32)
    p.dest_row = (base[flat] + rank_in_e).to(torch.int32)
    # rows that would fall outside the receive buffer are dropped (and reported by the kernel's
    # caller through the overflow flag below)
    over = p.dest_row >= ws.cap
    p.dest_rank = torch.where(over, torch.full_like(p.dest_rank, -1), p.dest_rank)
    p.overflow = over.any()
    p.src_row = (torch.arange(flat.numel(), device=dev) // k).to(torch.int32)
    mine = slice(ws.rank * ws.El, (ws.rank + 1) * ws.El)
    my_pad = padded[mine]
    p.seg = torch.cat([my_pad.new_zeros(1), my_pad.cumsum(0)]).clamp(max=ws.cap // 128 * 128).to(torch.int32)
    p.tot = tot[mine].to(torch.int32)
    return p


def _prepare(ws: _Workspace, plan: _Plan, recv_name: str, meta_name: str) -> None:
    x = ws.view(recv_name, ws.cap, torch.bfloat16, ws.H)
    meta = ws.view(meta_name, ws.cap, torch.int32, 1)
    _lib.check(ws.lib.xb_ep_prepare_recv(x.data_ptr(), meta.data_ptr(), plan.seg.data_ptr(),
                                         plan.tot.data_ptr(), ws.El, ws.cap, ws.H * 2,
                                         _lib.stream_ptr()), "xb_ep_prepare_recv")


def _meta_targets(meta: torch.Tensor):
    valid = meta >= 0
    rank = torch.where(valid, meta >> 24, torch.full_like(meta, -1))
    slot = torch.where(valid, meta & 0xFFFFFF, torch.zeros_like(meta))
    return rank.to(torch.int32), slot.to(torch.int32)


class _Dispatch(torch.autograd.Function):
    """token rows -> owners' receive buffers; backward: gradient rows -> source slots, summed over k."""

    @staticmethod
    def forward(ctx, x, ws: _Workspace, plan: _Plan):
        x = x.contiguous()
        _prepare(ws, plan, "recv_f", "meta_f")
        ws.push(x, plan.src_row, plan.dest_rank, plan.dest_row, None, "recv_f", "meta_f", S_DISP, C_DISP, "disp")
        ctx.ws, ctx.plan = ws, plan
        return ws.view("recv_f", ws.cap, torch.bfloat16, ws.H)

    @staticmethod
    def backward(ctx, dbuf):
        ws, plan = ctx.ws, ctx.plan
        meta = ws.view("meta_f", ws.cap, torch.int32, 1)
        r, s = _meta_targets(meta)
        ws.push(dbuf.contiguous(), None, r, s, None, "ret_b", None, S_BRET, C_BRET, "bret")
        dslots = ws.view("ret_b", plan.T * plan.k, torch.bfloat16, ws.H)
        dx = dslots.view(plan.T, plan.k, ws.H).float().sum(1).to(torch.bfloat16)
        return dx, None, None


class _Return(torch.autograd.Function):
    """expert output rows -> source slot buffers; backward: slot gradients -> owners' rows."""

    @staticmethod
    def forward(ctx, y, ws: _Workspace, plan: _Plan):
        meta = ws.view("meta_f", ws.cap, torch.int32, 1)
        r, s = _meta_targets(meta)
        ws.push(y.contiguous(), None, r, s, None, "ret_f", None, S_RET, C_RET, "ret")
        ctx.ws, ctx.plan = ws, plan
        return ws.view("ret_f", plan.T * plan.k, torch.bfloat16, ws.H)

    @staticmethod
    def backward(ctx, dslots):
        ws, plan = ctx.ws, ctx.plan
        _prepare(ws, plan, "recv_b", "meta_b")
        src_row = torch.arange(plan.T * plan.k, device=dslots.device, dtype=torch.int32)
        ws.push(dslots.contiguous(), src_row, plan.dest_rank, plan.dest_row, None, "recv_b", "meta_b",
                S_BDISP, C_BDISP, "bdisp")
        return ws.view("recv_b", ws.cap, torch.bfloat16, ws.H), None, None


class PhaseTimes:
    """Device time per phase of the fused MoE (``XORL_B200_EP_PHASE_TIMING=1``): CUDA events around the
    plan, the two pushes, the expert GEMMs and the combine, summed over calls; ``report()``
    synchronises and returns milliseconds per phase and call counts."""
    enabled = os.environ.get("XORL_B200_EP_PHASE_TIMING", "0") == "1"
    pending: list = []
    totals: Dict[str, float] = {}
    counts: Dict[str, int] = {}

    @classmethod
    def mark(cls):
        if not cls.enabled:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    @classmethod
    def add(cls, name: str, start, end=None):
        if cls.enabled and start is not None:
            cls.pending.append((name, start, end if end is not None else cls.mark()))

    @classmethod
    def report(cls) -> Dict[str, float]:
        if not cls.enabled:
            return {}
        torch.cuda.synchronize()
        for name, a, b in cls.pending:
            cls.totals[name] = cls.totals.get(name, 0.0) + a.elapsed_time(b)
            cls.counts[name] = cls.counts.get(name, 0) + 1
        cls.pending = []
        return {k: round(v, 3) for k, v in cls.totals.items()} | {f"n_{k}": c for k, c in cls.counts.items()}


class _Scratch:
    """Per-workspace local buffers of the single-function path: plan arrays, expert activations,
    return targets and (in fp8 mode) quantised operands.  Allocated once; every layer reuses them,
    which is safe because a layer's backward directly follows its (re)computed forward."""

    def __init__(self, ws: _Workspace, I2: int, act_I: int, fp8: bool):
        dev = ws.heap.device
        S, cap, H, El, E = ws.slots, ws.cap, ws.H, ws.El, ws.E
        i32 = dict(device=dev, dtype=torch.int32)
        bf = dict(device=dev, dtype=torch.bfloat16)
        self.I2, self.I = I2, act_I
        self.counts = torch.zeros(E, **i32)
        self.dest_rank = torch.empty(S, **i32)
        self.dest_row = torch.empty(S, **i32)
        self.seg = torch.zeros(El + 1, **i32)
        # seg[El] = end of the last expert segment: elementwise kernels over the worst-case sized
        # buffers stop there
        self.row_limit_ptr = self.seg.data_ptr() + 4 * El
        self.tot = torch.zeros(El, **i32)
        self.overflow = torch.zeros(1, **i32)
        self.ret_rank = torch.empty(cap, **i32)
        self.ret_slot = torch.empty(cap, **i32)
        from ..utils.canary import guarded_empty
        # capacity-sized activations indexed by computed rows: guarded when XORL_B200_CANARIES=1
        self.h = guarded_empty((cap, I2), torch.bfloat16, dev, "ep_scratch.h")
        self.a = guarded_empty((cap, act_I), torch.bfloat16, dev, "ep_scratch.a")
        self.y = guarded_empty((cap, H), torch.bfloat16, dev, "ep_scratch.y")   # forward: expert outputs; backward: dx rows
        self.da = guarded_empty((cap, act_I), torch.bfloat16, dev, "ep_scratch.da")
        self.dys = guarded_empty((S, H), torch.bfloat16, dev, "ep_scratch.dys")
        self.slot_idx: Dict[int, torch.Tensor] = {}
        self.tok_of_slot: Dict[int, torch.Tensor] = {}
        self.q = None
        if fp8:
            from ..ops.fp8_grouped import sf_stride
            u8 = dict(device=dev, dtype=torch.uint8)
            kmax = max(H, act_I, I2)
            self.q = torch.empty((cap, kmax), **u8)
            self.sf = torch.full((cap, sf_stride(kmax)), 127, **u8)

    def quantised_tokens(self, T: int, row_bytes: int) -> torch.Tensor:
        """[T, row_bytes] bytes: e4m3 values of a token followed by its 1 x 128 scales (16-byte padded)."""
        buf = getattr(self, "_xrow", None)
        if buf is None or buf.numel() < T * row_bytes:
            buf = self._xrow = torch.zeros(T * row_bytes, device=self.h.device, dtype=torch.uint8)
        return buf[:T * row_bytes].view(T, row_bytes)

    def slot_tables(self, k: int, dev):
        if k not in self.slot_idx:
            S = self.dest_rank.numel()
            self.slot_idx[k] = torch.arange(S, device=dev, dtype=torch.int64)
            self.tok_of_slot[k] = (torch.arange(S, device=dev) // k).to(torch.int32)
        return self.slot_idx[k], self.tok_of_slot[k]


def _scratch(ws: _Workspace, I2: int, act_I: int, fp8: bool) -> _Scratch:
    sc = getattr(ws, "_scratch", None)
    if sc is None or sc.I2 != I2 or sc.I != act_I or (fp8 and sc.q is None):
        sc = _Scratch(ws, I2, act_I, fp8)
        ws._scratch = sc
    return sc


def _rows_gemm(ws, sc, a, a_cols, w, out, n_out, b_mn: int, fp8, qe_w, qe_sf, st):
    """out[rows of e, :n_out] = a[rows of e, :a_cols] @ op(w[e]) over the local expert segments."""
    lib = ws.lib
    if fp8:
        _lib.check(lib.xb_quant_mx_rows_lim(a.data_ptr(), a.stride(0), sc.q.data_ptr(), sc.q.stride(0),
                                            sc.sf.data_ptr(), sc.sf.stride(0), ws.cap, a_cols, sc.row_limit_ptr, st),
                   "xb_quant_mx_rows_lim")
        _lib.check(lib.xb_grouped_gemm_mx_rows(sc.q.data_ptr(), sc.sf.data_ptr(), qe_w.data_ptr(), qe_sf.data_ptr(),
                                               out.data_ptr(), sc.seg.data_ptr(), ws.El, ws.cap, n_out, a_cols,
                                               sc.q.stride(0), out.stride(0), sc.sf.stride(0), qe_sf.stride(1), st),
                   "xb_grouped_gemm_mx_rows")
    else:
        _lib.check(lib.xb_grouped_gemm_rows(a.data_ptr(), w.data_ptr(), out.data_ptr(), sc.seg.data_ptr(), ws.El,
                                            ws.cap, n_out, a_cols, a.stride(0), out.stride(0), b_mn, st),
                   "xb_grouped_gemm_rows")


class _FusedEPMoE(torch.autograd.Function):
    """The whole expert-parallel MoE of one layer as ONE autograd node with a hand-written backward:
    histogram -> count exchange -> plan -> dispatch push -> grouped gate_up GEMM -> SwiGLU -> grouped
    down GEMM -> return push -> weighted sum over the k slots; backward runs the same pushes in the
    opposite roles.  Around twenty kernel launches each way, no PyTorch operator, no allocation
    besides the outputs, no host synchronisation.  (The composite path above builds the same
    computation from several autograd functions and is kept for experts with biases or clamped /
    non-gated activations.)"""

    @staticmethod
    def forward(ctx, x, weights, indices, gate_up, down, ws: _Workspace, fp8_mode, no_backward: bool = False):
        lib, st = ws.lib, _lib.stream_ptr()
        T, H = x.shape
        k = indices.shape[1]
        S = T * k
        El, I2 = gate_up.shape[0], gate_up.shape[2]
        I = down.shape[1]
        fp8 = fp8_mode is not None
        sc = _scratch(ws, I2, I, fp8)
        slot_idx, tok_of_slot = sc.slot_tables(k, x.device)
        x = x.contiguous()
        idx = indices.contiguous()
        w32 = weights.detach().float().contiguous()
        qg = qd = None
        if fp8:
            from ..ops.fp8_grouped import cached_quantized_experts
            qg, qd = cached_quantized_experts(gate_up), cached_quantized_experts(down)
        # ---- plan -------------------------------------------------------------------------------
        t0 = PhaseTimes.mark()
        _lib.check(lib.xb_moe_histogram(idx.data_ptr(), S, sc.counts.data_ptr(), ws.E, st), "xb_moe_histogram")
        ws.epoch["counts"] += 1
        _lib.check(lib.xb_ep_exchange_counts(sc.counts.data_ptr(), ws.ptrs(ws.o_table), ws.ptrs(0), S_COUNTS, ws.rank,
                                             ws.N, ws.E, ws.epoch["counts"], WAIT_MS, st), "xb_ep_exchange_counts")
        _lib.check(lib.xb_ep_plan(idx.data_ptr(), S, ctypes.c_void_p(ws.heap.data_ptr() + ws.o_table), ws.rank, ws.N,
                                  ws.E, ws.El, ws.cap, sc.dest_rank.data_ptr(), sc.dest_row.data_ptr(),
                                  sc.seg.data_ptr(), sc.tot.data_ptr(), sc.overflow.data_ptr(), st), "xb_ep_plan")
        # ---- dispatch ---------------------------------------------------------------------------
        t1 = PhaseTimes.mark()
        PhaseTimes.add("fwd_plan", t0, t1)
        recv = ws.view("recv_f", ws.cap, torch.bfloat16, H)
        meta = ws.view("meta_f", ws.cap, torch.int32, 1)
        # A pass that no backward follows (the first forward under recomputation, evaluation) keeps nothing
        # of the received rows, so with fp8 experts the tokens are quantised once at the source (T rows
        # instead of the T * k received ones) and travel as e4m3 values + scales: half the bytes on NVLink
        # and no quantiser pass at the experts.  The values are those the experts would compute themselves
        # (the 1 x 128 quantiser is per row), so both passes of a recomputed layer agree bit for bit.
        # (``no_backward`` is the caller's ``not torch.is_grad_enabled()``: inside ``forward`` gradient mode is
        # always off and ``needs_input_grad`` ignores it)
        pre_q = fp8 and no_backward and os.environ.get("XORL_B200_EP_FP8_PUSH", "1") != "0"
        if pre_q:
            from ..ops.fp8_grouped import sf_stride
            rb = H + sf_stride(H)
            xrow = sc.quantised_tokens(T, rb)
            _lib.check(lib.xb_quant_mx_rows(x.data_ptr(), x.stride(0), xrow.data_ptr(), rb, xrow.data_ptr() + H, rb,
                                            T, H, st), "xb_quant_mx_rows")
            _lib.check(lib.xb_ep_prepare_recv(recv.data_ptr(), meta.data_ptr(), sc.seg.data_ptr(), sc.tot.data_ptr(), El,
                                              ws.cap, rb, st), "xb_ep_prepare_recv")
            ws.push(xrow, tok_of_slot[:S], sc.dest_rank[:S], sc.dest_row[:S], None, "recv_f", "meta_f", S_DISP, C_DISP,
                    "disp", row_bytes=rb)
        else:
            _lib.check(lib.xb_ep_prepare_recv(recv.data_ptr(), meta.data_ptr(), sc.seg.data_ptr(), sc.tot.data_ptr(), El,
                                              ws.cap, H * 2, st), "xb_ep_prepare_recv")
            ws.push(x, tok_of_slot[:S], sc.dest_rank[:S], sc.dest_row[:S], None, "recv_f", "meta_f", S_DISP, C_DISP, "disp")
        # ---- experts ----------------------------------------------------------------------------
        t2 = PhaseTimes.mark()
        PhaseTimes.add("fwd_dispatch", t1, t2)
        if pre_q:
            _lib.check(lib.xb_grouped_gemm_mx_rows(recv.data_ptr(), recv.data_ptr() + H, qg.q_nk.data_ptr(),
                                                   qg.sf_nk.data_ptr(), sc.h.data_ptr(), sc.seg.data_ptr(), ws.El, ws.cap,
                                                   I2, H, rb, sc.h.stride(0), rb, qg.sf_nk.stride(1), st),
                       "xb_grouped_gemm_mx_rows")
        else:
            _rows_gemm(ws, sc, recv, H, gate_up, sc.h, I2, 1, fp8, None if qg is None else qg.q_nk,
                       None if qg is None else qg.sf_nk, st)
        _lib.check(lib.xb_swiglu_fwd_rows(sc.h.data_ptr(), sc.a.data_ptr(), ws.cap, I, 1, sc.row_limit_ptr, st),
                   "xb_swiglu_fwd_rows")
        _rows_gemm(ws, sc, sc.a, I, down, sc.y, H, 1, fp8, None if qd is None else qd.q_nk,
                   None if qd is None else qd.sf_nk, st)
        # ---- return -----------------------------------------------------------------------------
        t3 = PhaseTimes.mark()
        PhaseTimes.add("fwd_experts", t2, t3)
        _lib.check(lib.xb_ep_meta_targets(meta.data_ptr(), ws.cap, sc.ret_rank.data_ptr(), sc.ret_slot.data_ptr(), st),
                   "xb_ep_meta_targets")
        ws.push(sc.y, None, sc.ret_rank, sc.ret_slot, None, "ret_f", None, S_RET, C_RET, "ret")
        t4 = PhaseTimes.mark()
        PhaseTimes.add("fwd_return", t3, t4)
        y_slots = ws.view("ret_f", S, torch.bfloat16, H)
        out = torch.empty((T, H), device=x.device, dtype=torch.bfloat16)
        _lib.check(lib.xb_moe_gather_sum(out.data_ptr(), out.stride(0), y_slots.data_ptr(), H, slot_idx.data_ptr(),
                                         w32.data_ptr(), T, k, H, st), "xb_moe_gather_sum")
        PhaseTimes.add("fwd_combine", t4)
        moe_ops._launches += 14 + (2 if fp8 else 0)
        ctx.ws, ctx.sc, ctx.dims, ctx.fp8_mode = ws, sc, (T, H, k, S, El, I2, I), fp8_mode
        ctx.gate_up, ctx.down = gate_up, down
        ctx.save_for_backward(w32)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.grad_sink import grad_target, mark_written
        ws, sc = ctx.ws, ctx.sc
        T, H, k, S, El, I2, I = ctx.dims
        (w32,) = ctx.saved_tensors
        gate_up, down = ctx.gate_up, ctx.down
        lib, st = ws.lib, _lib.stream_ptr()
        fp8 = ctx.fp8_mode == "fp8"
        slot_idx, tok_of_slot = sc.slot_tables(k, dout.device)
        dout = dout.contiguous()
        y_slots = ws.view("ret_f", S, torch.bfloat16, H)
        qg = qd = None
        if fp8:
            from ..ops.fp8_grouped import cached_quantized_experts
            qg, qd = cached_quantized_experts(gate_up), cached_quantized_experts(down)
        # slot gradients and routing-weight gradients
        b0 = PhaseTimes.mark()
        dys = sc.dys[:S]
        _lib.check(lib.xb_moe_gather_rows(dys.data_ptr(), H, dout.data_ptr(), dout.stride(0), tok_of_slot.data_ptr(),
                                          w32.data_ptr(), S, H, st), "xb_moe_gather_rows")
        dw = None
        if ctx.needs_input_grad[1]:
            dw = torch.empty((T, k), device=dout.device, dtype=torch.float32)
            _lib.check(lib.xb_moe_slot_dots(dw.data_ptr(), dout.data_ptr(), dout.stride(0), y_slots.data_ptr(), H,
                                            slot_idx.data_ptr(), T, k, H, st), "xb_moe_slot_dots")
        # slot gradients -> owners' rows (same plan as the dispatch)
        recv_b = ws.view("recv_b", ws.cap, torch.bfloat16, H)
        meta_b = ws.view("meta_b", ws.cap, torch.int32, 1)
        _lib.check(lib.xb_ep_prepare_recv(recv_b.data_ptr(), meta_b.data_ptr(), sc.seg.data_ptr(), sc.tot.data_ptr(), El,
                                          ws.cap, H * 2, st), "xb_ep_prepare_recv")
        ws.push(dys, None, sc.dest_rank[:S], sc.dest_row[:S], None, "recv_b", "meta_b", S_BDISP, C_BDISP, "bdisp")
        recv_f = ws.view("recv_f", ws.cap, torch.bfloat16, H)
        b1 = PhaseTimes.mark()
        PhaseTimes.add("bwd_slots_dispatch", b0, b1)
        # down projection: input gradient, then weight gradient (bf16 operands)
        _rows_gemm(ws, sc, recv_b, H, down, sc.da, I, 0, fp8, None if qd is None else qd.q_kn,
                   None if qd is None else qd.sf_kn, st)
        for w, a_rows, b_rows, M_, N_ in ((down, sc.a, recv_b, I, H),):
            tgt, fresh = grad_target(w)
            dwt = tgt if tgt is not None else torch.empty_like(w)
            _lib.check(lib.xb_grouped_gemm_wgrad(a_rows.data_ptr(), b_rows.data_ptr(), dwt.data_ptr(), sc.seg.data_ptr(),
                                                 El, ws.cap, M_, N_, a_rows.stride(0), b_rows.stride(0),
                                                 int(dwt.dtype == torch.float32), int(tgt is not None and not fresh), st),
                       "xb_grouped_gemm_wgrad")
            if tgt is not None:
                mark_written(w)
            d_down = None if tgt is not None else dwt
        # SwiGLU backward in place: h becomes dh
        _lib.check(lib.xb_swiglu_bwd_rows(sc.da.data_ptr(), sc.h.data_ptr(), sc.h.data_ptr(), ws.cap, I,
                                          sc.row_limit_ptr, st), "xb_swiglu_bwd_rows")
        tgt, fresh = grad_target(gate_up)
        dwt = tgt if tgt is not None else torch.empty_like(gate_up)
        _lib.check(lib.xb_grouped_gemm_wgrad(recv_f.data_ptr(), sc.h.data_ptr(), dwt.data_ptr(), sc.seg.data_ptr(), El,
                                             ws.cap, H, I2, recv_f.stride(0), sc.h.stride(0),
                                             int(dwt.dtype == torch.float32), int(tgt is not None and not fresh), st),
                   "xb_grouped_gemm_wgrad")
        if tgt is not None:
            mark_written(gate_up)
        d_gate_up = None if tgt is not None else dwt
        _rows_gemm(ws, sc, sc.h, I2, gate_up, sc.y, H, 0, fp8, None if qg is None else qg.q_kn,
                   None if qg is None else qg.sf_kn, st)
        # row gradients -> source slots, summed over the k slots of a token
        b2 = PhaseTimes.mark()
        PhaseTimes.add("bwd_experts", b1, b2)
        meta_f = ws.view("meta_f", ws.cap, torch.int32, 1)
        _lib.check(lib.xb_ep_meta_targets(meta_f.data_ptr(), ws.cap, sc.ret_rank.data_ptr(), sc.ret_slot.data_ptr(), st),
                   "xb_ep_meta_targets")
        ws.push(sc.y, None, sc.ret_rank, sc.ret_slot, None, "ret_b", None, S_BRET, C_BRET, "bret")
        dslots = ws.view("ret_b", S, torch.bfloat16, H)
        dx = torch.empty((T, H), device=dout.device, dtype=torch.bfloat16)
        _lib.check(lib.xb_moe_gather_sum(dx.data_ptr(), dx.stride(0), dslots.data_ptr(), H, slot_idx.data_ptr(), None,
                                         T, k, H, st), "xb_moe_gather_sum")
        PhaseTimes.add("bwd_return_sum", b2)
        moe_ops._launches += 15 + (2 if fp8 else 0)
        return dx, dw, None, d_gate_up, d_down, None, None, None


def fused_ep_forward(x, weights, indices, experts, num_experts, ctx):
    T, H = x.shape
    k = indices.shape[1]
    slots = ctx.aux.get("ep_max_slots") or T * k
    ws = _workspace(H, max(slots, T * k), num_experts, x.device)
    if T * k > ws.slots:
        raise RuntimeError(f"{T * k} token slots exceed the EP workspace ({ws.slots})")
    kw = moe_ops.experts_mlp_kwargs(experts)
    fp8_mode = kw.pop("fp8", None)
    if not kw and os.environ.get("XORL_B200_EP_SINGLE_NODE_FN", "1") == "1":
        return _FusedEPMoE.apply(x, weights, indices, experts.gate_up_proj, experts.down_proj, ws, fp8_mode,
                                 not torch.is_grad_enabled())
    kw = moe_ops.experts_mlp_kwargs(experts)
    plan = _make_plan(ws, indices)
    buf = _Dispatch.apply(x, ws, plan)
    y = moe_ops.expert_mlp_aligned(buf, plan.seg, experts.gate_up_proj, experts.down_proj, **kw)
    y_slots = _Return.apply(y, ws, plan)
    if moe_ops._permute_kernels_ok(x):
        # weighted sum over the k slots of a token in one gather kernel (slot rows are contiguous)
        slots = torch.arange(T * k, device=x.device).view(T, k)
        tok = (torch.arange(T * k, device=x.device) // k).to(torch.int32)
        return moe_ops._Combine.apply(y_slots, weights, slots, tok)
    out = (y_slots.view(T, k, H).float() * weights.unsqueeze(-1).float()).sum(1)
    return out.to(x.dtype)
