"""Fused peer-memory transport for the ZeRO engine.

One symmetric heap per rank (allocated with ``torch.distributed._symmetric_memory`` and mapped
into every peer of the shard group) holds

* a 16 KiB flag area (epochs for barriers and for the ready/done handshake of gradient buffers),
* the compute-dtype parameter shards of every unit (what the all-gather reads),
* a small ring of full-size gradient buffers (what the reduce-scatter reads).

Collectives are the kernels of ``csrc/comm.cu``: a pull all-gather with plain peer loads and a
reduce-scatter that sums the owned slice over all peers in fp32 (peer loads in fixed rank order,
or one NVSwitch ``multimem.ld_reduce`` per vector), scales, accumulates into the fp32 gradient
shard and emits gradient-norm partials, all in one pass with bf16 on the wire.  They run on the
engine's side stream and overlap the neighbouring units' compute.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..utils.logging import info_rank0

FLAG_BYTES = 16 * 1024
BARRIER_SLOT = 0          # [0, 16)
BUF_SLOT0 = 64            # per gradient buffer: ready[16], done[16], counter -> 64 ints each
NUM_GRAD_BUFS = 3
WAIT_MS = 2000
# CTAs of the collective kernels (512 threads, no shared memory: they share SMs with the GEMM CTAs)
# and 16-byte loads in flight per thread of the all-gather
AG_CTAS = int(os.environ.get("XORL_B200_AG_CTAS", "128"))
AG_UNROLL = int(os.environ.get("XORL_B200_AG_UNROLL", "8"))
RS_CTAS = int(os.environ.get("XORL_B200_RS_CTAS", "128"))
# "dma": copy engines move the bytes (no SM taken from the GEMMs next to the collective), kernels only
# synchronise and reduce locally; "kernel": the pull kernels with peer loads
MODE = os.environ.get("XORL_B200_ZERO_TRANSPORT", "dma")


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class SymmetricTransport:
    def __init__(self, engine, heap: torch.Tensor, hdl, layout: Dict):
        self.engine = engine
        self.heap = heap
        self.hdl = hdl
        self.rank, self.world = hdl.rank, hdl.world_size
        self.base_ptrs: List[int] = [int(p) for p in hdl.buffer_ptrs]
        self.mc_base = 0
        if os.environ.get("XORL_B200_NVLS", "0") == "1" and hdl.has_multicast_support(
                engine.device.type, engine.device.index):
            self.mc_base = int(hdl.multicast_ptr)
        self.layout = layout
        self.barrier_epoch = 0
        self.buf_epoch = [0] * NUM_GRAD_BUFS
        self.buf_in_use = [False] * NUM_GRAD_BUFS
        self.buf_event = [None] * NUM_GRAD_BUFS
        self.buf_cursor = 0
        self.lib = _lib.cuda_lib()
        self._flag_ptrs = (ctypes.c_ulonglong * self.world)(*self.base_ptrs)
        self.partial = torch.zeros(max(RS_CTAS, 64), device=engine.device, dtype=torch.float32)
        self.mode = MODE if MODE in ("dma", "kernel") else "dma"
        self.staging: Optional[torch.Tensor] = None      # [world, shard] bf16, DMA reduce-scatter
        self.launches = 0

    # ------------------------------------------------------------------------------------------
    @classmethod
    def create(cls, engine) -> Optional["SymmetricTransport"]:
        if engine.shard_world <= 1 or not engine.is_cuda or engine.shard_pg is None:
            return None
        if engine.compute_dtype != torch.bfloat16:
            return None
        import torch.distributed._symmetric_memory as symm_mem
        groups = [g for g in engine.all_groups() if g.world == engine.shard_world and g.pg is engine.shard_pg]
        es = 2
        off = FLAG_BYTES
        layout = {"shard": {}, "grad": []}
        for g in groups:
            layout["shard"][id(g)] = off
            off = _align(off + g.shard_numel * es)
        max_padded = max(g.padded for g in groups)
        for _ in range(NUM_GRAD_BUFS):
            layout["grad"].append(off)
            off = _align(off + max_padded * es)
        layout["grad_numel"] = max_padded
        total = off
        heap = symm_mem.empty(total, dtype=torch.uint8, device=engine.device)
        heap[:FLAG_BYTES].zero_()
        hdl = symm_mem.rendezvous(heap, engine.shard_pg)
        self = cls(engine, heap, hdl, layout)
        # move the compute-dtype shards into the heap
        for g in groups:
            o = layout["shard"][id(g)]
            view = heap[o:o + g.shard_numel * es].view(torch.bfloat16)
            view.copy_(g.shard_lp)
            g.shard_lp = view
        torch.cuda.synchronize()
        dist.barrier(group=engine.shard_pg)
        info_rank0(f"symmetric heap: {total / 2 ** 30:.2f} GiB per rank, {len(groups)} parameter "
                   f"groups, {NUM_GRAD_BUFS} gradient buffers, multimem={'on' if self.mc_base else 'off'}")
        self._groups = {id(g) for g in groups}
        self._shard_sizes = [g.shard_numel for g in groups]
        return self

    # ------------------------------------------------------------------------------------------
    def _ptrs(self, offset: int):
        return (ctypes.c_ulonglong * self.world)(*[b + offset for b in self.base_ptrs])

    def can_gather(self, g) -> bool:
        return id(g) in self._groups

    def can_reduce(self, g) -> bool:
        return id(g) in self._groups

    def step_barrier(self, stream) -> None:
        """All ranks have finished writing their parameter shards (optimizer step) before any
        peer reads them."""
        self.barrier_epoch += 1
        _lib.check(self.lib.xb_symm_barrier(self._flag_ptrs, BARRIER_SLOT, self.rank, self.world,
                                            self.barrier_epoch, WAIT_MS, stream.cuda_stream),
                   "xb_symm_barrier")
        self.launches += 1

    def all_gather(self, g, comm_stream) -> None:
        eng = self.engine
        comm_stream.wait_stream(torch.cuda.current_stream())
        srcs = self._ptrs(self.layout["shard"][id(g)])
        if self.mode == "dma":
            _lib.check(self.lib.xb_symm_allgather_dma(g.full.data_ptr(), srcs, g.shard_numel * 2, self.rank,
                                                      self.world, comm_stream.cuda_stream), "xb_symm_allgather_dma")
        else:
            _lib.check(self.lib.xb_symm_allgather(g.full.data_ptr(), srcs, g.shard_numel * 2, self.rank,
                                                  self.world, AG_CTAS | (AG_UNROLL << 16), comm_stream.cuda_stream),
                       "xb_symm_allgather")
        g.gather_event = torch.cuda.Event()
        g.gather_event.record(comm_stream)
        self.launches += 1

    # ---- gradient buffers -----------------------------------------------------------------------
    def take_grad_buffer(self, g) -> torch.Tensor:
        """Next buffer of the ring; the compute stream first waits until every peer has finished
        reading its previous contents."""
        b = self.buf_cursor
        for _ in range(NUM_GRAD_BUFS):
            if not self.buf_in_use[b]:
                break
            b = (b + 1) % NUM_GRAD_BUFS
        else:
            raise RuntimeError("all symmetric gradient buffers are in use")
        self.buf_cursor = (b + 1) % NUM_GRAD_BUFS
        self.buf_in_use[b] = True
        if self.buf_event[b] is not None:
            # this rank's own reduce-scatter of the previous contents must have finished
            torch.cuda.current_stream().wait_event(self.buf_event[b])
            self.buf_event[b] = None
        o = self.layout["grad"][b]
        prev = self.buf_epoch[b]
        if prev > 0:
            flags = self.base_ptrs[self.rank] + 4 * (BUF_SLOT0 + 64 * b + 16)
            _lib.check(self.lib.xb_symm_wait(ctypes.c_void_p(flags), self.world, self.rank, prev,
                                             WAIT_MS, torch.cuda.current_stream().cuda_stream),
                       "xb_symm_wait")
            self.launches += 1
        buf = self.heap[o:o + g.padded * 2].view(torch.bfloat16)
        buf._xb_slot = b
        g._xb_grad_slot = b
        return buf

    def reduce_scatter_accumulate(self, g, gf: torch.Tensor, accumulate: bool, comm_stream) -> None:
        b = g._xb_grad_slot
        self.buf_epoch[b] += 1
        epoch = self.buf_epoch[b]
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        comm_stream.wait_event(ev)
        o = self.layout["grad"][b]
        grads = self._ptrs(o)
        slot = BUF_SLOT0 + 64 * b
        mc = self.mc_base + o if self.mc_base else 0
        # sum-of-squares partials of the updated shard come out of the same pass (one per CTA); they are
        # only kept when nothing later in the step changes the shard (engine._early_norm_ok)
        want_sq = self.engine._early_norm_ok(g)
        partial = self.partial[:RS_CTAS] if want_sq else None
        if self.mode == "dma" and not mc:
            # 1. everybody's gradients for this buffer are final
            _lib.check(self.lib.xb_symm_barrier(self._flag_ptrs, slot, self.rank, self.world, epoch, WAIT_MS,
                                                comm_stream.cuda_stream), "xb_symm_barrier")
            # 2. copy engines bring this rank's slice of every peer's buffer into local staging
            if self.staging is None or self.staging.numel() < self.world * g.shard_numel:
                from ..utils.canary import guarded_empty
                self.staging = guarded_empty(self.world * max(gg_numel for gg_numel in self._shard_sizes),
                                             torch.bfloat16, self.engine.device, "zero_transport.staging")
            sbytes = g.shard_numel * 2
            _lib.check(self.lib.xb_symm_gather_slices_dma(self.staging.data_ptr(), grads, g.rank * sbytes, sbytes,
                                                          self.rank, self.world, comm_stream.cuda_stream),
                       "xb_symm_gather_slices_dma")
            # 3. the reduce kernel on local pointers: staging slot r (own slice: in place), arranged so
            #    that pointer + slice offset lands on the slice
            base = self.staging.data_ptr()
            local = [(base + r * sbytes - g.rank * sbytes) if r != self.rank else self.base_ptrs[r] + o
                     for r in range(self.world)]
            lptrs = (ctypes.c_ulonglong * self.world)(*local)
            _lib.check(self.lib.xb_symm_reduce_scatter(
                g.grad_shard.data_ptr(), lptrs, ctypes.c_ulonglong(0), g.rank * g.shard_numel, g.shard_numel,
                int(accumulate), 1.0, _lib.ptr(partial), self._flag_ptrs, slot, slot + 16, slot + 32, self.rank,
                self.world, epoch, WAIT_MS, RS_CTAS, comm_stream.cuda_stream), "xb_symm_reduce_scatter")
            self.launches += 1
        else:
            _lib.check(self.lib.xb_symm_reduce_scatter(
                g.grad_shard.data_ptr(), grads, ctypes.c_ulonglong(mc), g.rank * g.shard_numel,
                g.shard_numel, int(accumulate), 1.0, _lib.ptr(partial), self._flag_ptrs, slot, slot + 16, slot + 32,
                self.rank, self.world, epoch, WAIT_MS, RS_CTAS, comm_stream.cuda_stream),
                "xb_symm_reduce_scatter")
        if want_sq:
            with torch.cuda.stream(comm_stream):
                if g.sq is None:
                    g.sq = torch.zeros(1, device=self.engine.device, dtype=torch.float32)
                torch.sum(partial, dim=0, keepdim=True, out=g.sq)
            g.sq_valid = True
        g.reduce_event = torch.cuda.Event()
        g.reduce_event.record(comm_stream)
        self.buf_event[b] = g.reduce_event
        self.buf_in_use[b] = False
        self.launches += 1
