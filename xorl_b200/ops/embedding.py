"""Token embedding gather / scatter-add (``csrc/elementwise.cu``)."""
from __future__ import annotations

import torch

from . import _lib
from .grad_sink import deliver_param_grad, grad_target, mark_written

_launches = 0


def launch_count() -> int:
    return _launches


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        global _launches
        flat = ids.reshape(-1).contiguous()
        T = flat.numel()
        V, H = table.shape
        out = torch.empty((T, H), device=table.device, dtype=table.dtype)
        _lib.check(_lib.cuda_lib().xb_embedding_fwd(flat.data_ptr(), table.data_ptr(),
                                                    out.data_ptr(), T, H, V, _lib.stream_ptr()),
                   "xb_embedding_fwd")
        _launches += 1
        ctx.save_for_backward(flat)
        ctx.table = table
        ctx.ids_shape = ids.shape
        return out.reshape(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        global _launches
        (flat,) = ctx.saved_tensors
        table = ctx.table
        V, H = table.shape
        T = flat.numel()
        d2 = dout.reshape(T, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        tgt, fresh = grad_target(table)
        lib = _lib.cuda_lib()
        if tgt is not None:
            if fresh:
                tgt.zero_()
                mark_written(table)
            _lib.check(lib.xb_embedding_bwd(flat.data_ptr(), d2.data_ptr(), tgt.data_ptr(),
                                            int(tgt.dtype == torch.float32), T, H, V,
                                            _lib.stream_ptr()), "xb_embedding_bwd")
            _launches += 1
            return None, None
        dt = torch.zeros((V, H), device=table.device, dtype=torch.float32)
        _lib.check(lib.xb_embedding_bwd(flat.data_ptr(), d2.data_ptr(), dt.data_ptr(), 1, T, H, V,
                                        _lib.stream_ptr()), "xb_embedding_bwd")
        _launches += 1
        return None, dt.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if table.is_cuda and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
        return _Embedding.apply(ids, table)
    return torch.nn.functional.embedding(ids, table)
