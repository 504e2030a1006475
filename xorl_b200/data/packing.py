"""Sample packing: first-fit-decreasing and sequential, through the C++ host library
(``csrc/host/ffd_pack.cpp``).  Same grouping semantics as src/xorl/data/prepare/packing.py:30-190
(``sample_packing_group_size`` samples are packed at a time, bins hold
``sample_packing_sequence_len`` tokens)."""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import numpy as np

from ..ops import _lib


def _as_i64(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int64))


def pack_bins(lengths: Sequence[int], capacity: int, method: str = "sequential",
              group_size: int = 100000) -> List[List[int]]:
    """Returns the sample indices of every bin."""
    lens = _as_i64(lengths)
    n = int(lens.shape[0])
    if n == 0:
        return []
    out = np.empty(n, dtype=np.int64)
    lib = _lib.host_lib()
    lp = lens.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))
    op = out.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))
    if method in ("ffd", "multipack", "first_fit_decreasing"):
        lib.xb_ffd_pack.restype = ctypes.c_int64
        nb = lib.xb_ffd_pack(lp, ctypes.c_int64(n), ctypes.c_int64(capacity),
                             ctypes.c_int64(group_size), op)
    elif method == "sequential":
        lib.xb_sequential_pack.restype = ctypes.c_int64
        nb = lib.xb_sequential_pack(lp, ctypes.c_int64(n), ctypes.c_int64(capacity), op)
    else:
        raise ValueError(f"unknown sample_packing_method {method!r}")
    bins: List[List[int]] = [[] for _ in range(int(nb))]
    for i, b in enumerate(out.tolist()):
        bins[b].append(i)
    return bins
