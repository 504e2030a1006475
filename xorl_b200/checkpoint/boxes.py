"""Checkpoint pieces straight from the ZeRO engine's flat shards.

A rank's flat shard covers a contiguous range of the concatenated parameters of a unit, so of one
parameter it holds a contiguous *flat* range -- in the parameter's own N-d shape that is at most
``2 * (ndim - 1) + 1`` rectangular boxes (a partial first row, whole rows, a partial last row, and the
same again one dimension down).  Each box is a view of the shard, so saving needs no all-gather and no
copy, and loading writes into the shard in place; ``torch.distributed.checkpoint`` stores a tensor as a
list of such chunks with offsets and sizes whatever object produced them, which keeps the on-disk
layout that of the reference (src/xorl/checkpoint/checkpointer.py: one logical tensor per parameter
FQN, resharded on load by chunk intersection) and lets checkpoints move between world sizes and
between this layout and ``DTensor``-saved ones.

Tensor-parallel slices (row sections or a column range of the full matrix) and expert-parallel slices
(a range of experts) only shift or split the boxes: ``RowMap`` translates local rows into rows of the
full tensor.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
from torch.distributed.checkpoint.metadata import (ChunkStorageMetadata, MetadataIndex, TensorProperties,
                                                   TensorStorageMetadata)
from torch.distributed.checkpoint.planner import LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType
from torch.distributed.checkpoint.planner_helpers import create_read_items_for_chunk_list

Box = Tuple[Tuple[int, ...], Tuple[int, ...], int, int]     # offsets, sizes, flat start, flat end (local)


def flat_range_boxes(shape: Sequence[int], a: int, b: int) -> List[Box]:
    """Rectangular boxes (in the coordinates of ``shape``) that tile the flat range ``[a, b)`` of a
    contiguous tensor of that shape, in flat order."""
    shape = tuple(shape) if len(shape) else (1,)
    if a >= b:
        return []
    if len(shape) == 1:
        return [((a,), (b - a,), a, b)]
    R = math.prod(shape[1:])
    r0, c0 = divmod(a, R)
    r1, c1 = divmod(b, R)
    sub = lambda row, lo, hi: [((row,) + o, (1,) + s, row * R + fa, row * R + fb)
                               for o, s, fa, fb in flat_range_boxes(shape[1:], lo, hi)]
    if r0 == r1:
        return sub(r0, c0, c1)
    out: List[Box] = []
    if c0:
        out += sub(r0, c0, R)
        r0 += 1
    if r1 > r0:
        out.append(((r0,) + (0,) * (len(shape) - 1), (r1 - r0,) + shape[1:], r0 * R, r1 * R))
    if c1:
        out += sub(r1, 0, c1)
    return out


@dataclasses.dataclass
class RowMap:
    """Where a local slice sits in the full tensor: ``segments`` are (local row start, rows, full row
    start) runs along dim 0 (sorted, covering all local rows); ``col_offset`` shifts dim 1."""
    segments: List[Tuple[int, int, int]]
    col_offset: int = 0

    @staticmethod
    def identity(rows: int) -> "RowMap":
        return RowMap([(0, rows, 0)])

    @staticmethod
    def row_sections(sections: Sequence[int], tp: int, rank: int) -> "RowMap":
        """Column-parallel weight: every section of the output rows is split evenly over ``tp``."""
        segs, loc, full = [], 0, 0
        for s in sections:
            per = s // tp
            segs.append((loc, per, full + rank * per))
            loc += per
            full += s
        return RowMap(segs)

    def translate(self, box: Box) -> List[Box]:
        off, size, fa, fb = box
        r, n = off[0], size[0]
        per_row = (fb - fa) // max(n, 1)
        out = []
        for ls, ln, gs in self.segments:
            lo, hi = max(r, ls), min(r + n, ls + ln)
            if lo >= hi:
                continue
            goff = (gs + lo - ls,) + tuple(off[1:])
            if self.col_offset and len(goff) > 1:
                goff = (goff[0], goff[1] + self.col_offset) + goff[2:]
            out.append((goff, (hi - lo,) + tuple(size[1:]), fa + (lo - r) * per_row, fa + (hi - r) * per_row))
        return out


class BoxedTensor:
    """This rank's pieces of one logical tensor: ``boxes`` is a list of (offsets, sizes, tensor) where
    every tensor has the shape ``sizes`` and is a view of the storage that owns the data."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype,
                 boxes: List[Tuple[Tuple[int, ...], Tuple[int, ...], torch.Tensor]]):
        self.shape = tuple(shape) if len(shape) else (1,)
        self.dtype = dtype
        self.boxes = boxes

    @staticmethod
    def from_flat(flat: torch.Tensor, local_shape: Sequence[int], a: int, b: int, flat_origin: int,
                  full_shape: Optional[Sequence[int]] = None, row_map: Optional[RowMap] = None) -> "BoxedTensor":
        """``flat[flat_origin + x]`` holds element ``x`` (flat index in ``local_shape``) for ``x`` in
        ``[a, b)``.  ``row_map`` places the local slice inside ``full_shape``."""
        boxes = []
        for box in flat_range_boxes(local_shape, a, b):
            for off, size, fa, fb in (row_map.translate(box) if row_map is not None else [box]):
                boxes.append((off, size, flat[flat_origin + fa:flat_origin + fb].view(size)))
        return BoxedTensor(full_shape if full_shape is not None else local_shape, flat.dtype, boxes)

    def to_host(self) -> "BoxedTensor":
        """A host snapshot (for asynchronous saves: the device shards keep changing)."""
        return BoxedTensor(self.shape, self.dtype, [(o, s, t.detach().to("cpu", copy=True)) for o, s, t in self.boxes])

    def numel_local(self) -> int:
        return sum(t.numel() for _, _, t in self.boxes)


def _split(state_dict):
    boxed = {k: v for k, v in state_dict.items() if isinstance(v, BoxedTensor)}
    rest = {k: v for k, v in state_dict.items() if not isinstance(v, BoxedTensor)}
    return boxed, rest


class BoxSavePlanner(DefaultSavePlanner):
    def set_up_planner(self, state_dict, storage_meta=None, is_coordinator=False) -> None:
        self._boxed, rest = _split(state_dict)
        super().set_up_planner(rest, storage_meta, is_coordinator)

    def create_local_plan(self) -> SavePlan:
        plan = super().create_local_plan()
        items = list(plan.items)
        for fqn, bt in self._boxed.items():
            for off, size, t in bt.boxes:
                items.append(WriteItem(
                    index=MetadataIndex(fqn, torch.Size(off)), type=WriteItemType.SHARD,
                    tensor_data=TensorWriteData(
                        chunk=ChunkStorageMetadata(offsets=torch.Size(off), sizes=torch.Size(size)),
                        properties=TensorProperties.create_from_tensor(t), size=torch.Size(bt.shape))))
        self.plan = dataclasses.replace(plan, items=items)
        return self.plan

    def lookup_object(self, index: MetadataIndex):
        bt = self._boxed.get(index.fqn)
        if bt is None:
            return super().lookup_object(index)
        for off, _, t in bt.boxes:
            if tuple(off) == tuple(index.offset):
                return t
        raise KeyError(f"{index.fqn}: no local piece at offset {tuple(index.offset)}")


class BoxLoadPlanner(DefaultLoadPlanner):
    def set_up_planner(self, state_dict, metadata=None, is_coordinator=False) -> None:
        self._boxed, rest = _split(state_dict)
        super().set_up_planner(rest, metadata, is_coordinator)

    def create_local_plan(self) -> LoadPlan:
        plan = super().create_local_plan()
        items = list(plan.items)
        for fqn, bt in self._boxed.items():
            md = self.metadata.state_dict_metadata.get(fqn)
            if md is None:
                if self.allow_partial_load:
                    continue
                raise RuntimeError(f"missing key in checkpoint: {fqn}")
            if not isinstance(md, TensorStorageMetadata) or tuple(md.size) != tuple(bt.shape):
                raise ValueError(f"{fqn}: checkpoint holds {getattr(md, 'size', type(md).__name__)}, "
                                 f"the model expects {bt.shape}")
            chunks = [ChunkStorageMetadata(offsets=torch.Size(o), sizes=torch.Size(s)) for o, s, _ in bt.boxes]
            items += create_read_items_for_chunk_list(fqn, md, chunks)
        return dataclasses.replace(plan, items=items)

    def lookup_tensor(self, index: MetadataIndex) -> torch.Tensor:
        bt = self._boxed.get(index.fqn)
        if bt is None:
            return super().lookup_tensor(index)
        if index.index is not None and index.index < len(bt.boxes) and \
                tuple(bt.boxes[index.index][0]) == tuple(index.offset):
            return bt.boxes[index.index][2]
        for off, _, t in bt.boxes:
            if tuple(off) == tuple(index.offset):
                return t
        raise KeyError(f"{index.fqn}: no local piece at offset {tuple(index.offset)}")
