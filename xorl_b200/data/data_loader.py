"""Stateful, rank-sharded loader of packed micro-batches.

Samples are packed into bins of ``sample_packing_sequence_len`` tokens (C++ packer), bins are
distributed round-robin over data-parallel ranks, every step yields a list of
``gradient_accumulation_steps`` packed rows.  ``state_dict`` / ``load_state_dict`` give exact resume
(src/xorl/data/data_loader.py:96-393 builds the same on torchdata's StatefulDataLoader)."""
from __future__ import annotations

import threading
from queue import Queue
from typing import Any, Dict, Iterator, List, Optional

import numpy as np
import torch

from .collators import PackingCollator, SequenceShardCollator
from .packing import pack_bins


class PackedDataLoader:
    def __init__(self, dataset, *, packing_len: int, micro_batch_size: int = 1, grad_accum: int = 1,
                 dp_rank: int = 0, dp_size: int = 1, packing_method: str = "sequential",
                 group_size: int = 100000, pad_to_multiple_of: int = 128, shuffle: bool = True,
                 seed: int = 42, drop_last: bool = True, pin_memory: bool = True,
                 shard_collator: Optional[SequenceShardCollator] = None, prefetch: int = 2,
                 pad_to_length: int = 0):
        self.dataset = dataset
        self.packing_len = packing_len
        self.mbs, self.ga = micro_batch_size, grad_accum
        self.dp_rank, self.dp_size = dp_rank, dp_size
        self.seed, self.shuffle, self.drop_last = seed, shuffle, drop_last
        self.pin = pin_memory and torch.cuda.is_available()
        self.collate = PackingCollator(pad_to_multiple_of, shift=True, pad_to_length=pad_to_length)
        self.shard = shard_collator
        self.prefetch = prefetch
        lengths = np.maximum(np.asarray(dataset.lengths) - 1, 1)  # after the shift
        self.bins = pack_bins(lengths, packing_len, packing_method, group_size)
        self.epoch = 0
        self.cursor = 0  # index into this epoch's per-rank bin order (in units of steps)
        per_step = self.mbs * self.ga * self.dp_size
        self.steps_per_epoch = len(self.bins) // per_step if drop_last else -(-len(self.bins) // per_step)

    def __len__(self) -> int:
        return self.steps_per_epoch

    def _order(self, epoch: int) -> np.ndarray:
        order = np.arange(len(self.bins))
        if self.shuffle:
            np.random.default_rng(self.seed + epoch).shuffle(order)
        return order

    def _make_step(self, order: np.ndarray, step: int) -> List[Dict[str, torch.Tensor]]:
        per_step = self.mbs * self.ga * self.dp_size
        base = step * per_step
        rows = []
        for a in range(self.ga):
            samples: List[Any] = []
            for m in range(self.mbs):
                k = base + (a * self.mbs + m) * self.dp_size + self.dp_rank
                if k >= len(order):
                    continue
                samples += [self.dataset[i] for i in self.bins[order[k]]]
            if not samples:
                continue
            row = self.collate(samples)
            if self.shard is not None:
                row = self.shard(row)
            if self.pin:
                row = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in row.items()}
            rows.append(row)
        return rows

    def __iter__(self) -> Iterator[List[Dict[str, torch.Tensor]]]:
        order = self._order(self.epoch)
        q: Queue = Queue(maxsize=max(1, self.prefetch))
        start = self.cursor
        stop = threading.Event()

        def worker():
            for s in range(start, self.steps_per_epoch):
                if stop.is_set():
                    return
                q.put(self._make_step(order, s))
            q.put(None)

        t = threading.Thread(target=worker, daemon=True)
        t.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    break
                self.cursor += 1
                yield item
        finally:
            stop.set()
        self.epoch += 1
        self.cursor = 0

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.epoch, self.cursor = int(sd["epoch"]), int(sd["cursor"])
        self.seed = int(sd.get("seed", self.seed))


def build_dataloader(dataset, data_args, train_args, pstate, shard_collator=None) -> PackedDataLoader:
    return PackedDataLoader(
        dataset, packing_len=int(data_args.sample_packing_sequence_len or 4096),
        micro_batch_size=train_args.micro_batch_size, grad_accum=train_args.gradient_accumulation_steps,
        dp_rank=pstate.dp_rank, dp_size=pstate.dp_size,
        packing_method=data_args.sample_packing_method or "sequential",
        group_size=int(data_args.sample_packing_group_size or 100000),
        pad_to_multiple_of=int(data_args.pad_to_multiple_of or 1),
        shuffle=bool(data_args.shuffle_merged_datasets), seed=train_args.seed,
        drop_last=bool(data_args.dataloader_drop_last), pin_memory=bool(data_args.dataloader_pin_memory),
        shard_collator=shard_collator, prefetch=int(data_args.dataloader_prefetch_factor or 2))
