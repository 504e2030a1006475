"""Teacher outputs for on-policy distillation.

The student samples sequences; a (larger) teacher scores exactly those tokens once; training then
minimises the reverse-KL estimate ``log p_student - log p_teacher`` on the sampled tokens
(``opd_loss``).  ``TeacherLogprobStore`` keeps the teacher's per-token log-probabilities keyed by a
content hash of the token sequence: an LRU of tensors in memory over append-only shard files on
disk, so that scoring and training can run in different processes or at different times
(src/xorl/distillation/: teacher caches and stores)."""
from __future__ import annotations

import hashlib
import json
import os
import struct
from collections import OrderedDict
from typing import Any, Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch


def sequence_key(tokens: Sequence[int]) -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(struct.pack(f"<{len(tokens)}q", *[int(t) for t in tokens]))
    return h.hexdigest()


class TeacherLogprobStore:
    def __init__(self, directory: Optional[str] = None, max_in_memory: int = 4096, shard_entries: int = 1024):
        self.dir = directory
        self.max_in_memory = max_in_memory
        self.shard_entries = shard_entries
        self.mem: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self.index: Dict[str, List[Any]] = {}           # key -> [shard file, offset, length]
        self._pending: List[tuple] = []
        self.hits = self.misses = 0
        if directory:
            os.makedirs(directory, exist_ok=True)
            ip = os.path.join(directory, "index.json")
            if os.path.exists(ip):
                with open(ip) as f:
                    self.index = json.load(f)

    def __len__(self):
        return len(set(self.index) | set(self.mem))

    def __contains__(self, tokens) -> bool:
        k = tokens if isinstance(tokens, str) else sequence_key(tokens)
        return k in self.mem or k in self.index

    def put(self, tokens: Sequence[int], logprobs) -> str:
        lp = torch.as_tensor(logprobs, dtype=torch.float32).detach().cpu().reshape(-1)
        if lp.numel() != len(tokens):
            raise ValueError(f"{lp.numel()} log-probs for {len(tokens)} tokens")
        k = sequence_key(tokens)
        self._remember(k, lp)
        if self.dir:
            self._pending.append((k, lp))
            if len(self._pending) >= self.shard_entries:
                self.flush()
        return k

    def _remember(self, k: str, lp: torch.Tensor) -> None:
        self.mem[k] = lp
        self.mem.move_to_end(k)
        while len(self.mem) > self.max_in_memory:
            self.mem.popitem(last=False)

    def get(self, tokens: Sequence[int]) -> Optional[torch.Tensor]:
        k = sequence_key(tokens)
        if k in self.mem:
            self.mem.move_to_end(k)
            self.hits += 1
            return self.mem[k]
        ent = self.index.get(k)
        if ent is None:
            self.misses += 1
            return None
        fname, off, n = ent
        arr = np.fromfile(os.path.join(self.dir, fname), dtype=np.float32, count=n, offset=off * 4)
        lp = torch.from_numpy(arr.copy())
        self._remember(k, lp)
        self.hits += 1
        return lp

    def flush(self) -> None:
        if not (self.dir and self._pending):
            return
        n_shards = len({v[0] for v in self.index.values()})
        fname = f"teacher-{n_shards:06d}.f32"
        off = 0
        with open(os.path.join(self.dir, fname), "wb") as f:
            for k, lp in self._pending:
                f.write(lp.numpy().astype(np.float32).tobytes())
                self.index[k] = [fname, off, int(lp.numel())]
                off += int(lp.numel())
        self._pending = []
        tmp = os.path.join(self.dir, "index.json.tmp")
        with open(tmp, "w") as f:
            json.dump(self.index, f)
        os.replace(tmp, os.path.join(self.dir, "index.json"))


def score_with_teacher(teacher_runner, datums: Iterable[Dict[str, Any]], store: TeacherLogprobStore,
                       model_id: str = "default", batch: int = 16) -> int:
    """Runs the teacher's forward pass over datums that are not in the store yet.  ``teacher_runner``
    is a ``ModelRunner`` (or anything with the same ``forward``).  Returns the number scored."""
    todo = [d for d in datums if d["tokens"] not in store]
    for s in range(0, len(todo), batch):
        chunk = todo[s:s + batch]
        out = teacher_runner.forward(model_id, chunk, None)
        for d, lp in zip(chunk, out["logprobs"]):
            store.put(d["tokens"], lp)
    store.flush()
    return len(todo)


def attach_teacher_logprobs(datums: List[Dict[str, Any]], store: TeacherLogprobStore) -> List[Dict[str, Any]]:
    """Adds ``teacher_logprobs`` (the loss input of ``opd_loss``) to every datum; raises KeyError for
    sequences the teacher has not scored."""
    out = []
    for d in datums:
        lp = store.get(d["tokens"])
        if lp is None:
            raise KeyError("sequence has no teacher log-probabilities; run score_with_teacher first")
        nd = dict(d)
        nd["teacher_logprobs"] = lp.tolist()
        out.append(nd)
    return out
