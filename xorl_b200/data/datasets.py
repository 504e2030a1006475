"""Datasets: synthetic ("dummy"), pre-tokenised JSONL / parquet / arrow, and a tokenising text
loader.  ``prepare_datasets`` mirrors src/xorl/data/prepare/prepare_datasets.py: every entry of
``data.datasets`` is ``{path, type, max_seq_len, ...}``; ``path: dummy`` builds identical samples
``[1, 2, ..., L-1, 0]`` on every rank without I/O (src/xorl/data/prepare/prepare_datasets.py:43-87)."""
from __future__ import annotations

import glob
import json
import os
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset


class TokenDataset(Dataset):
    """In-memory list of samples with ``input_ids`` / ``labels`` (unshifted) as int64 arrays."""

    def __init__(self, samples: List[Dict[str, np.ndarray]]):
        self.samples = samples

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        return self.samples[i]

    @property
    def lengths(self) -> np.ndarray:
        return np.array([len(s["input_ids"]) for s in self.samples], dtype=np.int64)


class DummyDataset(Dataset):
    """``num_samples`` identical samples of length k*16+1 (so that the shifted length is a
    multiple of 16), tokens 1..L-1 followed by the end-of-document id 0."""

    def __init__(self, seq_len: int, num_samples: int = 4096, vocab_size: int = 151936):
        L = max(1, ((max(seq_len, 1) - 1) // 16) * 16 + 1)
        toks = (np.arange(L, dtype=np.int64) + 1) % vocab_size
        toks[-1] = 0
        self.sample = {"input_ids": toks, "labels": toks.copy()}
        self.n = num_samples
        self.sample_len = L

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return self.sample

    @property
    def lengths(self) -> np.ndarray:
        return np.full(self.n, self.sample_len, dtype=np.int64)


class RandomTokenDataset(Dataset):
    """Documents with lengths uniform in [min_len, max_len] and tokens uniform over the vocabulary
    (deterministic per index)."""

    def __init__(self, num_samples: int, min_len: int, max_len: int, vocab_size: int, seed: int = 0):
        self.n, self.min_len, self.max_len, self.vocab, self.seed = num_samples, min_len, max_len, vocab_size, seed
        rng = np.random.default_rng(seed)
        self._lengths = rng.integers(min_len, max_len + 1, size=num_samples, dtype=np.int64)

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        rng = np.random.default_rng(self.seed * 1000003 + i + 1)
        toks = rng.integers(0, self.vocab, size=int(self._lengths[i]), dtype=np.int64)
        return {"input_ids": toks, "labels": toks.copy()}

    @property
    def lengths(self) -> np.ndarray:
        return self._lengths


def _read_jsonl(path: str) -> List[Dict[str, Any]]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
    return rows


def _load_rows(path: str, split: str = "train") -> List[Dict[str, Any]]:
    files: List[str] = []
    if os.path.isdir(path) and os.path.exists(os.path.join(path, "meta.json")) and \
            glob.glob(os.path.join(path, "data*.arrow")):
        # a directory written by ``cli.preprocess``: ``data*.arrow`` (one file or numbered shards) holds the
        # training rows, ``eval*.arrow`` the evaluation rows; the json files beside them are not data
        files = sorted(glob.glob(os.path.join(path, ("eval" if split in ("eval", "test", "validation") else "data") + "*.arrow")))
        if not files:
            raise FileNotFoundError(f"{path} holds no {split} split")
    elif os.path.isdir(path):
        for ext in ("*.jsonl", "*.json", "*.parquet", "*.arrow"):
            files += sorted(glob.glob(os.path.join(path, ext)))
    else:
        files = [path]
    rows: List[Dict[str, Any]] = []
    for f in files:
        if f.endswith(".jsonl"):
            rows += _read_jsonl(f)
        elif f.endswith(".json"):
            with open(f) as fh:
                d = json.load(fh)
            rows += d if isinstance(d, list) else [d]
        elif f.endswith(".parquet"):
            import pyarrow.parquet as pq
            rows += pq.read_table(f).to_pylist()
        elif f.endswith(".arrow"):
            import pyarrow as pa
            with pa.memory_map(f) as src:
                rows += pa.ipc.open_file(src).read_all().to_pylist()
        else:
            raise ValueError(f"unsupported dataset file {f}")
    return rows


def _spec_digest(spec: Dict[str, Any], tokenizer, select_columns) -> str:
    """Key of a prepared dataset: the spec, the tokenizer's identity, and the size / mtime of every
    source file, so that an edited file or another tokenizer never hits a stale cache
    (src/xorl/data/prepare/hash.py)."""
    import hashlib
    path = spec.get("path", "")
    files = []
    if os.path.isdir(path):
        for ext in ("*.jsonl", "*.json", "*.parquet", "*.arrow"):
            files += sorted(glob.glob(os.path.join(path, ext)))
    elif os.path.exists(path):
        files = [path]
    stat = [(f, os.path.getsize(f), int(os.path.getmtime(f))) for f in files]
    tok = (getattr(tokenizer, "name_or_path", type(tokenizer).__name__), len(tokenizer)) if tokenizer is not None else None
    blob = json.dumps([sorted((k, str(v)) for k, v in spec.items()), stat, tok, list(select_columns or [])])
    return hashlib.sha256(blob.encode()).hexdigest()[:24]


def _load_prepared(d: str) -> Optional["TokenDataset"]:
    if not os.path.exists(os.path.join(d, "done")):
        return None
    z = np.load(os.path.join(d, "tokens.npz"))
    off, ids, labels = z["offsets"], z["input_ids"], z["labels"]
    return TokenDataset([{"input_ids": ids[off[i]:off[i + 1]], "labels": labels[off[i]:off[i + 1]]}
                         for i in range(len(off) - 1)])


def _store_prepared(d: str, samples: List[Dict[str, np.ndarray]]) -> None:
    off = np.cumsum([0] + [len(s["input_ids"]) for s in samples]).astype(np.int64)
    cat = lambda k: np.concatenate([s[k] for s in samples]) if samples else np.zeros(0, np.int64)
    np.savez(os.path.join(d, "tokens.npz"), offsets=off, input_ids=cat("input_ids"), labels=cat("labels"))
    with open(os.path.join(d, "done"), "w") as f:
        f.write(str(len(samples)))


def _prepared_or_build(cache_dir: Optional[str], digest: str, build, wait_s: float = 3600.0) -> "TokenDataset":
    """One process tokenises and writes ``<cache_dir>/<digest>/``, every other process of the job (and
    every later run) reads it: the first to create the ``lock`` file is the builder, the others poll for
    the ``done`` marker (src/xorl/data/prepare/file_lock_loader.py)."""
    if not cache_dir:
        return TokenDataset(build())
    d = os.path.join(cache_dir, digest)
    os.makedirs(d, exist_ok=True)
    ds = _load_prepared(d)
    if ds is not None:
        return ds
    try:
        fd = os.open(os.path.join(d, "lock"), os.O_CREAT | os.O_EXCL | os.O_WRONLY)
    except FileExistsError:
        import time
        t0 = time.time()
        while time.time() - t0 < wait_s:
            ds = _load_prepared(d)
            if ds is not None:
                return ds
            time.sleep(0.2)
        raise TimeoutError(f"prepared dataset {d} did not appear within {wait_s:.0f}s (stale lock file?)")
    try:
        samples = build()
        _store_prepared(d, samples)
    except BaseException:
        os.close(fd)
        os.unlink(os.path.join(d, "lock"))        # let another process try
        raise
    os.close(fd)
    return TokenDataset(samples)


def prepare_datasets(specs: Sequence[Dict[str, Any]], tokenizer=None, vocab_size: int = 151936,
                     select_columns: Optional[Sequence[str]] = None, seed: int = 42,
                     cache_dir: Optional[str] = None) -> Dataset:
    """Builds (and concatenates) the datasets named by ``data.datasets``.  File-backed datasets are
    tokenised once and kept under ``cache_dir`` (``data.dataset_prepared_path``)."""
    built: List[Dataset] = []
    for spec in specs:
        path = spec.get("path")
        kind = spec.get("type", "tokenized")
        max_len = int(spec.get("max_seq_len", 4096))
        if path == "dummy":
            built.append(DummyDataset(max_len, int(spec.get("num_samples", 4096)), vocab_size))
            continue
        if path == "random":
            built.append(RandomTokenDataset(int(spec.get("num_samples", 4096)),
                                            int(spec.get("min_seq_len", 256)), max_len, vocab_size,
                                            int(spec.get("seed", seed))))
            continue
        built.append(_prepared_or_build(cache_dir, _spec_digest(spec, tokenizer, select_columns),
                                        lambda spec=spec, kind=kind, max_len=max_len, path=path:
                                        _tokenise_rows(_load_rows(path, spec.get("split", "train")), spec, kind, max_len, tokenizer)))
    if not built:
        raise ValueError("data.datasets is empty")
    if len(built) == 1:
        return built[0]
    return ConcatTokenDataset(built)


def _tokenise_rows(rows, spec, kind, max_len, tokenizer) -> List[Dict[str, np.ndarray]]:
    samples = []
    for r in rows:
        if kind == "tokenized":
            ids = np.asarray(r["input_ids"], dtype=np.int64)
            labels = np.asarray(r.get("labels", r["input_ids"]), dtype=np.int64)
        else:
            if tokenizer is None:
                raise ValueError(f"dataset type {kind!r} needs a tokenizer")
            text = r.get(spec.get("text_column", "text"))
            if text is None and "messages" in r:
                text = tokenizer.apply_chat_template(r["messages"], tokenize=False)
            ids = np.asarray(tokenizer(text)["input_ids"], dtype=np.int64)
            labels = ids.copy()
        ids, labels = ids[:max_len], labels[:max_len]
        if len(ids) >= 2:
            samples.append({"input_ids": ids, "labels": labels})
    return samples


class ConcatTokenDataset(Dataset):
    def __init__(self, parts: Sequence[Dataset]):
        self.parts = list(parts)
        self.cum = np.cumsum([0] + [len(p) for p in self.parts])

    def __len__(self):
        return int(self.cum[-1])

    def __getitem__(self, i):
        k = int(np.searchsorted(self.cum, i, side="right") - 1)
        return self.parts[k][i - int(self.cum[k])]

    @property
    def lengths(self):
        return np.concatenate([p.lengths for p in self.parts])


class SubsetDataset(Dataset):
    """Rows ``indices`` of another dataset (validation splits, job shards)."""

    def __init__(self, base, indices: Sequence[int]):
        self.base = base
        self.indices = np.asarray(indices, dtype=np.int64)
        self.lengths = np.asarray(base.lengths)[self.indices]

    def __len__(self) -> int:
        return len(self.indices)

    def __getitem__(self, i: int):
        return self.base[int(self.indices[i])]


def shard_dataset(ds, num_shards: int, index: int) -> "SubsetDataset":
    """Contiguous shard ``index`` of ``num_shards`` (sizes differ by at most one row, the first
    ``len % num_shards`` shards are the longer ones), for jobs that each train on a part of the data
    (``data.dataset_shard_num`` / ``dataset_shard_idx``; src/xorl/data/prepare/prepare_datasets.py:374-390)."""
    if not 0 <= index < num_shards:
        raise ValueError(f"dataset_shard_idx {index} outside 0..{num_shards - 1}")
    n = len(ds)
    base, extra = divmod(n, num_shards)
    start = index * base + min(index, extra)
    return SubsetDataset(ds, np.arange(start, start + base + (1 if index < extra else 0)))


def train_validation_split(ds, val_set_size: float, seed: int = 42):
    """(train, validation): ``val_set_size`` > 1 is a number of rows, otherwise a fraction; the rows are
    drawn with a generator seeded by ``seed`` so every rank and every run makes the same split
    (src/xorl/data/prepare/shared.py:391-415)."""
    n = len(ds)
    k = int(val_set_size) if val_set_size > 1 else int(round(n * float(val_set_size)))
    if not 0 < k < n:
        raise ValueError(f"val_set_size {val_set_size} leaves no rows for training or for validation ({n} rows)")
    perm = np.random.default_rng(seed).permutation(n)
    return SubsetDataset(ds, np.sort(perm[k:])), SubsetDataset(ds, np.sort(perm[:k]))


def prepare_train_eval(data_args, tokenizer=None, vocab_size: int = 151936, seed: int = 42):
    """(train dataset, evaluation dataset or None) as ``data`` configures them: ``datasets`` cut to this
    job's shard, then either ``test_datasets`` or a ``val_set_size`` split of the training data."""
    kw = dict(tokenizer=tokenizer, vocab_size=vocab_size, select_columns=data_args.select_columns, seed=seed,
              cache_dir=data_args.dataset_prepared_path)
    train = prepare_datasets(data_args.datasets, **kw)
    if data_args.dataset_shard_num:
        if data_args.dataset_shard_idx is None:
            raise ValueError("dataset_shard_num needs dataset_shard_idx")
        train = shard_dataset(train, int(data_args.dataset_shard_num), int(data_args.dataset_shard_idx))
    evald = None
    if data_args.test_datasets:
        evald = prepare_datasets(data_args.test_datasets, **kw)
    elif data_args.val_set_size:
        train, evald = train_validation_split(train, float(data_args.val_set_size), seed)
    return train, evald
