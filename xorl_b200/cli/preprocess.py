"""Tokenise / pack datasets ahead of training and cache the result.

    python -m xorl_b200.cli.preprocess cfg.yaml [--data.dataset_prepared_path out_dir]

Reads the ``data`` section of a training config, builds the datasets exactly as the trainer would
(tokenisation included), computes the first-fit-decreasing packing plan with the native packer and
writes one ``.arrow`` file of token ids / labels plus ``packing.json`` (bins of sample indices) and
``meta.json``.  The trainer can then point a ``tokenized`` dataset at the directory
(src/xorl/cli/preprocess.py, src/xorl/data/prepare/)."""
from __future__ import annotations

import json
import os
import sys
from typing import List, Optional

import numpy as np


def preprocess(args, out_dir: Optional[str] = None) -> str:
    import pyarrow as pa

    from ..data import packing
    from ..data.datasets import prepare_datasets
    tok = None
    if args.model.tokenizer_path or args.model.model_path:
        try:
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(args.model.tokenizer_path or args.model.model_path)
        except Exception:  # noqa: BLE001
            tok = None
    vocab = 151936
    if args.model.config_path or args.model.model_path:
        from ..models import build_model_config
        vocab = build_model_config(args.model).vocab_size
    ds = prepare_datasets(args.data.datasets, tokenizer=tok, vocab_size=vocab,
                          select_columns=args.data.select_columns, seed=args.train.seed)
    out_dir = out_dir or args.data.dataset_prepared_path
    os.makedirs(out_dir, exist_ok=True)
    ids, labels = [], []
    for i in range(len(ds)):
        s = ds[i]
        ids.append(np.asarray(s["input_ids"], dtype=np.int64))
        labels.append(np.asarray(s["labels"], dtype=np.int64))
    table = pa.table({"input_ids": pa.array([x.tolist() for x in ids], type=pa.list_(pa.int64())),
                      "labels": pa.array([x.tolist() for x in labels], type=pa.list_(pa.int64()))})
    with pa.OSFile(os.path.join(out_dir, "data.arrow"), "wb") as sink:
        with pa.ipc.new_file(sink, table.schema) as w:
            w.write_table(table)
    lengths = np.asarray([len(x) for x in ids], dtype=np.int64)
    cap = int(args.data.sample_packing_sequence_len or lengths.max())
    bins = packing.pack_bins(lengths, cap, method="ffd")
    with open(os.path.join(out_dir, "packing.json"), "w") as f:
        json.dump({"capacity": cap, "bins": [list(map(int, b)) for b in bins]}, f)
    meta = {"num_samples": int(len(ids)), "total_tokens": int(lengths.sum()), "num_bins": len(bins),
            "fill": float(lengths.sum() / max(1, len(bins) * cap)), "vocab_size": int(vocab)}
    with open(os.path.join(out_dir, "meta.json"), "w") as f:
        json.dump(meta, f, indent=2)
    return out_dir


def main(argv: Optional[List[str]] = None):
    from ..arguments import parse_args
    args = parse_args(argv=list(sys.argv[1:] if argv is None else argv))
    out = preprocess(args)
    print(out)
    return out


if __name__ == "__main__":
    main()
