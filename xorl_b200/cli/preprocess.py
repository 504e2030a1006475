"""Tokenise / pack datasets ahead of training and cache the result.

    python -m xorl_b200.cli.preprocess cfg.yaml [--data.dataset_prepared_path out_dir]

Reads the ``data`` section of a training config, builds the datasets exactly as the trainer would
(tokenisation included), computes the first-fit-decreasing packing plan with the native packer and
writes the token ids / labels as ``data.arrow`` (or ``data-XXXXX-of-YYYYY.arrow`` with
``data.num_dataset_shards_to_save``), the evaluation rows (``data.test_datasets`` or the ``data.val_set_size``
split) as ``eval.arrow``, plus ``packing.json`` (bins of sample indices) and ``meta.json``.  The trainer can
then point a ``tokenized`` dataset at the directory (``split: eval`` for the evaluation rows)
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
    from ..data.datasets import prepare_train_eval
    out_dir = out_dir or args.data.dataset_prepared_path
    cache = args.data.dataset_prepared_path
    args.data.dataset_prepared_path = None          # the output below is the prepared form; no second cache inside it
    try:
        ds, eval_ds = prepare_train_eval(args.data, tokenizer=tok, vocab_size=vocab, seed=args.train.seed)
    finally:
        args.data.dataset_prepared_path = cache
    os.makedirs(out_dir, exist_ok=True)

    def rows_of(d):
        ids, labels = [], []
        for i in range(len(d)):
            s = d[i]
            ids.append(np.asarray(s["input_ids"], dtype=np.int64))
            labels.append(np.asarray(s["labels"], dtype=np.int64))
        return ids, labels

    def write(path, ids, labels):
        table = pa.table({"input_ids": pa.array([x.tolist() for x in ids], type=pa.list_(pa.int64())),
                          "labels": pa.array([x.tolist() for x in labels], type=pa.list_(pa.int64()))})
        with pa.OSFile(path, "wb") as sink:
            with pa.ipc.new_file(sink, table.schema) as w:
                w.write_table(table)

    ids, labels = rows_of(ds)
    n_files = max(1, int(args.data.num_dataset_shards_to_save or 1))
    if n_files == 1:
        write(os.path.join(out_dir, "data.arrow"), ids, labels)
    else:
        # contiguous pieces, so reading the numbered files in order gives the rows in order
        bounds = np.linspace(0, len(ids), n_files + 1).astype(int)
        for k in range(n_files):
            write(os.path.join(out_dir, f"data-{k:05d}-of-{n_files:05d}.arrow"),
                  ids[bounds[k]:bounds[k + 1]], labels[bounds[k]:bounds[k + 1]])
    lengths = np.asarray([len(x) for x in ids], dtype=np.int64)
    cap = int(args.data.sample_packing_sequence_len or lengths.max())
    bins = packing.pack_bins(lengths, cap, method="ffd")
    with open(os.path.join(out_dir, "packing.json"), "w") as f:
        json.dump({"capacity": cap, "bins": [list(map(int, b)) for b in bins]}, f)
    meta = {"prepared": True, "num_samples": int(len(ids)), "total_tokens": int(lengths.sum()), "num_bins": len(bins),
            "fill": float(lengths.sum() / max(1, len(bins) * cap)), "vocab_size": int(vocab), "files": n_files}
    if eval_ds is not None:
        eids, elabels = rows_of(eval_ds)
        write(os.path.join(out_dir, "eval.arrow"), eids, elabels)
        meta["num_eval_samples"] = len(eids)
        meta["eval_tokens"] = int(sum(len(x) for x in eids))
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
