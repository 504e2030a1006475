"""Trainer end to end on CPU: dense single process (with checkpoint save + resume) and a tiny MoE
model with expert parallelism + ZeRO sharding on two gloo ranks."""
import json
import os
import sys

import pytest
import torch
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _cfg(tmp, model, **train):
    cfg = {
        "model": {"config_path": model},
        "data": {"datasets": [{"path": "dummy", "type": "tokenized", "max_seq_len": 200, "num_samples": 64}],
                 "sample_packing_sequence_len": 512, "pad_to_multiple_of": 64},
        "train": {"output_dir": str(tmp / "out"), "lr": 1e-3, "max_steps": 6, "use_wandb": False,
                  "device": "cpu", "save_hf_weights": False, "save_epochs": 0, **train},
    }
    p = tmp / "cfg.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return str(p)


def test_dense_train_save_resume(tmp_path):
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    cfg = _cfg(tmp_path, "tiny-qwen3", save_steps=3)
    r1 = main([cfg])
    assert r1["loss_history"][-1] < r1["loss_history"][0]
    assert os.path.exists(tmp_path / "out" / "checkpoints" / "global_step_6" / ".metadata")
    # resume from step 3 and replay steps 4..6: same losses as the uninterrupted run
    reset_parallel_state()
    r2 = main([cfg, "--train.load_checkpoint_path", str(tmp_path / "out" / "checkpoints" / "global_step_3")])
    assert r2["global_step"] == 6
    for a, b in zip(r1["loss_history"][3:], r2["loss_history"]):
        assert abs(a - b) < 1e-4, (r1["loss_history"], r2["loss_history"])
    for f in ("xorl_cli.yaml", "startup_metrics.json", "training_metrics.json"):
        assert os.path.exists(tmp_path / "out" / f)


@pytest.mark.distributed
def test_moe_ep2_fsdp_trains(tmp_path):
    from dist_utils import run_distributed
    cfg = _cfg(tmp_path, "tiny-qwen3-moe", expert_parallel_size=2, softmax_auxiliary_loss=True,
               auxiliary_loss_multiplier=1e-4)   # z-loss on the logits; the router loss comes from the model config
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg)
    with open(tmp_path / "out" / "training_metrics.json") as f:
        hist = json.load(f)["loss_history"]
    assert len(hist) == 6 and hist[-1] < hist[0]


def test_softmax_auxiliary_loss_is_the_z_loss_on_the_logits(tmp_path):
    """``train.softmax_auxiliary_loss`` adds ``auxiliary_loss_multiplier * logsumexp(logits)^2`` per
    supervised token to the lm-head loss (src/xorl/trainers/trainer.py:481-487); it is not the
    routers' load-balancing loss, whose weight is the model's ``router_aux_loss_coef``."""
    from xorl_b200.arguments import build_args
    from xorl_b200.models.config import preset
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    args = build_args({"model": {"config_path": "tiny-qwen3"},
                       "data": {"datasets": [{"path": "dummy", "type": "tokenized", "max_seq_len": 64,
                                              "num_samples": 8}], "sample_packing_sequence_len": 128},
                       "train": {"output_dir": str(tmp_path / "o"), "device": "cpu", "use_wandb": False,
                                 "softmax_auxiliary_loss": True, "auxiliary_loss_multiplier": 0.5,
                                 "save_hf_weights": False, "save_epochs": 0, "max_steps": 1}})
    tr = Trainer(args, model_config=preset("tiny-qwen3"))
    assert tr.model.z_loss_coef == 0.5
    eng = tr.engine
    ids = torch.randint(0, 1024, (1, 65))
    x, y = ids[:, :-1], ids[:, 1:]
    got = float(eng.forward_backward(x, y, grad_scale=1.0 / 64))
    hidden = eng.forward_only(x)
    w = dict(eng.iter_full_tensors("master"))["lm_head.weight"] if not tr.model_config.tie_word_embeddings \
        else dict(eng.iter_full_tensors("master"))["embed_tokens.weight"]
    logits = hidden.reshape(-1, hidden.shape[-1]).float() @ w.float().t()
    ce = torch.nn.functional.cross_entropy(logits, y.reshape(-1), reduction="sum")
    z = 0.5 * torch.logsumexp(logits, -1).pow(2).sum()
    assert abs(got - float(ce + z) / 64) < 1e-3 * abs(got), (got, float(ce + z) / 64)


def test_prepared_dataset_cache_is_built_once_and_keyed_by_content(tmp_path):
    import json
    import numpy as np
    from xorl_b200.data import datasets as D
    src = tmp_path / "d.jsonl"
    src.write_text("\n".join(json.dumps({"input_ids": list(range(3 + i, 20 + i))}) for i in range(5)))
    spec = [{"path": str(src), "type": "tokenized", "max_seq_len": 16}]
    cache = str(tmp_path / "prepared")
    calls = {"n": 0}
    real = D._load_rows

    def counting(path, *a):
        calls["n"] += 1
        return real(path, *a)
    D._load_rows = counting
    try:
        a = D.prepare_datasets(spec, cache_dir=cache)
        b = D.prepare_datasets(spec, cache_dir=cache)                 # second build: read from the cache
        assert calls["n"] == 1 and len(a) == len(b) == 5
        assert all(np.array_equal(a[i]["input_ids"], b[i]["input_ids"]) and len(b[i]["input_ids"]) == 16 for i in range(5))
        # an edited source file is a different key
        src.write_text("\n".join(json.dumps({"input_ids": list(range(50, 60))}) for _ in range(2)))
        import os
        os.utime(src, (1, 1))
        c = D.prepare_datasets(spec, cache_dir=cache)
        assert calls["n"] == 2 and len(c) == 2
        # a builder that fails releases the lock
        spec2 = [{"path": str(tmp_path / "missing.jsonl"), "type": "tokenized"}]
        for _ in range(2):
            try:
                D.prepare_datasets(spec2, cache_dir=cache)
            except (FileNotFoundError, ValueError, OSError):
                pass
            else:
                raise AssertionError("a missing file must raise")
    finally:
        D._load_rows = real


def test_dataset_shards_and_validation_split():
    import numpy as np
    from xorl_b200.data import datasets as D
    base = D.RandomTokenDataset(23, 8, 40, 1000, 1)
    shards = [D.shard_dataset(base, 4, i) for i in range(4)]
    assert [len(s) for s in shards] == [6, 6, 6, 5]
    assert np.concatenate([s.indices for s in shards]).tolist() == list(range(23))
    assert np.array_equal(shards[1][0]["input_ids"], base[6]["input_ids"]) and shards[3].lengths.tolist() == np.asarray(base.lengths)[18:].tolist()
    with pytest.raises(ValueError):
        D.shard_dataset(base, 4, 4)
    tr, va = D.train_validation_split(base, 0.25, seed=3)
    tr2, va2 = D.train_validation_split(base, 0.25, seed=3)
    assert len(va) == 6 and len(tr) == 17 and va.indices.tolist() == va2.indices.tolist()
    assert sorted(tr.indices.tolist() + va.indices.tolist()) == list(range(23))
    assert len(D.train_validation_split(base, 5, seed=0)[1]) == 5
    with pytest.raises(ValueError):
        D.train_validation_split(base, 23)


def test_validation_split_is_evaluated_at_saves_and_at_the_end(tmp_path):
    """``data.val_set_size``: the held-out rows never train, their loss is measured at every checkpoint and
    at the end, and it falls while the model learns the (shared) structure of the dummy data."""
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    cfg = yaml.safe_load(open(_cfg(tmp_path, "tiny-qwen3", save_steps=3, max_steps=6)))
    cfg["data"]["val_set_size"] = 0.125
    cfg["data"]["eval_sample_packing"] = False
    p = tmp_path / "eval.yaml"
    p.write_text(yaml.safe_dump(cfg))
    r = main([str(p)])
    ev = r["eval_history"]
    assert [e["step"] for e in ev] == [3, 6] and ev[0]["eval_tokens"] == ev[1]["eval_tokens"] > 0
    assert ev[1]["eval_loss"] < ev[0]["eval_loss"] and abs(ev[1]["eval_perplexity"] - 2.718281828 ** ev[1]["eval_loss"]) < 1e-3 * ev[1]["eval_perplexity"]
    with open(tmp_path / "out" / "training_metrics.json") as f:
        assert len(json.load(f)["eval_history"]) == 2
    reset_parallel_state()


@pytest.mark.distributed
def test_test_datasets_are_evaluated_on_two_ranks(tmp_path):
    """``data.test_datasets`` on two data-parallel ranks gives the loss a single process measures on the same
    rows (the ragged tail aside: the row count here divides by the ranks)."""
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    cfg = yaml.safe_load(open(_cfg(tmp_path, "tiny-qwen3", max_steps=1, lr=1e-10)))
    cfg["data"]["test_datasets"] = [{"path": "random", "type": "tokenized", "max_seq_len": 200, "min_seq_len": 150,
                                     "num_samples": 8}]
    cfg["data"]["eval_sample_packing"] = False
    evals = {}
    for name, n in (("one", 1), ("two", 2)):
        cfg["train"]["output_dir"] = str(tmp_path / name)
        p = tmp_path / f"{name}.yaml"
        p.write_text(yaml.safe_dump(cfg))
        if n == 1:
            reset_parallel_state()
            main([str(p)])
            reset_parallel_state()
        else:
            run_distributed("-m", 2, "xorl_b200.cli.train", str(p))
        with open(tmp_path / name / "training_metrics.json") as f:
            evals[name] = json.load(f)["eval_history"][-1]
    assert evals["one"]["eval_tokens"] == evals["two"]["eval_tokens"]
    assert abs(evals["one"]["eval_loss"] - evals["two"]["eval_loss"]) < 1e-4, evals


@pytest.mark.distributed
def test_hybrid_shared_expert_lora_under_expert_parallelism(tmp_path):
    """Two ranks with the experts split over them against the same two ranks with all experts everywhere: the
    factors shared by all experts are reduced over both ranks, the per-expert ones over their owners, and
    the loss curves agree."""
    from dist_utils import run_distributed
    curves = {}
    for name, ep in (("ep1", 1), ("ep2", 2)):
        cfg = yaml.safe_load(open(_cfg(tmp_path, "tiny-qwen3-moe", expert_parallel_size=ep, max_steps=4, lr=5e-3)))
        cfg["train"]["output_dir"] = str(tmp_path / name)
        cfg["lora"] = {"enable_lora": True, "lora_rank": 4, "lora_alpha": 8, "moe_hybrid_shared_lora": True,
                       "lora_b_init_std": 0.02, "lora_target_modules": ["q_proj", "gate_proj", "up_proj", "down_proj"]}
        p = tmp_path / f"{name}.yaml"
        p.write_text(yaml.safe_dump(cfg))
        run_distributed("-m", 2, "xorl_b200.cli.train", str(p))
        with open(tmp_path / name / "training_metrics.json") as f:
            curves[name] = json.load(f)["loss_history"]
    assert curves["ep1"][-1] < curves["ep1"][0]
    for a, b in zip(curves["ep1"], curves["ep2"]):
        assert abs(a - b) < 3e-4, curves


def test_evaluation_on_an_unsupported_layout_is_refused_at_start_up(tmp_path, monkeypatch):
    from xorl_b200.arguments import build_args
    from xorl_b200.models.config import preset
    from xorl_b200.parallel import state as pstate
    from xorl_b200.trainers.trainer import Trainer
    pstate.reset_parallel_state()
    args = build_args({"model": {"config_path": "tiny-qwen3"},
                       "data": {"datasets": [{"path": "dummy", "type": "tokenized", "max_seq_len": 64, "num_samples": 16}],
                                "sample_packing_sequence_len": 128, "val_set_size": 0.25},
                       "train": {"output_dir": str(tmp_path / "o"), "device": "cpu", "use_wandb": False,
                                 "save_hf_weights": False, "save_epochs": 0, "max_steps": 1}})
    real = pstate.init_parallel_state

    def fake(**kw):
        st = real(**kw)
        st.sizes["tp"] = 2                      # as if the body were tensor parallel
        return st
    monkeypatch.setattr("xorl_b200.trainers.trainer.init_parallel_state", fake)
    with pytest.raises(NotImplementedError, match="evaluation pass"):
        Trainer(args, model_config=preset("tiny-qwen3"))
    pstate.reset_parallel_state()
