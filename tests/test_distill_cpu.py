"""Teacher log-prob store, the on-policy distillation loop on a tiny model, numerical programme."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_store_roundtrip_and_persistence(tmp_path):
    from xorl_b200.distillation import TeacherLogprobStore
    st = TeacherLogprobStore(str(tmp_path), max_in_memory=2, shard_entries=2)
    seqs = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    for s in seqs:
        st.put(s, [-0.1 * t for t in s])
    st.flush()
    assert len(st) == 3 and [1, 2, 3] in st and [9, 9] not in st
    assert torch.allclose(st.get([1, 2, 3]), torch.tensor([-0.1, -0.2, -0.3]))      # evicted from memory, read from disk
    st2 = TeacherLogprobStore(str(tmp_path))
    assert torch.allclose(st2.get([6, 7, 8, 9]), torch.tensor([-0.6, -0.7, -0.8, -0.9])) and st2.get([0]) is None


def test_on_policy_distillation_moves_student_towards_teacher(tmp_path):
    from xorl_b200.distillation import TeacherLogprobStore, attach_teacher_logprobs, score_with_teacher
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer

    def runner(seed, name):
        reset_parallel_state()
        sa = ServerArguments(model_preset="tiny-qwen3", output_dir=str(tmp_path / name), device="cpu", seed=seed,
                             sample_packing_sequence_len=128, enable_mixed_precision=False)
        return ModelRunner(Trainer(sa.to_trainer_arguments()))

    teacher = runner(7, "t")
    data = [{"tokens": list(range(3 + i, 40 + i))} for i in range(3)]
    store = TeacherLogprobStore(str(tmp_path / "store"))
    assert score_with_teacher(teacher, data, store) == 3 and score_with_teacher(teacher, data, store) == 0
    student = runner(1, "s")
    batch = attach_teacher_logprobs(data, store)

    def gap():
        lp = student.forward("default", data, None)["logprobs"]
        return sum(abs(a - b) for s, d in zip(lp, batch) for a, b in zip(s[:-1], d["teacher_logprobs"][:-1]))

    g0 = gap()
    for _ in range(8):
        student.forward_backward("default", batch, None, loss_fn="opd_loss")
        student.optim_step("default", adam_params={"learning_rate": 3e-3})
    assert gap() < g0
    reset_parallel_state()


def test_numerical_program():
    from xorl_b200.models.config import preset
    from xorl_b200.models.numerics import describe, resolve_numerical_program

    class T:
        fsdp_reduce_dtype = "bf16"
        deterministic = True

    p = resolve_numerical_program(preset("tiny-deepseek-v3"), None, T())
    assert p.router_fp32 and p.reduce_dtype == "bf16" and p.batch_invariant
    rep = describe(p)
    assert "atomics" in rep["attention_backward"] and "note" in rep


def test_trainer_distillation_adds_the_teacher_kl(tmp_path):
    """``distill.enable_distillation``: the step loss is CE + weight * KL(teacher || student) over the
    supervised tokens (weight 500 here: freshly initialised models are close to uniform, so the KL is small next to the CE), the teacher being a frozen second model; training lowers the KL."""
    from xorl_b200.arguments import build_args
    from xorl_b200.models.config import preset
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    args = build_args({"model": {"config_path": "tiny-qwen3"},
                       "data": {"datasets": [{"path": "dummy", "type": "tokenized", "max_seq_len": 64,
                                              "num_samples": 8}], "sample_packing_sequence_len": 128},
                       "train": {"output_dir": str(tmp_path / "o"), "device": "cpu", "use_wandb": False, "lr": 2e-3,
                                 "save_hf_weights": False, "save_epochs": 0, "max_steps": 1},
                       "distill": {"enable_distillation": True, "teacher_model_path": "tiny-qwen3",
                                   "distillation_loss_type": "forward_kl", "distillation_loss_weight": 500.0}})
    tr = Trainer(args, model_config=preset("tiny-qwen3"))
    assert tr.teacher_engine is not None
    assert all(getattr(g, "frozen", False) for g in tr.teacher_engine.all_groups())
    ids = torch.randint(0, 1024, (1, 65))
    mb = {"input_ids": ids[:, :-1], "labels": ids[:, 1:]}
    # manual value of the first step's loss
    eng, te = tr.engine, tr.teacher_engine
    hs = eng.forward_only(mb["input_ids"]).reshape(-1, 256).float()
    ht = te.forward_only(mb["input_ids"]).reshape(-1, 256).float()
    ws = dict(eng.iter_full_tensors("master"))
    wt = dict(te.iter_full_tensors("master"))
    head_s = ws.get("lm_head.weight", ws["embed_tokens.weight"]).float()
    head_t = wt.get("lm_head.weight", wt["embed_tokens.weight"]).float()
    lps, lpt = torch.log_softmax(hs @ head_s.t(), -1), torch.log_softmax(ht @ head_t.t(), -1)
    ce = torch.nn.functional.nll_loss(lps, mb["labels"].reshape(-1), reduction="sum")
    kl = (lpt.exp() * (lpt - lps)).sum()
    want = float(ce + 500.0 * kl) / 64
    first = float(tr.train_step([mb])["loss"])
    assert abs(first - want) < 1e-3 * abs(want), (first, want)
    assert float(kl) > 0.5                                            # different seeds: the models disagree
    for _ in range(8):
        last = float(tr.train_step([mb])["loss"])
    assert last < first - 0.2, (first, last)
    with torch.no_grad():
        hs2 = eng.forward_only(mb["input_ids"]).reshape(-1, 256).float()
        head_s2 = dict(eng.iter_full_tensors("master"))
        head_s2 = head_s2.get("lm_head.weight", head_s2["embed_tokens.weight"]).float()
        lps2 = torch.log_softmax(hs2 @ head_s2.t(), -1)
    assert float((lpt.exp() * (lpt - lps2)).sum()) < float(kl)


def test_distillation_needs_a_teacher():
    import pytest
    from xorl_b200.arguments import build_args
    from xorl_b200.models.config import preset
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    args = build_args({"model": {"config_path": "tiny-qwen3"}, "train": {"device": "cpu", "use_wandb": False},
                       "data": {"datasets": [{"path": "dummy", "type": "tokenized", "max_seq_len": 64, "num_samples": 8}]},
                       "distill": {"enable_distillation": True}})
    with pytest.raises(ValueError, match="teacher_model_path"):
        Trainer(args, model_config=preset("tiny-qwen3"))
