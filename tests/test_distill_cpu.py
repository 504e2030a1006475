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
