"""Service runner under pipeline parallelism (2 stages on 2 gloo ranks) against the single-process
results written by the test."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build_runner(out, pp):
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    sa = ServerArguments(model_preset="tiny-qwen3", output_dir=out, device="cpu", sample_packing_sequence_len=128,
                         enable_mixed_precision=False, pipeline_parallel_size=pp)
    ta = sa.to_trainer_arguments()
    ta.model.foundation = {"tie_word_embeddings": False, "num_hidden_layers": 4}
    return ModelRunner(Trainer(ta))


def drive(r):
    from xorl_b200.server.orchestrator import RequestProcessor
    datums = [{"tokens": list(range(3 + i, 40 + 2 * i))} for i in range(3)]
    plan = RequestProcessor(dp_size=1, packing_len=64).plan(datums)         # three micro-batches
    a = r.forward_backward("default", datums, plan)
    f = r.forward("default", datums, plan)
    r.optim_step("default", adam_params={"learning_rate": 1e-2})
    b = r.forward_backward("default", datums, plan)
    return {"loss_a": a["loss"], "loss_b": b["loss"], "lp_a": a["logprobs"], "lp_f": f["logprobs"]}


def main():
    import torch.distributed as dist
    out, ref_path = sys.argv[1], sys.argv[2]
    r = build_runner(out, pp=2)
    got = drive(r)
    if dist.get_rank() == 0:
        ref = json.load(open(ref_path))
        assert abs(got["loss_a"] - ref["loss_a"]) < 1e-3 * abs(ref["loss_a"]), (got["loss_a"], ref["loss_a"])
        assert abs(got["loss_b"] - ref["loss_b"]) < 1e-3 * abs(ref["loss_b"]), (got["loss_b"], ref["loss_b"])
        assert got["loss_b"] < got["loss_a"]
        for x, y in zip(got["lp_a"], ref["lp_a"]):
            assert len(x) == len(y) and max(abs(p - q) for p, q in zip(x, y)) < 1e-3
        for x, y in zip(got["lp_f"], got["lp_a"]):                         # forward-only pass: same numbers
            assert max(abs(p - q) for p, q in zip(x, y)) < 1e-5
        print("PP_RUNNER_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
