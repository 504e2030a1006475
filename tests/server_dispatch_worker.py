"""Two gloo ranks behind one dispatcher: rank 0 issues commands, rank 1 follows; a failure raised
on one rank only is seen by both before the next command."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xorl_b200.server.launcher import build_local_backend  # noqa: E402
from xorl_b200.server.orchestrator import RequestProcessor  # noqa: E402
from xorl_b200.server.server_arguments import ServerArguments  # noqa: E402


def main(out_dir):
    sa = ServerArguments(model_preset="tiny-qwen3", output_dir=out_dir, device="cpu",
                         sample_packing_sequence_len=128, enable_mixed_precision=False)
    backend, disp = build_local_backend(sa)
    rank = dist.get_rank()
    if rank != 0:
        # make this rank's host-side checks fail on its third forward_backward only
        orig = disp.runner.preflight
        n = {"c": 0}

        def flaky(op, args):
            n["c"] += op == "forward_backward"
            if op == "forward_backward" and n["c"] == 3:
                raise RuntimeError("injected on rank 1")
            return orig(op, args)

        disp.runner.preflight = flaky
        disp.worker_loop()
        dist.destroy_process_group()
        return
    datums = [{"tokens": list(range(3 + i, 40 + 2 * i))} for i in range(4)]
    plan = RequestProcessor(dp_size=2, packing_len=128).plan(datums)
    losses = []
    for _ in range(2):
        out = backend.forward_backward("default", datums, plan, "cross_entropy", {})
        # every datum comes back with its log-probabilities, whichever data-parallel rank ran it
        assert all(len(lp) == len(d["tokens"]) for lp, d in zip(out["logprobs"], datums)), [len(x) for x in out["logprobs"]]
        losses.append(out["loss"])
        m = backend.optim_step("default", adam_params={"learning_rate": 5e-3})["metrics"]
        assert m["tokens"] == sum(len(d["tokens"]) - 1 for d in datums), m
    assert losses[1] < losses[0], losses
    try:
        backend.forward_backward("default", datums, plan, "cross_entropy", {})
        raise SystemExit("expected the injected failure to surface on rank 0")
    except RuntimeError as e:
        assert "injected on rank 1" in str(e), e
    backend.abort_gradient_epoch("default")
    out = backend.forward_backward("default", datums, plan, "cross_entropy", {})     # fleet still usable
    assert out["loss"] > 0
    backend.shutdown()
    dist.destroy_process_group()
    print("DISPATCH_OK")


if __name__ == "__main__":
    main(sys.argv[1])
