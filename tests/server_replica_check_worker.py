"""Two gloo ranks in DDP behind one dispatcher, LoRA adapters, XORL_VALIDATE_ADAPTER_REPLICAS=1: the digests of
the replicas agree after an optimizer step; once one rank's copy of an adapter shard is disturbed, the next
optimizer step reports it on every rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xorl_b200.server.launcher import build_local_backend  # noqa: E402
from xorl_b200.server.orchestrator import RequestProcessor  # noqa: E402
from xorl_b200.server.server_arguments import ServerArguments  # noqa: E402


def main(out_dir):
    os.environ["XORL_VALIDATE_ADAPTER_REPLICAS"] = "1"
    sa = ServerArguments(model_preset="tiny-qwen3", output_dir=out_dir, device="cpu", data_parallel_mode="ddp",
                         sample_packing_sequence_len=128, enable_mixed_precision=False, enable_lora=True, lora_rank=4)
    backend, disp = build_local_backend(sa)
    runner = disp.runner
    if dist.get_rank() != 0:
        # disturb this rank's copy after the second optimizer step it takes part in
        orig, n = runner.optim_step, {"c": 0}

        def wrapped(model_id, **kw):
            n["c"] += 1
            if n["c"] == 2:
                g = [g for g in runner.engine.all_groups() if not getattr(g, "frozen", False)][0]
                g.master[0] += 1.0
            return orig(model_id, **kw)

        runner.optim_step = wrapped
        disp.worker_loop()
        dist.destroy_process_group()
        return
    datums = [{"tokens": list(range(3 + i, 40 + 2 * i))} for i in range(4)]
    plan = RequestProcessor(dp_size=2, packing_len=128).plan(datums)
    backend.create_model("default2")                      # brings the adapter manager (and its checks) up
    backend.forward_backward("default", datums, plan, "cross_entropy", {})
    assert backend.optim_step("default", adam_params={"learning_rate": 1e-3})["metrics"]["step"] == 1.0
    backend.forward_backward("default", datums, plan, "cross_entropy", {})
    try:
        backend.optim_step("default", adam_params={"learning_rate": 1e-3})
        raise SystemExit("expected the replica check to fail")
    except RuntimeError as e:
        assert "replicas of" in str(e) and "differ" in str(e), e
    backend.shutdown()
    dist.destroy_process_group()
    print("REPLICA_CHECK_OK")


if __name__ == "__main__":
    dist.init_process_group("gloo")
    main(sys.argv[1])
