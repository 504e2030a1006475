"""Two gloo ranks behind one dispatcher, routing replay for a MoE model: the expert choices of every datum
travel beside the broadcast command (chunk files + per-datum references), each rank reads the rows of the
datums it runs, the result equals the inline transport, and the chunks are gone afterwards."""
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xorl_b200.server.launcher import build_local_backend  # noqa: E402
from xorl_b200.server.orchestrator import RequestProcessor  # noqa: E402
from xorl_b200.server.server_arguments import ServerArguments  # noqa: E402
from xorl_b200.server.side_payloads import is_routing_ref  # noqa: E402


def main(out_dir):
    sa = ServerArguments(model_preset="tiny-qwen3-moe", output_dir=out_dir, device="cpu",
                         sample_packing_sequence_len=128, enable_mixed_precision=False)
    backend, disp = build_local_backend(sa)
    if dist.get_rank() != 0:
        loads = []
        seen = disp.runner.payloads.load
        disp.runner.payloads.load = lambda ref: (loads.append(ref["chunk"]), seen(ref))[1]
        disp.worker_loop()
        assert 1 <= len(loads) < 4, loads          # this rank read the rows of the datums it ran, not all four
        dist.destroy_process_group()
        return
    datums = [{"tokens": list(range(3 + i, 40 + 2 * i))} for i in range(4)]
    for d in datums:
        d["routed_experts"] = [[[0, 1], [2, 3]] for _ in d["tokens"]]      # [tokens, 2 MoE layers, top-2]
    plan = RequestProcessor(dp_size=2, packing_len=128).plan(datums)
    sent = []
    orig = disp.execute
    disp.execute = lambda cmd: (sent.append(cmd), orig(cmd))[1]
    store_dir = os.path.join(out_dir, "side_payloads")
    backend.payloads.min_bytes = 1 << 40                                   # inline: the lists ride in the command
    inline = backend.forward_backward("default", datums, plan, "cross_entropy", {})
    backend.abort_gradient_epoch("default")
    assert not is_routing_ref(sent[0]["args"]["datums"][0]["routed_experts"])
    backend.payloads.min_bytes = 0                                         # beside the command
    backend.payloads.chunk_bytes = 400                                     # several chunks for four datums
    beside = backend.forward_backward("default", datums, plan, "cross_entropy", {})
    refs = [d["routed_experts"] for d in sent[2]["args"]["datums"]]
    assert all(is_routing_ref(r) for r in refs) and len({r["chunk"] for r in refs}) > 1, refs
    assert abs(inline["loss"] - beside["loss"]) < 1e-6, (inline["loss"], beside["loss"])
    assert inline["metrics"]["moe/max_imbalance_ratio"] == beside["metrics"]["moe/max_imbalance_ratio"] > 1.5
    assert os.listdir(store_dir) == [], os.listdir(store_dir)             # cleaned up after the command
    # the choices really are replayed: the router's own routing gives another loss
    backend.abort_gradient_epoch("default")
    free = backend.forward_backward("default", [{"tokens": d["tokens"]} for d in datums], plan, "cross_entropy", {})
    assert abs(free["loss"] - beside["loss"]) > 1e-4
    # a malformed payload fails before anything is stored or broadcast
    bad = [dict(datums[0], routed_experts=[[0, 1]] * len(datums[0]["tokens"]))]
    try:
        backend.forward_backward("default", bad, RequestProcessor(dp_size=2, packing_len=128).plan(bad), "cross_entropy", {})
        raise SystemExit("expected a payload error")
    except RuntimeError as e:
        assert "moe_layers" in str(e), e
    assert os.listdir(store_dir) == []
    backend.shutdown()
    dist.destroy_process_group()
    print("ROUTING_PAYLOAD_OK")


if __name__ == "__main__":
    dist.init_process_group("gloo")
    main(sys.argv[1])
