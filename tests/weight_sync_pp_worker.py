"""Two pipeline stages on two gloo ranks: the weight-sync stream on rank 0 carries the whole model."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist
    from xorl_b200.arguments import build_args
    from xorl_b200.server.weight_sync import FileTransport, WeightSyncHandler, iter_sync_tensors
    from xorl_b200.trainers.trainer import Trainer
    out = sys.argv[1]
    args = build_args({
        "model": {"config_path": "tiny-qwen3", "foundation": {"num_hidden_layers": 4, "tie_word_embeddings": False}},
        "data": {"datasets": [{"path": "random", "type": "tokenized", "max_seq_len": 64, "min_seq_len": 16, "num_samples": 32}],
                 "sample_packing_sequence_len": 128},
        "train": {"output_dir": out, "device": "cpu", "use_wandb": False, "enable_mixed_precision": False,
                  "pipeline_parallel_size": 2, "pipeline_parallel_schedule": "1F1B", "max_steps": 1,
                  "save_hf_weights": False, "save_epochs": 0}})
    tr = Trainer(args)
    rank = dist.get_rank()
    got = {n: t.clone() for n, t in iter_sync_tensors(tr.engine, tr.model_config, torch.float32)}
    # what each stage holds locally, by Hugging Face name
    from xorl_b200.checkpoint.handlers import get_checkpoint_handler
    h = get_checkpoint_handler(tr.model_config)
    local = {}
    for fqn, full in tr.engine.iter_full_tensors("master"):
        for name, part in h.to_hf(fqn, full.float()):
            local[name] = part.clone()
    everyone = [None, None]
    dist.all_gather_object(everyone, {k: v.sum().item() for k, v in local.items()})
    if rank == 0:
        want = {**everyone[0], **everyone[1]}
        assert set(got) == set(want), sorted(set(want) ^ set(got))[:6]
        assert all(abs(got[k].sum().item() - want[k]) < 1e-4 for k in want)
        assert any(k.startswith("model.layers.3.") for k in got) and "lm_head.weight" in got
        # the stream is in model order: all of stage 0 first
        order = list(got)
        assert order.index("model.layers.0.input_layernorm.weight") < order.index("model.layers.3.input_layernorm.weight")
        print("PP_SYNC_OK " + json.dumps(len(got)))
    else:
        assert got == {}
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
