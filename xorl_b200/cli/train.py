"""``torchrun --nproc_per_node N -m xorl_b200.cli.train cfg.yaml [--section.field value ...]``

Same contract as the reference's ``xorl.cli.train`` (src/xorl/cli/train.py:10-32): environment
defaults first, then argument parsing, then ``Trainer(args).train()``."""
import os

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def main(argv=None):
    from ..arguments import Arguments, parse_args
    from ..trainers.trainer import Trainer
    args = parse_args(Arguments, argv)
    trainer = Trainer(args)
    result = trainer.train()
    import torch.distributed as dist
    if dist.is_initialized():
        # leave no communicator (or its watchdog thread) behind at interpreter shutdown
        if torch_cuda_available():
            import torch
            torch.cuda.synchronize()
        try:
            dist.barrier()
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
    return result


def torch_cuda_available() -> bool:
    import torch
    return torch.cuda.is_available()


if __name__ == "__main__":
    import sys
    main()
    sys.stdout.flush()
    sys.stderr.flush()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # all results are on disk and the process groups are destroyed; skip interpreter teardown,
        # where communicator threads of sub-groups can abort the process
        os._exit(0)
