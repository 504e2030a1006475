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
    return trainer.train()


if __name__ == "__main__":
    main()
