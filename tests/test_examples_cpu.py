"""Every shipped example configuration parses against the argument schema."""
import glob
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "local", "*.yaml"))))
def test_local_examples_parse(path, monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "8")                      # the examples are written for one 8-GPU box
    from xorl_b200.arguments import parse_args
    from xorl_b200.models import build_model_config
    args = parse_args(argv=[path])
    cfg = build_model_config(args.model)
    assert cfg.num_hidden_layers > 0 and args.train.output_dir.startswith("outputs/")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "server", "*.yaml"))))
def test_server_examples_parse(path):
    from xorl_b200.server.server_arguments import ServerArguments
    sa = ServerArguments.from_yaml(path)
    targs = sa.to_trainer_arguments()
    assert targs.lora.enable_lora == sa.enable_lora and targs.train.output_dir == sa.output_dir
