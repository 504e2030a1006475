"""``python -m xorl_b200.cli.export_nvfp4 --src <hf_dir> --dst <out_dir>``: NVFP4 (e2m1 codes, one
e4m3 scale per 16 values, one fp32 scale per tensor) export of a Hugging Face checkpoint
(src/xorl/cli/export_nvfp4.py).  Same engine as ``export_quantized`` with the format fixed."""
from __future__ import annotations

from .export_quantized import main as _main


def main(argv=None):
    return _main(argv, default_format="nvfp4")


if __name__ == "__main__":
    main()
