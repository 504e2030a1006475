"""Checkpointing: PyTorch DCP directories (reshardable) and Hugging Face safetensors."""
from .checkpointer import (DistributedCheckpointer, build_checkpointer,  # noqa: F401
                           resolve_checkpoint_path)
