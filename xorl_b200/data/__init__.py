"""Data pipeline: datasets, C++ packing, collators, stateful loader."""
from .collators import PackingCollator, SequenceShardCollator, shift_sample, zigzag_indices  # noqa: F401
from .data_loader import PackedDataLoader, build_dataloader  # noqa: F401
from .datasets import DummyDataset, RandomTokenDataset, TokenDataset, prepare_datasets  # noqa: F401
from .packing import pack_bins  # noqa: F401
