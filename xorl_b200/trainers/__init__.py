"""Trainer and the training utilities shared with the server runner."""
from .trainer import Trainer  # noqa: F401
