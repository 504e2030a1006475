"""Adapters applied to a freshly built model: LoRA / QLoRA, block-fp8 training, QARL fake-quant."""
from __future__ import annotations


def apply_adapters(model, cfg, args) -> None:
    lora = getattr(args, "lora", None)
    train = getattr(args, "train", None)
    if train is not None and getattr(train, "enable_fp8_training", False):
        from .fp8 import inject_fp8_training
        inject_fp8_training(model, train)
    if train is not None and getattr(train, "enable_qarl", False):
        from .qarl import inject_fake_quant
        inject_fake_quant(model, train)
    if lora is not None and lora.enable_lora:
        if lora.enable_qlora:
            from .qlora import inject_qlora
            inject_qlora(model, lora)
        else:
            from .lora import inject_lora
            inject_lora(model, lora)
