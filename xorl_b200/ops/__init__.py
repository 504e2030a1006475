"""Operators.  Each module exposes a functional API that dispatches to the sm_100a kernel for CUDA
tensors and to a plain PyTorch implementation for CPU tensors (used by the gloo test lane)."""
