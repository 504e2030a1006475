"""xorl_b200: a Blackwell (sm_100a) native LLM training framework.

PyTorch provides tensors, autograd plumbing and process groups; every hot operator is a
hand-written CUDA kernel in ``xorl_b200/csrc`` reached through ``xorl_b200.ops``.
"""

__version__ = "0.1.0"
