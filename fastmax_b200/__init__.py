"""fastmax_b200 -- Fastmax (polynomial-kernel) attention for NVIDIA B200 (sm_100a).

Drop-in for the Python interface of armingerami/fastmax: the module
``FASTMultiHeadAttention``, the autograd function behind it and the pure-PyTorch
``fastmax_function``.  The compute path is hand-written CUDA behind the C ABI in
``include/fastmax_b200.h``; build it with ``python -m fastmax_b200.build``.
"""
from .attention import (FASTMultiHeadAttention, FASTMultiHeadAttention_Function, fastmax_function,
                        rpe_matrix_creator)
from .call_site import fastmax_attention_from_qkv
from .decode import FastmaxDecodeState

__all__ = ["FASTMultiHeadAttention", "FASTMultiHeadAttention_Function", "fastmax_function",
           "rpe_matrix_creator", "fastmax_attention_from_qkv", "FastmaxDecodeState"]
__version__ = "0.1.0"
