"""Kernel-backed ops.  CUDA tensors run the sm_100a kernels of ``ceo_b200/csrc``;
CPU tensors run the fp32 PyTorch oracles in ``reference.py``."""
from . import reference  # noqa: F401
from .matmul import gemm, linear  # noqa: F401
from .nn import (activation, cross_entropy_rows, embedding, layernorm,  # noqa: F401
                 linear_cross_entropy, rmsnorm, softmax, swiglu)
