"""ceo_b200: a Blackwell (sm_100a) training framework for EFLA linear-attention
language models - PyTorch as the framework layer, hand-written CUDA kernels
(tcgen05 / TMEM / TMA) for the hot ops, NCCL and in-kernel peer access over
NVLink for the collectives."""

__version__ = "0.1.0"
