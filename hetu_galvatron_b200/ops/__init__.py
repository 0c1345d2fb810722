"""Operators of the runtime. Each op runs a hand-written sm_100a kernel for bf16 CUDA tensors and a
plain PyTorch reference for CPU ranks (gloo plumbing tests) and for fp32/fp16 runs."""
from .gemm import gemm  # noqa: F401
