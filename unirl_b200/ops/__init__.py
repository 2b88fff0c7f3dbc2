"""Operator layer: every hot op has a fused sm_100a kernel (``unirl_b200._C``) and a PyTorch fp32 reference.

Dispatch rule: CUDA tensors go to the native kernel — and raise if the extension is missing, a GPU
run must never silently fall back to eager PyTorch — while CPU tensors use the reference expression
(which is also the oracle the kernel tests compare against).
"""
from unirl_b200.ops._ext import ext, have_ext, require_ext  # noqa: F401
