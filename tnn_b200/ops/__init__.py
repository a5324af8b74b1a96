"""Operators: hand-written sm_100a kernels on CUDA tensors, torch math on CPU tensors."""
