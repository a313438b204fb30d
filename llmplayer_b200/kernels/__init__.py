"""Compiled CUDA kernels: building them (build) and calling them (ops)."""
