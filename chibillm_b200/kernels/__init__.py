"""Python side of the CUDA kernels."""
