"""Python wrappers of the CUDA kernels."""
