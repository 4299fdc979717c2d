"""Hand-written CUDA kernels for sm_100a and their Python binding."""
