"""ctypes wrappers of the compiled kernels (ops, attention, gemm)."""
