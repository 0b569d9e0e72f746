"""CUDA sources of the kernels and the helper that compiles and loads them (build.py)."""
