"""Test infrastructure: recipe that builds the reference project's own CUDA kernels as a checker (see build_ref.py)."""
