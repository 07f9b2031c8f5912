"""SparseCore embedding path on NVIDIA B200 (sm_100a CUDA behind a C ABI)."""

__version__ = "0.1.0"
