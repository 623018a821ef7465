"""B200-native SDDMM engine: P_ij = S_ij * (A_i . B_j) on the pattern of S.

The product is the CUDA library behind include/sddmm_b200.h and the C++
competitor in dphpc_b200/src; this package holds their sources, the in-tree
build and thin ctypes bindings used by the tests and bench.py.
"""
from .capi import (  # noqa: F401
    BF16, FP32, FP32_TC, TF32, Dataset, Engine, Pipeline, SddmmError, device_count, load_dataset_lib, load_engine_lib,
)
