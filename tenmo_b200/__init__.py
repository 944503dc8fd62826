"""tenmo_b200: the B200 (sm_100a) implementation of tenmo's dense fp32 training path.

``libtenmo_cuda.so`` (hand-written CUDA behind the C ABI in ``include/tenmo_cuda.h``) does the work;
this package is the host side above it, mirroring the reference's operator interface for the path.
"""
from .lib import (ACT_NONE, ACT_RELU, ACT_SIGMOID, ALGO_AUTO, ALGO_SIMT_FP32, ALGO_TC_3XTF32, Mat, TenmoCuda,
                  TenmoError, make_mat)

__all__ = ["TenmoCuda", "TenmoError", "Mat", "make_mat", "ALGO_AUTO", "ALGO_SIMT_FP32", "ALGO_TC_3XTF32", "ACT_NONE",
           "ACT_RELU", "ACT_SIGMOID"]
