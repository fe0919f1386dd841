"""segquant_b200: the real-quantized segmented linear path of SegQuant on B200 (sm_100a).

Python API mirrors the reference package (segquant.layers / optimum / quantizers / calibrator /
config / utils.extension); the compute is hand-written CUDA behind a C ABI
(include/segquant_b200.h, segquant_b200/csrc).  Importing the package is cheap and does not need a
GPU; the first kernel call loads libsegquant_b200.so and raises if it is missing.
"""
from .config import Calibrate, DType, Optimum, SegPattern, default_quantize_config  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("SegmentLinear", "create_segment_linear", "DualScale"):
        from .layers import SegmentLinear as _m
        return getattr(_m, name)
    raise AttributeError(name)
