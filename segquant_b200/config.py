"""Configuration enums and the default quantisation recipe.

Same names, values and dictionary schema as the reference's segquant/config.py:18-97, so YAML / dict
recipes written for it are accepted unchanged.  One key is new: `weight_quant.group_size`
(int, default None) selects K-group-wise weight scales.
"""
from enum import Enum


class DType(Enum):
    INT4 = "int4"
    INT6 = "int6"
    INT8 = "int8"
    INT16 = "int16"
    FP8E5M2 = "fpe5m2"
    FP8E4M3 = "fpe4m3"
    FP16 = "fp16"
    BF16 = "bf16"


class Optimum(Enum):
    DEFAULT = "default"
    SMOOTH = "smooth"
    SVD = "svd"


class Calibrate(Enum):
    AMAX = "amax"
    GPTQ = "gptq"


class SegPattern(Enum):
    LINEAR2CHUNK = "linear_to_chunk"
    LINEAR2SPLIT = "linear_to_split"
    CONCAT2LINEAR = "concat_to_linear"
    STACK2LINEAR = "stack_to_linear"
    RESHAPE2LINEAR = "reshape_to_linear"
    ACTIVATION2LINEAR = "activation_to_linear"

    @classmethod
    def seg(cls):
        """Patterns that split a linear layer into segments."""
        return [p for p in cls if p is not cls.ACTIVATION2LINEAR]

    @classmethod
    def all(cls):
        return list(cls)


default_quantize_config = {
    "default": {
        "enable": True,
        "seglinear": True,
        "search_patterns": SegPattern.all(),
        "real_quant": False,
        "opt": {"type": Optimum.SMOOTH, "alpha": 0.5},
        "calib": {"type": Calibrate.AMAX},
        "input_quant": {"type": DType.INT8, "axis": None},
        "weight_quant": {"type": DType.INT8, "axis": None},
    },
}
