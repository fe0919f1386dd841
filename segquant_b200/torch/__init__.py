"""Model-level entry point: quantize() replaces the nn.Linear layers of a model by calibrated SegmentLinear layers."""
from .quantization import quantize  # noqa: F401
