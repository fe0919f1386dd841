from .quantizer import BaseQuantizer, FloatQuantizer, IntQuantizer, QuantizerRegistry  # noqa: F401
