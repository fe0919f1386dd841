"""Calibrators: own one quantiser and feed it calibration batches.

`amax` mirrors the reference's AMaxCalibrator (segquant/calibrator/calibrator.py:91-116): inputs
accumulate a running maximum over every batch, a weight is calibrated once, and
finish_calibrate(weight) returns the quantised weight (fake-quantised floats, or the packed
low-bit tensor when the quantiser is in real_quant mode).  `gptq` (calibrator.py:118-338) is an
offline weight search outside this library's scope and raises NotImplementedError.
"""
from ..quantizers.quantizer import QuantizerRegistry


class BaseCalibrator:
    def __init__(self, data_type, quant_type, quant_args):
        if data_type not in ("weight", "input"):
            raise ValueError(f"data_type must be 'weight' or 'input', got {data_type!r}")
        self.data_type = data_type
        self.quantizer = QuantizerRegistry.create(quant_type, **(quant_args or {}))

    def quantize(self, x):
        return self.quantizer.quantize(x)

    pos_scale = property(lambda self: self.quantizer.pos_scale)
    neg_scale = property(lambda self: self.quantizer.neg_scale)
    scale = property(lambda self: self.quantizer.scale)
    dynamic = property(lambda self: self.quantizer.dynamic)

    def to(self, device):
        self.quantizer = self.quantizer.to(device)
        return self

    def __repr__(self):
        return repr(self.quantizer)


class CalibratorRegistry:
    _registry = {}

    @classmethod
    def register(cls, name):
        def deco(obj):
            cls._registry[name] = obj
            return obj
        return deco

    @classmethod
    def get(cls, name):
        return cls._registry.get(name)

    @classmethod
    def create(cls, name, **kwargs):
        factory = cls.get(name)
        if factory is None:
            raise ValueError(f"Calibrator '{name}' not found in registry.")
        return factory(**kwargs)


@CalibratorRegistry.register("amax")
class AMaxCalibrator(BaseCalibrator):
    def __init__(self, data_type, quant_type, quant_args, **kwargs):
        super().__init__(data_type, quant_type, quant_args)
        self.has_calibrated = False

    def reset(self):
        self.has_calibrated = False
        self.quantizer.reset()

    def calibrate(self, x, **kwargs):
        if self.data_type == "weight" and self.has_calibrated:
            return
        self.quantizer.calibrate(x)
        self.has_calibrated = True

    def finish_calibrate(self, weight_data=None):
        return self.quantizer.quantize(weight_data) if self.data_type == "weight" else None

    def __repr__(self):
        return f"AMaxCalibrator(quantizer={self.quantizer!r})"


def colpacked1d_to_rowpacked1d(q_colpacked_1d, out, cols):
    """Re-pack int4 weights from the column-major pairing a blocked weight search produces -- byte (c, j) of a
    (cols, out/2) array holds rows 2j (low nibble) and 2j+1 (high nibble) of column c -- into this library's storage:
    row-major [out, cols/2] bytes, element 2k of a row in the low nibble, 2k+1 in the high nibble (what the GEMM's
    TMA loads consume).  Same contract as GPTQCalibrator.colpacked1d_to_rowpacked1d of the reference
    (segquant/calibrator/calibrator.py:202-223).  Returns a 1-D uint8 tensor of out * cols / 2 bytes."""
    import torch
    if out % 2 or cols % 2:
        raise ValueError("Output and columns must be even for int4 quantization.")
    b = q_colpacked_1d.reshape(cols, out // 2)
    full = torch.empty((out, cols), dtype=torch.uint8, device=b.device)     # one nibble per entry, [row, column]
    full[0::2] = (b & 0x0F).t()
    full[1::2] = (b >> 4).t()
    return (full[:, 0::2] | (full[:, 1::2] << 4)).reshape(-1)


@CalibratorRegistry.register("gptq")
def _gptq(**kwargs):
    raise NotImplementedError("GPTQ calibration is an offline weight search that this library does not provide; "
                              "use calib type 'amax'")
