"""Extension loaders with the reference's names and return conventions.

The reference JIT-builds five pybind11 modules and returns them (segquant/utils/extension.py:66-213).
Here every loader returns a thin Python object over the one ahead-of-time library
libsegquant_b200.so; the objects expose the same functions:

    real_quantized_quantize_weights(weights, outputs, scale_w)          seg_utils.h:82-120
    {P}_real_quantized_gemm_scaled(inputs, weights, scale_x, scale_w)    seg_utils.h:122-141
    {P}_real_quantized_gemm_dual_scaled(inputs, weights, pos, neg, sw)   seg_utils.h:143-160
    create_quantized_weights(x)                                          extension.py:110-113 ...
    fake_e4m3fy(inputs)                                                  quantizer_fp8.cpp:41-43

P in {Wint8Aint8, Wfpe4m3Afpe4m3, Wint4Aint8}.  The prefixes this build has no kernel for
(Wint4Aint4, Wint8Afp16, Wfp16Afp16) are absent, and asking SegmentLinear for them with
real_quant=True raises instead of silently falling back to fake quantisation.
"""
import torch

from .. import _lib as L
from .. import ops

supported_type = ["Wint8Aint8", "Wint4Aint8", "Wfpe4m3Afpe4m3"]

_STORAGE = {L.SQ_Q_INT8: torch.int8, L.SQ_Q_E4M3: torch.uint8, L.SQ_Q_INT4: torch.uint8}


class _RealQuantModule:
    """Stands in for one pybind11 module of the reference."""

    def __init__(self, name, weight_kind, prefixes):
        self.__name__ = name
        self._weight_kind = weight_kind
        for p in prefixes:
            setattr(self, f"{p}_real_quantized_gemm_scaled", self._make_scaled(p))
            setattr(self, f"{p}_real_quantized_gemm_dual_scaled", self._make_dual(p))

    @staticmethod
    def _make_scaled(prefix):
        def fn(inputs, weights, scale_x, scale_w):
            return ops.real_quantized_gemm_scaled(prefix, inputs, weights, scale_x, scale_w)
        fn.__name__ = f"{prefix}_real_quantized_gemm_scaled"
        return fn

    @staticmethod
    def _make_dual(prefix):
        def fn(inputs, weights, pos_scale_x, neg_scale_x, scale_w):
            return ops.real_quantized_gemm_scaled(prefix, inputs, weights, pos_scale_x, scale_w, neg_scale_x=neg_scale_x)
        fn.__name__ = f"{prefix}_real_quantized_gemm_dual_scaled"
        return fn

    def create_quantized_weights(self, x):
        if self._weight_kind == L.SQ_Q_INT4:
            return torch.empty((x.numel() + 1) // 2, dtype=torch.uint8, device=x.device)
        return torch.empty_like(x, dtype=_STORAGE[self._weight_kind])

    def real_quantized_quantize_weights(self, weights, outputs, scale_w, group_size=0):
        if self._weight_kind is None:
            raise RuntimeError("the mix module registers no weight quantiser (quantized_mix.cpp:23)")
        return ops.quantize_weight(weights, outputs, scale_w, self._weight_kind, group_size=group_size)


class _FakeQuantFp8Module:
    __name__ = "segquant_fake_quant_fp8"

    @staticmethod
    def fake_e4m3fy(inputs):
        """fp -> e4m3 -> fp, saturating at +-448 and rounding to nearest even."""
        return inputs.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(inputs.dtype)


_cache = {}


def _module(key, factory, required):
    if key not in _cache:
        try:
            L.load()
        except (ImportError, OSError) as e:
            if required:
                raise RuntimeError(f"Required extension '{key}' failed to load.") from e
            raise
        _cache[key] = factory()
    return _cache[key]


def load_fake_quant_fp8_ext(verbose=False, required=False):
    return _cache.setdefault("fake_fp8", _FakeQuantFp8Module())


def load_real_quant_fp8_ext(verbose=False, required=False):
    pre = ("Wfpe4m3Afpe4m3",)
    return _module("segquant_real_quant_fp8", lambda: _RealQuantModule("segquant_real_quant_fp8", L.SQ_Q_E4M3, pre), required), pre


def load_real_quant_int8_ext(verbose=False, required=False):
    pre = ("Wint8Aint8",)
    return _module("segquant_real_quant_int8", lambda: _RealQuantModule("segquant_real_quant_int8", L.SQ_Q_INT8, pre), required), pre


def load_real_quant_int4_ext(verbose=False, required=False):
    # The reference's int4 module carries Wint4Aint4 GEMMs; this build only keeps its weight packer.
    return _module("segquant_real_quant_int4", lambda: _RealQuantModule("segquant_real_quant_int4", L.SQ_Q_INT4, ()), required), ()


def load_real_quant_mix_ext(verbose=False, required=False):
    pre = tuple(supported_type)
    return _module("segquant_real_quant_mix", lambda: _RealQuantModule("segquant_real_quant_mix", None, pre), required), pre
