"""`ext_dict`: kernel-type string -> the two GEMM entry points, as in the reference
(segquant/layers/__init__.py:3-21).  Built lazily so that importing the package does not need the
native library; looking a kernel up does."""
from ..utils.extension import (load_real_quant_fp8_ext, load_real_quant_int4_ext, load_real_quant_int8_ext,
                               load_real_quant_mix_ext)


def build_ext_dict():
    d = {}
    for loader in (load_real_quant_mix_ext, load_real_quant_fp8_ext, load_real_quant_int8_ext, load_real_quant_int4_ext):
        ext, prefixes = loader(required=True)
        for p in prefixes:
            d[p] = {
                "gemm_scaled_fn": getattr(ext, f"{p}_real_quantized_gemm_scaled", None),
                "gemm_dual_scaled_fn": getattr(ext, f"{p}_real_quantized_gemm_dual_scaled", None),
            }
    return d


class _LazyExtDict(dict):
    _built = False

    def _ensure(self):
        if not self._built:
            self.update(build_ext_dict())
            self._built = True

    def __contains__(self, key):
        self._ensure()
        return super().__contains__(key)

    def __getitem__(self, key):
        self._ensure()
        return super().__getitem__(key)

    def keys(self):
        self._ensure()
        return super().keys()


ext_dict = _LazyExtDict()
