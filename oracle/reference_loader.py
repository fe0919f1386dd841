"""Import the REFERENCE's own Python package (OptiSys-ZJU/segquant) without building its CUDA/CUTLASS
extensions -- TEST INFRASTRUCTURE.  Nothing of the reference is copied; it is imported from

  1. the checkout named by the environment variable SEGQUANT_REFERENCE (a directory holding `segquant/`), or
  2. `baseline/_ref/` of this repository: the unmodified package as `pip install --target baseline/_ref`
     leaves it (git-ignored; __graft_entry__.build() installs it where a checkout is present).

`import segquant` would execute segquant/__init__.py:3-7, which JIT-builds every extension with
required=True; the package module is therefore pre-registered with only its __path__.  The five loader
functions of segquant/utils/extension.py:66-213 are then replaced, before anything imports them, by

  loaders="stub"    objects without GEMM functions: SegmentLinear takes its fake-quant branch
                    (segquant/layers/SegmentLinear.py:105-113), i.e. the reference's CPU path.  This is what
                    bench.py's reference arm and the golden-vector generator run.
  loaders="native"  the loaders of segquant_b200.utils.extension: the reference's unmodified layer,
                    optimizers and quantizers then run on this library's kernels (the drop-in test).

fake_e4m3fy comes from the reference's own C++ built into oracle/_ref/ when that exists, else from the
torch cast it was verified identical to.  Only tests/, bench.py's baseline legs and the fixture generator
may import this module.
"""
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)


def find_reference():
    """Directory that holds the reference's `segquant/` package, or None."""
    cands = []
    env = os.environ.get("SEGQUANT_REFERENCE")
    if env:
        cands.append(env)
    cands.append(os.path.join(REPO, "baseline", "_ref"))
    for c in cands:
        if os.path.isfile(os.path.join(c, "segquant", "layers", "SegmentLinear.py")):
            return c
    return None


class _NoKernels:
    """A loaded 'extension' without any GEMM function."""


def _fake_fp8_module():
    from oracle.build_ref import load_prebuilt
    mod = load_prebuilt()
    if mod is not None:
        return mod, "reference C++ (oracle/_ref)"
    import torch

    class _TorchCast:
        @staticmethod
        def fake_e4m3fy(x):
            return x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(x.dtype)
    return _TorchCast(), "torch cast"


def import_reference(loaders="stub", root=None):
    """Returns a namespace with SegmentLinear, quantizer (module), optimizer (module), root, fp8_source.
    Re-imports the package from scratch on every call, so both loader sets can be used in one process."""
    root = root or find_reference()
    if root is None:
        raise FileNotFoundError("reference package not found: set SEGQUANT_REFERENCE or install it into baseline/_ref")
    for name in [m for m in sys.modules if m == "segquant" or m.startswith("segquant.")]:
        del sys.modules[name]
    if root not in sys.path:
        sys.path.insert(0, root)
    pkg = types.ModuleType("segquant")
    pkg.__path__ = [os.path.join(root, "segquant")]
    sys.modules["segquant"] = pkg
    import segquant.utils.extension as ext
    fp8, fp8_source = _fake_fp8_module()
    ext.load_fake_quant_fp8_ext = lambda verbose=False, required=False: fp8
    if loaders == "stub":
        ext.load_real_quant_fp8_ext = lambda verbose=False, required=False: (_NoKernels(), ("Wfpe4m3Afpe4m3",))
        ext.load_real_quant_int8_ext = lambda verbose=False, required=False: (_NoKernels(), ("Wint8Aint8",))
        ext.load_real_quant_int4_ext = lambda verbose=False, required=False: (_NoKernels(), ("Wint4Aint4",))
        ext.load_real_quant_mix_ext = lambda verbose=False, required=False: (_NoKernels(), tuple(ext.supported_type))
    elif loaders == "native":
        from segquant_b200.utils import extension as mine
        ext.load_real_quant_fp8_ext = mine.load_real_quant_fp8_ext
        ext.load_real_quant_int8_ext = mine.load_real_quant_int8_ext
        ext.load_real_quant_int4_ext = mine.load_real_quant_int4_ext
        ext.load_real_quant_mix_ext = mine.load_real_quant_mix_ext
    else:
        raise ValueError("loaders must be 'stub' or 'native'")
    import segquant.quantizers.quantizer as quantizer
    import segquant.optimum.optimizer as optimizer
    from segquant.layers.SegmentLinear import SegmentLinear
    return types.SimpleNamespace(SegmentLinear=SegmentLinear, quantizer=quantizer, optimizer=optimizer, root=root,
                                 fp8_source=fp8_source, ext=ext)
