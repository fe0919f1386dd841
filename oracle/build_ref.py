"""Compile the reference's fake-quant fp8 extension from its own sources into oracle/_ref/.

    python oracle/build_ref.py [<reference checkout>]

The two files (segquant/src/fake_quant/quantizer_fp8.cpp and .cu) are compiled where they lie; only
build products are written, and only under oracle/_ref/.  The result is the function
`fake_e4m3fy(float32 tensor) -> float32 tensor` (quantizer_fp8.cpp:25-43), used to pin the oracle's
e4m3 encoder and by the golden-vector generator.  Test infrastructure only.
"""
import os
import sys


def build(reference_root):
    from torch.utils.cpp_extension import load
    here = os.path.dirname(os.path.abspath(__file__))
    out = os.path.join(here, "_ref")
    os.makedirs(out, exist_ok=True)
    src = os.path.join(reference_root, "segquant", "src", "fake_quant")
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return load(
        name="segquant_fake_quant_fp8",
        sources=[os.path.join(src, "quantizer_fp8.cpp"), os.path.join(src, "quantizer_fp8.cu")],
        build_directory=out,
        verbose=False,
    )


def load_prebuilt():
    """Import oracle/_ref/segquant_fake_quant_fp8.so if it was built earlier; None otherwise."""
    import importlib.util
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "_ref", "segquant_fake_quant_fp8.so")
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("segquant_fake_quant_fp8", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SEGQUANT_REFERENCE")
    if not root:
        raise SystemExit("usage: build_ref.py <reference checkout>  (or set SEGQUANT_REFERENCE)")
    m = build(root)
    print("built", m.__file__ if hasattr(m, "__file__") else m)
