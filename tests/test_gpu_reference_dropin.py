"""GPU: the drop-in claim, exercised.  The REFERENCE's own, unmodified SegmentLinear / optimizers / quantizers
(segquant/layers/SegmentLinear.py, segquant/optimum/optimizer.py, segquant/quantizers/quantizer.py) are imported with the
five loader functions of segquant/utils/extension.py:66-213 replaced by segquant_b200.utils.extension's -- the whole change
a maintainer makes -- and run with real_quant=True: calibrate -> finish_calibrate -> forward go through the reference's
code (weight packing through `real_quantized_quantize_weights`, `.contiguous()` segment views, `call_func`, the torch-side
segment sum and bias add) and land on this library's kernels through the pybind-contract functions.

The reference package is imported from $SEGQUANT_REFERENCE or from baseline/_ref (an unmodified `pip install --target`
of it, made by __graft_entry__.build() where a checkout exists); the tests skip where neither is present."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle.reference_loader import find_reference, import_reference
from segquant_b200 import ops

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ref(native_lib):
    if find_reference() is None:
        pytest.skip("reference package not available (no SEGQUANT_REFERENCE, no baseline/_ref)")
    r = import_reference("native")
    import segquant.layers as layers
    assert set(layers.ext_dict.keys()) == {"Wint8Aint8", "Wint4Aint8", "Wfpe4m3Afpe4m3"}
    return r


def max_rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def cosine(a, b):
    a, b = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


CASES = [  # golden fixture, seg_mode, chunks, quant type, input args, weight args
    ("input_seg_int8", "input", 4, "int8", {"axis": None}, {"axis": 1}),
    ("dual_fp8", "weight", 1, "fpe4m3", {"axis": None, "dual_scale": True}, {"axis": 1}),
    ("weight_seg_dual_int8", "weight", 6, "int8", {"axis": None, "dual_scale": True}, {"axis": None}),
]


@pytest.mark.parametrize("name,mode,chunks,qt,ia,wa", CASES)
def test_reference_layer_runs_on_this_librarys_kernels(golden, ref, name, mode, chunks, qt, ia, wa):
    g = golden(name)
    x, w, b = (torch.from_numpy(g[k]).to(DEV) for k in "xwb")

    def build(real):
        lin = ref.SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w.clone(),
                                custom_bias_tensor=b.clone(), input_quant_type=qt, weight_quant_type=qt,
                                input_quant_args=dict(ia, real_quant=real), weight_quant_args=dict(wa, real_quant=real),
                                opt_type="default", opt_kwargs={}, calib_type="amax", calib_kwargs={}, device=DEV)
        lin.calibrate(x.clone())
        lin.finish_calibrate()
        return lin

    real = build(True)
    assert real.optimizer.real_quant, "the reference layer fell back to fake quantisation: kernels not found"
    assert real.optimizer.weight_manager.weight_tensor.dtype in (torch.int8, torch.uint8)
    n0 = ops.launch_count
    y = real(x.clone())
    assert ops.launch_count - n0 == 2, "one quantise + one GEMM launch of this library per reference forward"
    y = y.cpu().numpy()
    assert max_rel(y, g["y"]) <= 1e-2 and cosine(y, g["y"]) >= 0.9999          # stated tolerance vs the reference's CPU output
    assert max_rel(y, g["y"]) <= 2e-5                                          # measured: fp32 rounding only
    fake = build(False)(x.clone()).cpu().numpy()                               # the same reference layer, fake quant, on the GPU
    assert max_rel(y, fake) <= 2e-5
    assert ops.device_status() == 0


def test_reference_smooth_layer_and_bf16(golden, ref):
    g = golden("smooth_input_seg_int8")
    x, w, b = (torch.from_numpy(g[k]).to(DEV) for k in "xwb")
    lin = ref.SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode="input", chunks=4, custom_weight_tensor=w.clone(),
                            custom_bias_tensor=b.clone(), input_quant_type="int8", weight_quant_type="int8",
                            input_quant_args={"real_quant": True, "axis": None}, weight_quant_args={"real_quant": True, "axis": 1},
                            opt_type="smooth", opt_kwargs={"alpha": 0.5}, calib_type="amax", calib_kwargs={}, device=DEV)
    lin.trace(x.clone())
    lin.smooth()
    lin.calibrate(x.clone())
    lin.finish_calibrate()
    y = lin(x.clone()).cpu().numpy()
    assert max_rel(y, g["y"]) <= 1e-2 and cosine(y, g["y"]) >= 0.9999
    yb = lin(x.to(torch.bfloat16))       # the kernels return bf16; the reference's `+ bias_data` (fp32 here) promotes the sum
    assert cosine(yb.float().cpu().numpy(), g["y"]) >= 0.9999
    assert ops.device_status() == 0
