"""GPU: quantize() end to end on the real-quant path -- the nn.Linear layers of a model become SegmentLinear layers that
run this library's kernels -- and the on-disk form of the result (torch.save / torch.load, bit-identical outputs; packed
int4 layouts of segquant/layers/segment_tensor_manager.py:56-80)."""
import io
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from toy_model import ToyBlock, toy_batches, toy_config  # noqa: E402

from segquant_b200 import ops  # noqa: E402
from segquant_b200.config import Calibrate, DType, Optimum  # noqa: E402
from segquant_b200.layers.SegmentLinear import SegmentLinear  # noqa: E402
from segquant_b200.torch import quantize  # noqa: E402

DEV = "cuda:0"


def cosine(a, b):
    return float(torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0))


def _to_dev(batches):
    return [((x.to(DEV), c.to(DEV)),) for ((x, c),) in batches]


@pytest.mark.parametrize("search", [False, True])
def test_quantize_real_path_equals_reference_quantize_and_round_trips(golden, native_lib, search):
    g = golden("quantize_toy_search" if search else "quantize_toy_smooth")
    model = ToyBlock().to(DEV)
    batches = _to_dev(toy_batches())
    qm = quantize(model, batches, toy_config(DType, Optimum, Calibrate, search=search, real_quant=True))
    mods = (qm.norm_lin, qm.to_q, qm.to_k, qm.to_v, qm.ff[0], qm.ff[2], qm.proj_out)
    assert [isinstance(m, SegmentLinear) for m in mods] == list(g["replaced"])
    assert all(m.optimizer.real_quant and m.optimizer.weight_manager.weight_tensor.dtype == torch.int8 for m in mods[:-1])
    alphas = [qm.to_q.optimizer.alpha[0], qm.ff[2].optimizer.alpha[0], qm.norm_lin.optimizer.alpha[0]]
    assert np.allclose(alphas, g["alphas"]), (alphas, g["alphas"])       # the search settles where the reference's did
    x, c = batches[0][0]
    n0 = ops.launch_count
    y = qm(x, c)
    assert ops.launch_count - n0 == 2 * 6                                 # quantise + GEMM per replaced linear: the native path ran
    want = torch.from_numpy(g["y"]).to(DEV)
    y = y.detach()
    rel = float((y - want).abs().max() / want.abs().max())
    assert rel <= 1e-2 and cosine(y, want) >= 0.9999, (rel, cosine(y, want))   # stated tolerance vs the reference's fake-quant model
    buf = io.BytesIO()
    torch.save(qm, buf)
    buf.seek(0)
    qm2 = torch.load(buf, weights_only=False)
    assert torch.equal(qm2(x, c), y)
    assert ops.device_status() == 0


def test_quantize_w4a8_svd_segments_packed_layout_round_trip(native_lib):
    """W4A8 + SVD + segments through quantize(): adaLN projection as 6 N-chunks with DualScale, the MLP down-projection
    as 2 K-segments with DualScale; packed int4 storage has the reference's shapes; save / load is bit-identical."""
    model = ToyBlock().to(DEV)
    batches = _to_dev(toy_batches())
    cfg = {"default": {"enable": True, "seglinear": True, "search_patterns": [], "real_quant": True,
                       "opt": {"type": Optimum.SVD, "alpha": 0.5, "low_rank": 8, "precision": "float32"},
                       "calib": {"type": Calibrate.AMAX}, "input_quant": {"type": DType.INT8, "axis": None},
                       "weight_quant": {"type": DType.INT4, "axis": 1}},
           "*proj_out": {"enable": False}}
    seg_map = {"norm_lin": {"seg_mode": "weight", "chunks": 6}, "ff.2": {"seg_mode": "input", "chunks": 2}}
    y_float = model(*batches[0][0])
    qm = quantize(model, batches, cfg, seg_map=seg_map, dual_scale=["norm_lin", "ff.2"])
    h = 64
    # storage: [N, K/2] bytes row-major (what the GEMM's TMA loads read); iter_view() hands out the reference's
    # (segments, bytes) form: contiguous per N-chunk, gathered per K-slice
    wt = qm.norm_lin.optimizer.weight_manager
    assert wt.packed and wt.weight_tensor.dtype == torch.uint8 and wt.weight_tensor.shape == (6 * h, h // 2)
    assert wt.iter_view().shape == (6, h * h // 2) and wt.iter_view().data_ptr() == wt.weight_tensor.data_ptr()
    wk = qm.ff[2].optimizer.weight_manager
    assert wk.packed and wk.weight_tensor.shape == (h, 4 * h // 2)
    seg_bytes = wk.iter_view()
    assert seg_bytes.shape == (2, h * (2 * h) // 2)
    full = ops.unpack_int4(wk.weight_tensor.reshape(-1)).view(h, 4 * h)
    for s_ in range(2):                                     # segment s of the reference layout = packed W[:, s K/2 : (s+1) K/2]
        assert torch.equal(ops.unpack_int4(seg_bytes[s_].contiguous()).view(h, 2 * h), full[:, s_ * 2 * h:(s_ + 1) * 2 * h])
    assert qm.to_q.optimizer.weight_manager.weight_tensor.numel() == h * h // 2
    x, c = batches[0][0]
    y = qm(x, c)
    assert cosine(y, y_float) >= 0.99                                  # int4 weights: a coarse check that the model still works
    buf = io.BytesIO()
    torch.save(qm, buf)
    buf.seek(0)
    qm2 = torch.load(buf, weights_only=False, map_location=DEV)
    assert torch.equal(qm2(x, c), y)
    assert ops.device_status() == 0
