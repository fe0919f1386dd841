"""CPU: quantize() end to end (collect -> trace -> smooth -> [alpha search] -> calibrate -> replace) against outputs of
the REFERENCE's own quantize() on the same toy model (tests/golden/quantize_toy_*.npz, made by make_golden.py), the
torch.save / torch.load form of a quantised model, and the packed-int4 layouts."""
import io
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from toy_model import ToyBlock, toy_batches, toy_config  # noqa: E402

from segquant_b200.calibrator.calibrator import colpacked1d_to_rowpacked1d  # noqa: E402
from segquant_b200.config import Calibrate, DType, Optimum  # noqa: E402
from segquant_b200.layers.SegmentLinear import SegmentLinear  # noqa: E402
from segquant_b200.torch import quantize  # noqa: E402


@pytest.mark.parametrize("name,search", [("quantize_toy_smooth", False), ("quantize_toy_search", True)])
def test_quantize_equals_reference_quantize(golden, name, search):
    g = golden(name)
    model = ToyBlock()
    batches = toy_batches()
    x, c = batches[0][0]
    assert np.allclose(model(x, c).detach().numpy(), g["y_float"], atol=1e-6)
    qm = quantize(model, batches, toy_config(DType, Optimum, Calibrate, search=search))
    mods = (qm.norm_lin, qm.to_q, qm.to_k, qm.to_v, qm.ff[0], qm.ff[2], qm.proj_out)
    assert [isinstance(m, SegmentLinear) for m in mods] == list(g["replaced"])     # *proj_out stays an nn.Linear
    alphas = [qm.to_q.optimizer.alpha[0], qm.ff[2].optimizer.alpha[0], qm.norm_lin.optimizer.alpha[0]]
    assert np.allclose(alphas, g["alphas"])
    assert np.allclose(qm.to_q.optimizer.scale_tensor[0].numpy(), g["sx_to_q"], rtol=1e-6)
    assert np.allclose(qm.ff[2].optimizer.scale_tensor[1].numpy(), g["sw_ff2"], rtol=1e-6)
    x0 = x.clone()
    y = qm(x, c).detach().numpy()
    assert torch.equal(x, x0)
    assert np.abs(y - g["y"]).max() <= 2e-5 * np.abs(g["y"]).max()
    # the on-disk form: the whole module pickled, outputs bit-identical after the round trip
    buf = io.BytesIO()
    torch.save(qm, buf)
    buf.seek(0)
    qm2 = torch.load(buf, weights_only=False)
    assert torch.equal(qm2(x, c), qm(x, c))


def test_quantize_segment_map_dual_scale_and_patterns():
    model = ToyBlock()
    batches = toy_batches()
    cfg = toy_config(DType, Optimum, Calibrate)
    cfg["default"]["seglinear"] = True
    cfg["default"]["opt"] = {"type": "default"}                      # plain strings (a parsed YAML file) work like enums
    cfg["default"]["input_quant"] = {"type": "int8", "axis": None}
    with pytest.raises(NotImplementedError, match="seg_map"):
        quantize(ToyBlock(), batches, cfg)
    cfg["to_v"] = {"enable": True, "seglinear": False}
    seg_map = {"norm_lin": {"seg_mode": "weight", "chunks": 6}, "ff.2": {"seg_mode": "input", "chunksizes": [128, 128]},
               "to_v": {"seg_mode": "input", "chunks": 2}, "not_a_layer": {"seg_mode": "weight", "chunks": 2}}
    qm = quantize(model, batches, cfg, seg_map=seg_map, dual_scale=["norm_lin", "ff.2"])
    assert qm.norm_lin.seg_mode == "weight" and qm.norm_lin.chunks == 6 and qm.norm_lin.optimizer.dual_scale
    assert qm.ff[2].seg_mode == "input" and qm.ff[2].chunksizes == [128, 128] and qm.ff[2].optimizer.dual_scale
    assert qm.to_v.chunks == 1 and not qm.to_v.optimizer.dual_scale   # matched a pattern with seglinear: false
    assert isinstance(qm.proj_out, torch.nn.Linear)
    x, c = batches[1][0]
    y, y_float = qm(x, c), ToyBlock()(x, c)
    assert torch.nn.functional.cosine_similarity(y.flatten(), y_float.flatten(), dim=0) > 0.999
    off = {"default": dict(cfg["default"], enable=False)}
    m = ToyBlock()
    assert quantize(m, batches, off) is m and isinstance(m.to_q, torch.nn.Linear)


def test_colpacked_to_rowpacked_int4():
    g = torch.Generator().manual_seed(3)
    out, cols = 6, 8
    w = torch.randint(0, 16, (out, cols), generator=g, dtype=torch.uint8)          # nibbles
    col = (w[0::2] | (w[1::2] << 4)).t().contiguous().reshape(-1)                   # (cols, out/2): rows paired
    row = colpacked1d_to_rowpacked1d(col, out, cols)
    want = (w[:, 0::2] | (w[:, 1::2] << 4)).reshape(-1)
    assert torch.equal(row, want)
    with pytest.raises(ValueError):
        colpacked1d_to_rowpacked1d(col[:3], 3, 2)
