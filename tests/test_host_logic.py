"""CPU: host-side mirror of the reference's layer / optimizer / quantizer API."""
import numpy as np
import pytest
import torch

from segquant_b200.calibrator.calibrator import CalibratorRegistry
from segquant_b200.config import Calibrate, DType, Optimum, SegPattern, default_quantize_config
from segquant_b200.layers.SegmentLinear import DualScale, SegmentLinear, create_segment_linear
from segquant_b200.layers.segment_tensor_manager import InputSegmentTensorManager, WeightSegmentTensorManager
from segquant_b200.quantizers.quantizer import FloatQuantizer, IntQuantizer, QuantizerRegistry


def make_layer(g, seg_mode, chunks, itype, wtype, iargs, wargs, **kw):
    x, w, b = (torch.from_numpy(g[k]) for k in "xwb")
    lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=seg_mode, chunks=chunks, custom_weight_tensor=w,
                        custom_bias_tensor=b, input_quant_type=itype, weight_quant_type=wtype, input_quant_args=iargs,
                        weight_quant_args=wargs, device="cpu", **kw)
    lin.calibrate(x)
    lin.finish_calibrate()
    return lin, x


def test_fake_layer_equals_reference_int8_k_segments(golden):
    g = golden("input_seg_int8")
    lin, x = make_layer(g, "input", 4, "int8", "int8", {"real_quant": False, "axis": None}, {"real_quant": False, "axis": 1})
    x0 = x.clone()
    y = lin(x)
    assert torch.equal(x, x0), "forward must not write into its input"
    assert torch.allclose(y, torch.from_numpy(g["y"]), rtol=1e-6, atol=1e-6)
    sx, sw = lin.optimizer.scale_tensor
    assert sx.shape == (4,) and sw.shape == (4, 64) and sx.dtype == torch.float32
    assert np.allclose(sx.numpy(), g["sx"]) and np.allclose(sw.numpy(), g["sw"])
    parts = lin(x, chunked=True)
    assert parts.shape == (4, x.shape[0], 64)
    assert torch.allclose(parts.sum(0) + lin.bias_data, y, atol=1e-5)


def test_fake_layer_equals_reference_dual_fp8_and_weight_segments(golden):
    g = golden("dual_fp8")
    lin, x = make_layer(g, "weight", 1, "fpe4m3", "fpe4m3", {"real_quant": False, "axis": None, "dual_scale": True},
                        {"real_quant": False, "axis": 1})
    assert torch.allclose(lin(x), torch.from_numpy(g["y"]), rtol=1e-5, atol=1e-6)
    pos, neg, sw = lin.optimizer.scale_tensor
    assert np.allclose(pos.numpy(), g["sx_pos"]) and np.allclose(neg.numpy(), g["sx_neg"]) and np.allclose(sw.numpy(), g["sw"])
    g = golden("weight_seg_dual_int8")
    lin, x = make_layer(g, "weight", 6, "int8", "int8", {"real_quant": False, "axis": None, "dual_scale": True},
                        {"real_quant": False, "axis": None})
    assert torch.allclose(lin(x), torch.from_numpy(g["y"]), rtol=1e-6, atol=1e-6)
    assert lin.optimizer.scale_tensor[2].shape == (6,)
    assert lin(x, chunked=True).shape == (6, x.shape[0], 32)


def test_quantizers_equal_reference_vectors(golden):
    g = golden("quantizers")
    x = torch.from_numpy(g["int8_x"])
    q = IntQuantizer(num_bits=8)
    q.calibrate(x)
    assert np.isclose(q.scale, g["int8_scale"]) and torch.equal(q.fake_quantize(x), torch.from_numpy(g["int8_fake"]))
    q = IntQuantizer(num_bits=8, axis=1)
    q.calibrate(x)
    assert torch.allclose(q.scale, torch.from_numpy(g["int8_axis1_scale"])) and torch.equal(q.fake_quantize(x), torch.from_numpy(g["int8_axis1_fake"]))
    xs = torch.from_numpy(g["dual_x"])
    q = IntQuantizer(dual_scale=True)
    q.calibrate(xs)
    assert np.isclose(q.pos_scale, g["dual_int8_pos"]) and np.isclose(q.neg_scale, g["dual_int8_neg"])
    assert torch.equal(q.fake_quantize(xs), torch.from_numpy(g["dual_int8_fake"]))
    f = FloatQuantizer()
    f.calibrate(x)
    assert np.isclose(f.scale, g["fp8_scale"]) and torch.equal(f.fake_quantize(x), torch.from_numpy(g["fp8_fake"]))
    f = FloatQuantizer(dual_scale=True)
    f.calibrate(xs)
    assert torch.equal(f.fake_quantize(xs), torch.from_numpy(g["dual_fp8_fake"]))
    d = IntQuantizer(axis=-1, dynamic=True)
    assert torch.equal(d.quantize(x), torch.from_numpy(g["dyn_fake"])) and torch.allclose(d.scale, torch.from_numpy(g["dyn_scale"]))
    # new: group-wise int4 equals the reference's quantiser applied to W.view(N, K/g, g)
    w = torch.from_numpy(g["int4_w"])
    q4 = QuantizerRegistry.create("int4", group_size=128)
    q4.calibrate(w)
    assert torch.allclose(q4.scale, torch.from_numpy(g["int4_group_scale"]))
    assert torch.equal(q4.fake_quantize(w), torch.from_numpy(g["int4_group_fake"]))
    repr(f), repr(q4), repr(FloatQuantizer(axis=1))   # the reference's FloatQuantizer.__repr__ crashes for axis amax


def test_running_max_and_epsilon_guard():
    q = IntQuantizer()
    q.calibrate(torch.tensor([1.0, -2.0]))
    q.calibrate(torch.tensor([0.5]))
    assert q.amax == 2.0 and q.scale == 127 / 2.0
    z = IntQuantizer()
    z.calibrate(torch.zeros(4))
    assert z.scale == 1.0
    d = FloatQuantizer(dual_scale=True)
    d.calibrate(torch.tensor([1.0, 2.0]))        # no negatives at all
    assert d.neg_scale == 1.0 and d.pos_scale == 224.0
    with pytest.raises(ValueError):
        QuantizerRegistry.create("int3")
    with pytest.raises(AssertionError):
        IntQuantizer(real_quant=True, axis=0)


def test_segment_views():
    x = torch.arange(2 * 3 * 8, dtype=torch.float32).view(2, 3, 8)
    m = InputSegmentTensorManager(x, "input", 4, 2)
    v = m.iter_view()
    assert v.shape == (4, 2, 3, 2) and v.data_ptr() == x.data_ptr() and torch.equal(v[1], x[..., 2:4])
    e = InputSegmentTensorManager(x, "weight", 3, 0).iter_view()
    assert e.shape == (3, 2, 3, 8) and e.stride(0) == 0
    u = InputSegmentTensorManager(x, "input", 2, 2, segment_sizes=[2, 6])
    assert [t.shape[-1] for t in u.iter_list()] == [2, 6]
    with pytest.raises(NotImplementedError):
        u.iter_view()
    w = torch.arange(6 * 8, dtype=torch.float32).view(6, 8)
    wm = WeightSegmentTensorManager(w, "input", 4, 2)
    assert wm.iter_view().shape == (4, 6, 2) and torch.equal(wm.iter_view()[3], w[:, 6:8])
    wm2 = WeightSegmentTensorManager(w, "weight", 3, 2)
    assert wm2.iter_view().shape == (3, 2, 8)
    wm2.replace_with_segments_layout(torch.stack([w[0:2] * 2, w[2:4] * 2, w[4:6] * 2]))
    assert torch.equal(wm2.weight_tensor, w * 2)
    # packed int4 bytes: (S, N/S * K/2) per segment in weight mode
    packed = torch.arange(3 * 2 * 4, dtype=torch.uint8).view(3, 8)
    wm2.replace_with_segments_layout(packed, packed=True)
    assert wm2.packed and wm2.weight_tensor.shape == (6, 4) and torch.equal(wm2.iter_view(), packed)


def test_unequal_k_segments_fake_path():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(16, 96, generator=g)
    x[:, 32:] *= 3
    w = torch.randn(8, 96, generator=g) * 0.05
    lin = SegmentLinear(96, 8, bias=False, seg_mode="input", chunks=2, chunksizes=[32, 64], custom_weight_tensor=w,
                        input_quant_type="int8", weight_quant_type="int8", input_quant_args={"real_quant": False},
                        weight_quant_args={"real_quant": False, "axis": 1}, device="cpu")
    lin.calibrate(x)
    lin.finish_calibrate()
    y = lin(x)
    assert y.shape == (16, 8) and lin.optimizer.scale_tensor[0].shape == (2,)
    assert torch.nn.functional.cosine_similarity(y.flatten(), (x @ w.t()).flatten(), dim=0) > 0.999
    with pytest.raises(NotImplementedError):
        SegmentLinear(96, 8, seg_mode="weight", chunks=2, chunksizes=[3, 5], input_quant_type="int8", weight_quant_type="int8",
                      input_quant_args={}, weight_quant_args={}, device="cpu")


def test_real_quant_never_falls_back(native_lib):
    w = torch.randn(8, 32)
    with pytest.raises(RuntimeError, match="no fake-quant fallback"):
        SegmentLinear(32, 8, input_quant_type="int4", weight_quant_type="int4", input_quant_args={"real_quant": True},
                      weight_quant_args={"real_quant": True}, custom_weight_tensor=w, device="cpu")
    lin = SegmentLinear(32, 8, input_quant_type="int8", weight_quant_type="int8", input_quant_args={"real_quant": True},
                        weight_quant_args={"real_quant": True, "axis": 1}, custom_weight_tensor=w, device="cpu")
    lin.calibrate(torch.randn(4, 32))
    with pytest.raises(RuntimeError, match="CUDA device"):
        lin.finish_calibrate()      # the weight packer is a CUDA kernel; CPU tensors are refused, not emulated
    with pytest.raises(AssertionError):
        SegmentLinear(32, 8, input_quant_type="int8", weight_quant_type="int8", input_quant_args={"real_quant": True},
                      weight_quant_args={"real_quant": False}, device="cpu")
    with pytest.raises(ValueError):
        SegmentLinear(32, 8, input_quant_type="int8", weight_quant_type="int8", input_quant_args={},
                      weight_quant_args={"dual_scale": True}, device="cpu")


def test_config_and_registries():
    assert DType.FP8E4M3.value == "fpe4m3" and Optimum.SVD.value == "svd" and Calibrate.GPTQ.value == "gptq"
    assert len(SegPattern.all()) == 6 and SegPattern.ACTIVATION2LINEAR not in SegPattern.seg()
    d = default_quantize_config["default"]
    assert d["real_quant"] is False and d["opt"]["type"] is Optimum.SMOOTH and d["input_quant"]["type"] is DType.INT8
    with pytest.raises(NotImplementedError):
        CalibratorRegistry.create("gptq", data_type="weight", quant_type="int8", quant_args={})
    lin = create_segment_linear(DType.INT8, DType.INT8, Optimum.DEFAULT, Calibrate.AMAX, 16, 4, {}, {}, {"real_quant": False},
                                {"real_quant": False}, device="cpu")
    assert isinstance(lin, SegmentLinear) and lin.optimizer.kernel_type == "Wint8Aint8"
    d2 = DualScale(16, 4, input_quant_type="int8", weight_quant_type="int8", weight_quant_args={}, device="cpu")
    assert d2.optimizer.dual_scale and d2.optimizer.func_name == "gemm_scaled_fn"   # fake quant: plain function


def test_extension_loader_names(native_lib):
    from segquant_b200.utils import extension as E
    from segquant_b200.layers import ext_dict
    ext, pre = E.load_real_quant_int8_ext(required=True)
    assert pre == ("Wint8Aint8",) and callable(ext.Wint8Aint8_real_quantized_gemm_scaled) and callable(ext.Wint8Aint8_real_quantized_gemm_dual_scaled)
    assert ext.create_quantized_weights(torch.zeros(4, 8)).dtype == torch.int8
    ext4, _ = E.load_real_quant_int4_ext()
    assert ext4.create_quantized_weights(torch.zeros(4, 8)).shape == (16,)
    extf, pref = E.load_real_quant_fp8_ext()
    assert pref == ("Wfpe4m3Afpe4m3",) and extf.create_quantized_weights(torch.zeros(2, 2)).dtype == torch.uint8
    _, mix = E.load_real_quant_mix_ext()
    assert set(mix) == {"Wint8Aint8", "Wint4Aint8", "Wfpe4m3Afpe4m3"} == set(ext_dict.keys())
    f = E.load_fake_quant_fp8_ext().fake_e4m3fy(torch.tensor([1000.0, 17.0, -0.3]))
    assert f.tolist() == [448.0, 16.0, -0.3125]
    with pytest.raises(RuntimeError, match="CUDA device"):
        ext.Wint8Aint8_real_quantized_gemm_scaled(torch.zeros(1, 4, 32), torch.zeros(1, 8, 32, dtype=torch.int8), torch.ones(1), torch.ones(1))


@pytest.mark.parametrize("name,mode,chunks", [("smooth_input_seg_int8", "input", 4), ("smooth_weight_seg_int8", "weight", 2)])
def test_smooth_optimizer_equals_reference(golden, name, mode, chunks):
    """trace -> smooth -> calibrate -> finish -> forward against vectors the reference's SmoothOptimizer produced
    (segquant/optimum/optimizer.py:295-521)."""
    g = golden(name)
    x, w, b = (torch.from_numpy(g[k]) for k in "xwb")
    lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w,
                        custom_bias_tensor=b, input_quant_type="int8", weight_quant_type="int8",
                        input_quant_args={"real_quant": False, "axis": None}, weight_quant_args={"real_quant": False, "axis": 1},
                        opt_type="smooth", opt_kwargs={"alpha": 0.5}, device="cpu")
    with pytest.raises(AssertionError):
        lin.calibrate(x)                      # not smoothed yet
    lin.trace(x)
    lin.smooth()
    lin.calibrate(x)
    lin.finish_calibrate()
    s = torch.stack(lin.optimizer.s)
    assert np.allclose(s.numpy(), g["s"], rtol=1e-6)
    sx, sw = lin.optimizer.scale_tensor
    assert np.allclose(sx.numpy(), g["sx"], rtol=1e-6) and np.allclose(sw.numpy(), g["sw"], rtol=1e-6)
    x0 = x.clone()
    y = lin(x)
    assert torch.equal(x, x0)
    assert torch.allclose(y, torch.from_numpy(g["y"]), rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------------------------------------
# SVDOptimizer (low-rank branch) and SmoothOptimizer's alpha search
# ---------------------------------------------------------------------------------------------
def _svd_layer(g, mode, chunks, dynamic=False, real=False, device="cpu", **opt):
    x, w, b = (torch.from_numpy(g[k]) for k in "xwb")
    in_args = {"real_quant": real, "axis": -1, "dynamic": True} if dynamic else {"real_quant": real, "axis": None}
    lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w.to(device),
                        custom_bias_tensor=b.to(device), input_quant_type="int8", weight_quant_type="int4", input_quant_args=in_args,
                        weight_quant_args={"real_quant": real, "axis": 1}, opt_type="svd",
                        opt_kwargs=dict({"alpha": 0.5, "low_rank": int(g["low_rank"]), "precision": "float64"}, **opt), device=device)
    x = x.to(device)
    lin.trace(x)
    lin.smooth()
    lin.calibrate(x)
    lin.finish_calibrate()
    return lin, x


@pytest.mark.parametrize("name,mode,dynamic", [("svd_w4a8_input_seg", "input", False), ("svd_w4a8_dynamic", "weight", True),
                                               ("svd_w4a8_weight_seg", "weight", False)])
def test_svd_optimizer_fake_path_equals_reference(golden, name, mode, dynamic):
    """opt_type="svd" with real_quant=False reproduces the reference's CPU output, its smoothing vector, the product of
    its low-rank factors (the factors themselves are only defined up to the sign of each singular pair) and the
    fake-quantised residual weight."""
    g = golden(name)
    lin, x = _svd_layer(g, mode, int(g["chunks"]), dynamic)
    opt = lin.optimizer
    assert np.allclose(torch.stack(opt.s).numpy(), g["s"], rtol=1e-6)
    prod = torch.bmm(opt.l1s, opt.l2s).numpy()
    want = np.matmul(g["l1s"], g["l2s"])
    assert np.abs(prod - want).max() <= 1e-6 * np.abs(want).max() + 1e-7
    assert opt.l1s.shape == g["l1s"].shape and opt.l2s.shape == g["l2s"].shape
    assert np.allclose(opt.weight_manager.weight_tensor.numpy(), g["w_fake"], atol=1e-6)
    x0 = x.clone()
    y = lin(x).numpy()
    assert torch.equal(x, x0)
    assert np.abs(y - g["y"]).max() <= 2e-5 * np.abs(g["y"]).max()
    parts = lin(x, chunked=True)
    y2 = (parts.sum(0) if mode == "input" else parts.movedim(0, -2).reshape(x.shape[0], -1)) + lin.bias_data
    assert np.abs(y2.numpy() - y).max() <= 1e-5
    assert "SVDOptimizer" in repr(lin)


def test_smooth_alpha_search_life_cycle(golden):
    """search_alpha_config: candidates are tried in order, the best alpha per chunk is kept, the weight is restored
    between candidates, and (as in the reference) the last candidate of the range is never evaluated."""
    g = golden("smooth_input_seg_int8")
    x, w, b = (torch.from_numpy(g[k]) for k in "xwb")
    lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode="input", chunks=4, custom_weight_tensor=w, custom_bias_tensor=b,
                        input_quant_type="int8", weight_quant_type="int8", input_quant_args={"real_quant": False, "axis": None},
                        weight_quant_args={"real_quant": False, "axis": 1}, opt_type="smooth",
                        opt_kwargs={"alpha": 0.5, "search_alpha_config": {"enable": True, "min": 0.2, "max": 0.8, "step": 0.2}}, device="cpu")
    opt = lin.optimizer
    assert opt.search_alpha and opt.alpha == [pytest.approx(0.2)] * 4
    lin.trace(x)
    tried, done = [], False
    while not done:
        tried.append(opt.alpha[0])
        lin.smooth()
        lin.calibrate(x)
        lin.finish_calibrate()
        real = lin.segment_forward(x, w)
        cur = lin(x, chunked=True)
        errs = [((r - c) ** 2).mean().item() for r, c in zip(real, cur)]
        # make chunk 2 prefer the second candidate whatever the data says
        if len(tried) == 2:
            errs[2] = -1.0
        done = opt.search_step(errs, origin_weight=w)
        assert torch.equal(opt.weight_manager.weight_tensor, w) and not opt.has_smoothed
    assert [round(a, 6) for a in tried] == [0.2, 0.4, 0.6]            # 0.8 is popped by the step that ends the search
    assert not opt.search_alpha and opt.alpha[2] == pytest.approx(0.4)
    lin.smooth()
    lin.calibrate(x)
    lin.finish_calibrate()
    y = lin(x)
    assert torch.isfinite(y).all() and opt.max_x is None
    ref = x @ w.t() + b
    assert torch.nn.functional.cosine_similarity(y.flatten(), ref.flatten(), dim=0) > 0.999
