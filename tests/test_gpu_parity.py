"""GPU: the CUDA path, called through the C ABI (segquant_b200.ops -> libsegquant_b200.so), against the
CPU oracle on the same seeded inputs and against the reference's own outputs in tests/golden/.

Bars: quantised bytes, packed weights and int32 accumulators are bit-exact; dequantised fp32 outputs
are within 1e-5 relative of the oracle (it divides by the scale product, the kernel multiplies by
its fp32 reciprocal); outputs versus the reference's fake-quant path: max rel err <= 1e-2 and
cosine >= 0.9999 (the tolerance the task states), bf16 outputs compared after one bf16 rounding.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import fake_path as F
from oracle import oracle as O
from segquant_b200 import _lib as L
from segquant_b200 import ops
from segquant_b200.layers.SegmentLinear import SegmentLinear

DEV = "cuda:0"
KIND = {"i8": (L.SQ_GEMM_W8A8_I8, O.GEMM_I8), "f8": (L.SQ_GEMM_W8A8_F8, O.GEMM_F8), "w4": (L.SQ_GEMM_W4A8, O.GEMM_W4A8)}


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield
    assert ops.device_status() == 0, "a kernel reported a bounded wait that ran out"


def max_rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def cosine(a, b):
    a, b = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def t(a, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a))
    return (x.to(dtype) if dtype else x).to(DEV)


# ---------------------------------------------------------------------------------------------
# activation quantise
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kind", [O.Q_INT8, O.Q_E4M3])
@pytest.mark.parametrize("dual", [False, True])
def test_act_quant_bit_exact(dtype, kind, dual):
    g = torch.Generator().manual_seed(11)
    M, K = 333, 1536
    bounds = [0, 384, 768, 1152, 1536]
    x = torch.randn(M, K, generator=g)
    for s, f in enumerate([0.5, 1.0, 4.0, 16.0]):
        x[:, bounds[s]:bounds[s + 1]] *= f
    x[0, :8] = torch.tensor([0.0, -0.0, 6e4, -6e4, 0.5, -0.5, 1.5, 2.5])   # finite in fp16 too
    x = x.to(dtype)
    xf = x.float().numpy()
    qmax = 127.0 if kind == O.Q_INT8 else 448.0
    sx = np.array([qmax / np.abs(xf[:, bounds[s]:bounds[s + 1]]).max() for s in range(4)], np.float32)
    sxn = (sx * 7.3).astype(np.float32) if dual else None
    want = O.quantize_act(xf, bounds, sx, sx_neg=sxn, out_kind=kind)
    xq, xqn = ops.quantize_act(x.to(DEV), bounds, t(sx), t(sxn) if dual else None, kind)
    if dual:
        assert np.array_equal(xq[0].cpu().numpy(), want[0].view(np.uint8)) and np.array_equal(xqn[0].cpu().numpy(), want[1].view(np.uint8))
    else:
        assert np.array_equal(xq[0].cpu().numpy(), want.view(np.uint8))


def test_act_quant_strided_views_and_unequal_segments():
    g = torch.Generator().manual_seed(12)
    base = torch.randn(64, 512 + 64, generator=g).to(DEV)
    x = base[:, 32:32 + 512]                       # row stride 576, 16-byte aligned start
    bounds = [0, 128, 512]
    sx = np.array([30.0, 11.0], np.float32)
    xq, _ = ops.quantize_act(x, bounds, t(sx), None, L.SQ_Q_INT8)
    want = O.quantize_act(x.cpu().numpy(), bounds, sx, out_kind=O.Q_INT8)
    assert np.array_equal(xq[0].cpu().numpy().view(np.int8), want)
    # (S, M, K/S) permuted view of one [M, K] matrix: the reference's input-segment view, read in place
    y = torch.randn(40, 4, 96, generator=g).to(DEV)
    v = y.permute(1, 0, 2)                          # (4, 40, 96), batch stride 96, row stride 384
    s4 = np.array([5.0, 9.0, 13.0, 21.0], np.float32)
    xq, _ = ops.quantize_act(v, [0, 96], t(s4), None, L.SQ_Q_E4M3)
    for s in range(4):
        want = O.quantize_act(v[s].cpu().numpy(), [0, 96], s4[s:s + 1], out_kind=O.Q_E4M3)
        assert np.array_equal(xq[s].cpu().numpy(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dual", [False, True])
def test_act_quant_dynamic_per_token(dtype, dual):
    g = torch.Generator().manual_seed(13)
    M, K = 77, 1024
    bounds = [0, 256, 1024]
    x = (torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 5).to(dtype)
    if dual:
        x = torch.nn.functional.silu(x.float()).to(dtype)
    xq, xqn, sx, sxn = ops.quantize_act_dynamic(x.to(DEV), bounds, L.SQ_Q_INT8, dual=dual)
    # the reference's definition: qmax / amax.clamp(eps) computed on the tensor's own dtype
    sx_ref, sxn_ref = [], []
    for s in range(2):
        seg = x[:, bounds[s]:bounds[s + 1]]
        if dual:
            pos = torch.where(seg > 0, seg, torch.zeros_like(seg)).amax(dim=-1)
            neg = torch.where(seg < 0, -seg, torch.zeros_like(seg)).amax(dim=-1)
            sx_ref.append((127.0 / pos.clamp(min=F.EPS)).float())
            sxn_ref.append((128.0 / neg.clamp(min=F.EPS)).float())
        else:
            sx_ref.append(F.amax_scale(seg, 127.0, axis=-1).float())
    sx_ref = torch.stack(sx_ref)
    assert torch.equal(sx.cpu(), sx_ref)
    if dual:
        sxn_ref = torch.stack(sxn_ref)
        assert torch.equal(sxn.cpu(), sxn_ref)
        want = O.quantize_act(x.float().numpy(), bounds, sx_ref.numpy(), sx_neg=sxn_ref.numpy(), out_kind=O.Q_INT8)
        assert np.array_equal(xq.cpu().numpy().view(np.int8), want[0]) and np.array_equal(xqn.cpu().numpy().view(np.int8), want[1])
    else:
        want = O.quantize_act(x.float().numpy(), bounds, sx_ref.numpy(), out_kind=O.Q_INT8)
        assert np.array_equal(xq.cpu().numpy().view(np.int8), want)


def test_act_quant_empty_and_errors():
    x = torch.zeros(0, 64, device=DEV)
    xq, _ = ops.quantize_act(x, [0, 64], t(np.ones(1, np.float32)), None, L.SQ_Q_INT8)
    assert xq.shape == (1, 0, 64)
    with pytest.raises(L.SegQuantError) as e:
        ops.quantize_act(torch.zeros(4, 24, device=DEV), [0, 24], t(np.ones(1, np.float32)), None, L.SQ_Q_INT8)
    assert e.value.status == L.SQ_ERR_ALIGNMENT
    with pytest.raises(RuntimeError, match="CUDA device"):
        ops.quantize_act(torch.zeros(4, 32), [0, 32], torch.ones(1), None, L.SQ_Q_INT8)


# ---------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", [O.Q_INT8, O.Q_E4M3, O.Q_INT4])
@pytest.mark.parametrize("mode", ["scalar", "row", "group"])
def test_weight_quant_bit_exact(dtype, kind, mode):
    g = torch.Generator().manual_seed(14)
    N, K = 96, 512
    w = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    wf = w.float().numpy()
    qmax = {O.Q_INT8: 127.0, O.Q_E4M3: 448.0, O.Q_INT4: 7.0}[kind]
    if mode == "scalar":
        scale, group = float(qmax / np.abs(wf).max()), 0
        scale_t = scale
    elif mode == "row":
        scale, group = (qmax / np.abs(wf).max(axis=1)).astype(np.float32), 0
        scale_t = t(scale)
    else:
        group = 128
        scale = (qmax / np.abs(wf.reshape(N, K // group, group)).max(axis=2)).astype(np.float32)
        scale_t = t(scale)
    want = O.quantize_weight(wf, scale, kind, group_size=group)
    out = torch.empty(N * K // 2 if kind == O.Q_INT4 else (N, K), dtype=torch.uint8, device=DEV)
    ops.quantize_weight(w.to(DEV), out, scale_t, kind, group_size=group)
    assert np.array_equal(out.cpu().numpy().reshape(-1), want.view(np.uint8).reshape(-1))
    if kind == O.Q_INT4:
        un = ops.unpack_int4(out)
        assert np.array_equal(un.cpu().numpy(), O.unpack_int4(want, N * K))
        assert un.min() >= -8 and un.max() <= 7


def test_weight_quant_odd_shapes():
    """K not a multiple of 16 takes the scalar-load kernel (the reference accepts any numel)."""
    g = torch.Generator().manual_seed(15)
    w = torch.randn(7, 22, generator=g)
    scale = (127.0 / w.abs().amax(dim=1)).numpy()
    out = torch.empty((7, 22), dtype=torch.uint8, device=DEV)
    ops.quantize_weight(w.to(DEV), out, t(scale), O.Q_INT8)
    assert np.array_equal(out.cpu().numpy().view(np.int8), O.quantize_weight(w.numpy(), scale, O.Q_INT8))
    out4 = torch.empty(77, dtype=torch.uint8, device=DEV)
    ops.quantize_weight(w.to(DEV), out4, 40.0, O.Q_INT4)
    assert np.array_equal(out4.cpu().numpy(), O.quantize_weight(w.numpy(), 40.0, O.Q_INT4))
    un = ops.unpack_int4(out4[:3].clone(), 6)      # tail kernel (fewer than 16 packed bytes)
    assert np.array_equal(un.cpu().numpy(), O.unpack_int4(out4[:3].cpu().numpy(), 6))


# ---------------------------------------------------------------------------------------------
# GEMM: accumulators bit-exact, outputs vs oracle
# ---------------------------------------------------------------------------------------------
def random_operands(kind, M, N, K, seed):
    rng = np.random.default_rng(seed)
    if kind == "f8":
        xq = O.e4m3_encode(rng.standard_normal((M, K)).astype(np.float32) * 30)
        xn = O.e4m3_encode(-np.abs(rng.standard_normal((M, K))).astype(np.float32) * 3)
        wq = O.e4m3_encode(rng.standard_normal((N, K)).astype(np.float32) * 60)
        return xq, xn, wq, wq
    xq = rng.integers(-128, 128, (M, K)).astype(np.int8)
    xn = rng.integers(-128, 1, (M, K)).astype(np.int8)
    if kind == "w4":
        w = rng.integers(-8, 8, (N, K)).astype(np.int8)
        u = (w.astype(np.int16) & 0xF).astype(np.uint8)
        packed = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
        return xq, xn, packed, packed.reshape(-1)
    w = rng.integers(-128, 128, (N, K)).astype(np.int8)
    return xq, xn, w, w


CASES = [
    # kind, M, N, K, bounds, group, dual
    ("i8", 128, 256, 128, None, 0, False),
    ("i8", 1, 16, 32, None, 0, False),                       # smallest legal problem
    ("i8", 130, 300, 1536, [0, 384, 768, 1152, 1536], 0, False),
    ("i8", 200, 264, 1536, [0, 192, 384, 576, 768, 960, 1152, 1344, 1536], 128, False),   # segments straddle groups
    ("i8", 257, 520, 3072, [0, 1024, 3072], 0, True),
    ("i8", 96, 64, 1536, [64 * i for i in range(25)], 0, False),    # 24 segments of 64 (heads x head_dim)
    ("f8", 128, 256, 128, None, 0, False),
    ("f8", 300, 1536, 6144, None, 0, True),
    ("f8", 150, 272, 1024, [0, 256, 1024], 0, False),
    ("w4", 128, 256, 128, None, 128, False),
    ("w4", 260, 528, 3072, [0, 1024, 3072], 128, False),
    ("w4", 140, 256, 1024, None, 128, True),
    ("w4", 64, 96, 512, None, 0, False),                      # int4 weights with per-channel scales only
]


@pytest.mark.parametrize("kind,M,N,K,bounds,group,dual", CASES)
def test_gemm_accumulators_bit_exact_and_output(kind, M, N, K, bounds, group, dual):
    bounds = bounds or [0, K]
    S = len(bounds) - 1
    xq, xn, wq, wq_oracle = random_operands(kind, M, N, K, seed=M + N + K)
    rng = np.random.default_rng(1)
    sx = rng.uniform(0.5, 4.0, S).astype(np.float32)
    sxn = rng.uniform(5.0, 40.0, S).astype(np.float32)
    G = K // group if group else 1
    sw = rng.uniform(50, 150, (G, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    y_ref, acc_ref = O.seg_gemm(KIND[kind][1], xq, wq_oracle, bounds, sx, sw if group else sw[0], xq_neg=xn if dual else None,
                                sx_neg=sxn if dual else None, group_size=group, bias=bias, want_acc=True)
    y, acc = ops.gemm(KIND[kind][0], t(xq.view(np.uint8)).unsqueeze(0), t(wq.view(np.uint8)).unsqueeze(0), N, bounds, t(sx), t(sw),
                      xq_neg=t(xn.view(np.uint8)).unsqueeze(0) if dual else None, sx_neg=t(sxn) if dual else None,
                      group_size=group, sw_strides=(0, 0, N if group else 0, 1), bias=t(bias), out_dtype=torch.float32, want_acc=True)
    acc = acc[0].cpu().numpy()
    assert acc.shape == acc_ref.shape
    if kind == "f8":
        got, want = acc.view(np.float32), acc_ref
        assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()   # fp32 accumulation order differs, nothing else
    else:
        assert np.array_equal(acc, acc_ref), "int32 accumulators must be bit-exact"
    assert max_rel(y[0].cpu().numpy(), y_ref) < 1e-5


def test_gemm_per_token_scales_and_bf16_group_scales():
    M, N, K = 192, 320, 1024
    xq, _, wq, wq_o = random_operands("w4", M, N, K, seed=3)
    rng = np.random.default_rng(2)
    sx = rng.uniform(0.5, 4.0, (1, M)).astype(np.float32)
    sw_bf16 = torch.from_numpy(rng.uniform(50, 150, (K // 128, N)).astype(np.float32)).to(torch.bfloat16)
    y_ref = O.seg_gemm(O.GEMM_W4A8, xq, wq_o, [0, K], sx, sw_bf16.float().numpy(), group_size=128)
    y = ops.gemm(L.SQ_GEMM_W4A8, t(xq.view(np.uint8)).unsqueeze(0), t(wq).unsqueeze(0), N, [0, K], t(sx), sw_bf16.to(DEV),
                 per_token=True, group_size=128, sw_strides=(0, 0, N, 1), out_dtype=torch.float32)
    assert max_rel(y[0].cpu().numpy(), y_ref) < 1e-5


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
def test_gemm_half_outputs_and_unaligned_rows(out_dtype):
    M, N, K = 70, 100, 256                         # N*2 bytes is not a multiple of 16: scalar store path
    xq, _, wq, _ = random_operands("i8", M, N, K, seed=4)
    sx, sw = np.array([2.0], np.float32), np.full(N, 80.0, np.float32)
    y_ref = O.seg_gemm(O.GEMM_I8, xq, wq, [0, K], sx, sw)
    y = ops.gemm(L.SQ_GEMM_W8A8_I8, t(xq.view(np.uint8)).unsqueeze(0), t(wq.view(np.uint8)).unsqueeze(0), N, [0, K], t(sx), t(sw),
                 out_dtype=out_dtype)
    want = torch.from_numpy(y_ref).to(out_dtype).float().numpy()
    got = y[0].float().cpu().numpy()
    assert np.abs(got - want).max() <= np.abs(want).max() * 2.0 ** -8   # at most one rounding step apart


def test_gemm_errors():
    xq = torch.zeros((1, 16, 48), dtype=torch.uint8, device=DEV)
    wq = torch.zeros((1, 16, 48), dtype=torch.uint8, device=DEV)
    one = torch.ones(1, device=DEV)
    with pytest.raises(L.SegQuantError) as e:
        ops.gemm(L.SQ_GEMM_W8A8_I8, xq, wq, 16, [0, 48], one, torch.ones(16, device=DEV))
    assert e.value.status == L.SQ_ERR_ALIGNMENT and "divisible by 32" in str(e.value)
    with pytest.raises(L.SegQuantError):
        ops.gemm(L.SQ_GEMM_W8A8_I8, xq[:, :, :32].contiguous(), wq[:, :, :32].contiguous(), 16, [0, 16, 32], one, torch.ones(16, device=DEV))


# ---------------------------------------------------------------------------------------------
# the reference's pybind contract and the layer
# ---------------------------------------------------------------------------------------------
def test_pybind_contract_against_reference_golden_int8(golden):
    g = golden("input_seg_int8")
    S, seg = 4, int(g["bounds"][1])
    x = t(g["x"])
    wq = torch.empty(g["w"].shape, dtype=torch.int8, device=DEV)
    ops.quantize_weight(t(g["w"]), wq, t(g["sw"][0]), L.SQ_Q_INT8)
    from segquant_b200.layers import ext_dict
    fn = ext_dict["Wint8Aint8"]["gemm_scaled_fn"]
    xin = x.view(-1, S, seg).permute(1, 0, 2)            # the reference's iter_view(): not contiguous
    win = wq.view(-1, S, seg).permute(1, 0, 2)
    out = fn(xin, win, t(g["sx"]), t(g["sw"]))
    assert out.shape == (S, x.shape[0], wq.shape[0]) and out.dtype == torch.float32
    want = O.real_quantized_gemm_scaled("Wint8Aint8", xin.cpu().numpy(), win.cpu().numpy(), g["sx"], g["sw"])
    assert max_rel(out.cpu().numpy(), want) < 1e-5
    y = (out.sum(0) + t(g["b"])).cpu().numpy()
    assert max_rel(y, g["y"]) <= 1e-2 and cosine(y, g["y"]) >= 0.9999      # vs the reference's fake-quant output
    assert max_rel(y, g["y"]) < 1e-5                                        # in fact equal up to fp32 rounding


def test_layer_real_vs_reference_golden(golden):
    cases = [("input_seg_int8", "input", 4, "int8", {"axis": None}, {"axis": 1}),
             ("dual_fp8", "weight", 1, "fpe4m3", {"axis": None, "dual_scale": True}, {"axis": 1}),
             ("weight_seg_dual_int8", "weight", 6, "int8", {"axis": None, "dual_scale": True}, {"axis": None})]
    for name, mode, chunks, qt, ia, wa in cases:
        g = golden(name)
        x, w, b = t(g["x"]), t(g["w"]), t(g["b"])
        lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w,
                            custom_bias_tensor=b, input_quant_type=qt, weight_quant_type=qt,
                            input_quant_args=dict(ia, real_quant=True), weight_quant_args=dict(wa, real_quant=True), device=DEV)
        lin.calibrate(x)
        lin.finish_calibrate()
        y = lin(x).cpu().numpy()
        assert max_rel(y, g["y"]) <= 1e-2 and cosine(y, g["y"]) >= 0.9999, name
        assert max_rel(y, g["y"]) < 2e-5, name
        parts = lin(x, chunked=True)                     # the reference-contract path: un-summed segments
        if mode == "input":
            y2 = (parts.sum(0) + lin.bias_data).cpu().numpy()
        else:
            y2 = (parts.movedim(0, -2).reshape(x.shape[0], -1) + lin.bias_data).cpu().numpy()
        assert max_rel(y2, g["y"]) < 2e-5, name
        # bf16 in, bf16 out: one output rounding away from the fp32 reference result
        lin16 = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w,
                              custom_bias_tensor=b, input_quant_type=qt, weight_quant_type=qt,
                              input_quant_args=dict(ia, real_quant=True), weight_quant_args=dict(wa, real_quant=True), device=DEV)
        lin16.calibrate(x)
        lin16.finish_calibrate()
        xb = x.to(torch.bfloat16)
        yb = lin16(xb)
        assert yb.dtype == torch.bfloat16
        lin_ref = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w.cpu(),
                                custom_bias_tensor=b.cpu(), input_quant_type=qt, weight_quant_type=qt,
                                input_quant_args=dict(ia, real_quant=False), weight_quant_args=dict(wa, real_quant=False), device="cpu")
        lin_ref.calibrate(x.cpu())
        lin_ref.finish_calibrate()
        want = lin_ref(xb.float().cpu()).numpy()
        got = yb.float().cpu().numpy()
        assert max_rel(got, want) <= 1e-2 and cosine(got, want) >= 0.9999, name


def test_layer_w4a8_group128_unequal_segments_and_dynamic():
    """BASELINE config-3 recipe at reduced size: int4 weights (g=128), K-segments 1024 + 2048."""
    g = torch.Generator().manual_seed(2)
    M, K, N = 300, 3072, 768
    x = torch.randn(M, K, generator=g)
    x[:, 1024:] *= 3.0
    w = torch.randn(N, K, generator=g) * 0.02
    xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
    # weights: the bf16 values up-cast to fp32, so that both sides derive identical fp32 scales
    lin = SegmentLinear(K, N, bias=False, seg_mode="input", chunks=2, chunksizes=[1024, 2048], custom_weight_tensor=wb.float().to(DEV),
                        input_quant_type="int8", weight_quant_type="int4", input_quant_args={"real_quant": True, "axis": None},
                        weight_quant_args={"real_quant": True, "axis": 1, "group_size": 128}, device=DEV)
    lin.calibrate(xb.to(DEV))
    lin.finish_calibrate()
    y = lin(xb.to(DEV))
    assert y.dtype == torch.bfloat16 and y.shape == (M, N)
    # oracle: fp32 fake path on the up-cast tensors, group-wise int4 weights from the same definition
    wf, wscale = F.fake_weight_int(wb.float(), 7.0, group_size=128)
    sx = [F.amax_scale(xb.float()[:, :1024], 127.0), F.amax_scale(xb.float()[:, 1024:], 127.0)]
    want = F.seg_linear_fake(xb.float(), wf, None, [0, 1024, 3072], act="int8", sx=sx).numpy()
    got = y.float().cpu().numpy()
    assert max_rel(got, want) <= 1e-2 and cosine(got, want) >= 0.9999
    assert lin.optimizer.weight_manager.packed and lin.optimizer.weight_manager.weight_tensor.shape == (N, K // 2)
    assert torch.allclose(lin.optimizer.scale_tensor[1][0].cpu(), wscale, rtol=1e-6)
    # dynamic per-token activation scales (the W4A8 recipes of the reference use dynamic: true)
    lin_d = SegmentLinear(K, N, bias=False, seg_mode="input", chunks=1, custom_weight_tensor=wb.float().to(DEV),
                          input_quant_type="int8", weight_quant_type="int4",
                          input_quant_args={"real_quant": True, "axis": -1, "dynamic": True},
                          weight_quant_args={"real_quant": True, "axis": 1, "group_size": 128}, device=DEV)
    lin_d.calibrate(xb.to(DEV))
    lin_d.finish_calibrate()
    yd = lin_d(xb.to(DEV)).float().cpu().numpy()
    xs = xb.float()
    s_tok = (127.0 / xb.abs().amax(dim=-1).clamp(min=F.EPS)).float().unsqueeze(1)
    want_d = (torch.clamp(torch.round(xs * s_tok), -128, 127) / s_tok) @ wf.t()
    assert max_rel(yd, want_d.numpy()) <= 1e-2 and cosine(yd, want_d.numpy()) >= 0.9999


# ---------------------------------------------------------------------------------------------
# full-size configurations through size-independent properties
# ---------------------------------------------------------------------------------------------
def test_full_size_config1_int8_segments_properties():
    """BASELINE config 1 (M=4096, K=N=1536, 4 segments): the layer is linear in its integer
    operands, so (a) the summed output equals the sum of four single-segment runs, and (b) the
    int32 accumulators of a row sample are bit-exact against the oracle."""
    g = torch.Generator().manual_seed(0)
    M, K, N, S = 4096, 1536, 1536, 4
    x = torch.randn(M, K, generator=g)
    for s, f in enumerate([0.5, 1.0, 4.0, 16.0]):
        x[:, s * 384:(s + 1) * 384] *= f
    x[:, torch.randperm(K, generator=g)[:30]] *= 20.0
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    bounds = [0, 384, 768, 1152, 1536]
    sx = np.array([127.0 / x[:, bounds[s]:bounds[s + 1]].abs().max().item() for s in range(S)], np.float32)
    sw = (127.0 / w.abs().amax(dim=1)).numpy()
    wq = torch.empty((N, K), dtype=torch.int8, device=DEV)
    ops.quantize_weight(w.to(DEV), wq, t(sw), L.SQ_Q_INT8)
    xq, _ = ops.quantize_act(x.to(DEV), bounds, t(sx), None, L.SQ_Q_INT8)
    y = ops.gemm(L.SQ_GEMM_W8A8_I8, xq, wq.view(torch.uint8).unsqueeze(0), N, bounds, t(sx), t(sw), bias=t(b.numpy()))[0]
    total = torch.zeros_like(y)
    for s in range(S):
        xs = torch.zeros_like(xq)
        xs[:, :, bounds[s]:bounds[s + 1]] = xq[:, :, bounds[s]:bounds[s + 1]]
        total += ops.gemm(L.SQ_GEMM_W8A8_I8, xs, wq.view(torch.uint8).unsqueeze(0), N, bounds, t(sx), t(sw))[0]
    total += t(b.numpy())
    assert torch.allclose(y, total, rtol=1e-5, atol=1e-5)
    rows = slice(1000, 1064)
    y_ref, acc_ref = O.seg_gemm(O.GEMM_I8, xq[0, rows].cpu().numpy().view(np.int8), wq.cpu().numpy(), bounds, sx, sw, bias=b.numpy(), want_acc=True)
    _, acc = ops.gemm(L.SQ_GEMM_W8A8_I8, xq[:, rows].contiguous(), wq.view(torch.uint8).unsqueeze(0), N, bounds, t(sx), t(sw), want_acc=True)
    assert np.array_equal(acc[0].cpu().numpy(), acc_ref)
    assert max_rel(y[rows].cpu().numpy(), y_ref) < 1e-5
    want = F.seg_linear_fake(x, F.fake_weight_int(w, 127.0)[0], b, bounds, act="int8", sx=[float(s) for s in sx]).numpy()
    assert max_rel(y.cpu().numpy(), want) <= 1e-2 and cosine(y.cpu().numpy(), want) >= 0.9999


def test_full_size_config2_dual_fp8_properties():
    """BASELINE config 2 (M=4096, K=6144, N=1536, DualScale FP8 after GELU): the positive and the
    negative activation tensors have disjoint support; the dual output equals the sum of the two
    single-sided runs; output within tolerance of the fp32 fake-quant path."""
    g = torch.Generator().manual_seed(1)
    M, K, N = 4096, 6144, 1536
    x = torch.nn.functional.gelu(torch.randn(M, K, generator=g).to(torch.bfloat16).float()).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(N, generator=g) * 0.01).to(torch.bfloat16)
    # weights: bf16 values up-cast to fp32 so that the layer and the oracle derive the same fp32 scales
    lin = SegmentLinear(K, N, bias=True, seg_mode="weight", chunks=1, custom_weight_tensor=w.float().to(DEV), custom_bias_tensor=b.to(DEV),
                        input_quant_type="fpe4m3", weight_quant_type="fpe4m3",
                        input_quant_args={"real_quant": True, "axis": None, "dual_scale": True},
                        weight_quant_args={"real_quant": True, "axis": 1}, device=DEV)
    xd = x.to(DEV)
    lin.calibrate(xd)
    lin.finish_calibrate()
    y = lin(xd)
    f = lin.optimizer._fused
    assert 50 < f["sx"].item() < 150 and 1500 < f["sx_neg"].item() < 4000      # GELU: negatives live in [-0.17, 0]
    xq, xqn = ops.quantize_act(xd, [0, K], f["sx"], f["sx_neg"], L.SQ_Q_E4M3)
    assert not bool(((xq & 0x7F) != 0).logical_and((xqn & 0x7F) != 0).any())
    kw = dict(sw_strides=f["sw_strides"], out_dtype=torch.float32)
    yp = ops.gemm(L.SQ_GEMM_W8A8_F8, xq, f["wq"], N, [0, K], f["sx"], f["sw"], **kw)[0]
    yn = ops.gemm(L.SQ_GEMM_W8A8_F8, xqn, f["wq"], N, [0, K], f["sx_neg"], f["sw"], **kw)[0]
    yd = ops.gemm(L.SQ_GEMM_W8A8_F8, xq, f["wq"], N, [0, K], f["sx"], f["sw"], xq_neg=xqn, sx_neg=f["sx_neg"], **kw)[0]
    assert torch.allclose(yd, yp + yn, rtol=1e-4, atol=1e-5)
    wf, _ = F.fake_weight_fp8(w.float())
    sp, sn = F.dual_scales(x.float(), 448.0, 448.0)
    want = F.seg_linear_fake(x.float(), wf, b.float(), [0, K], act="fp8", sx_pos=[sp], sx_neg=[sn]).numpy()
    got = y.float().cpu().numpy()
    assert max_rel(got, want) <= 1e-2 and cosine(got, want) >= 0.9999


@pytest.mark.parametrize("name,mode,chunks", [("smooth_input_seg_int8", "input", 4), ("smooth_weight_seg_int8", "weight", 2)])
def test_smooth_optimizer_real_path_vs_reference_golden(golden, name, mode, chunks):
    """SmoothOptimizer on the real-quant path: the division by s runs inside the activation-quantise kernel, K-segments
    take one GEMM with per-(segment, column) weight scales, N-segments one GEMM per chunk writing its columns in place."""
    from segquant_b200.layers.SegmentLinear import SegmentLinear
    g = golden(name)
    x, w, b = (torch.from_numpy(g[k]).to(DEV) for k in "xwb")
    lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w,
                        custom_bias_tensor=b, input_quant_type="int8", weight_quant_type="int8",
                        input_quant_args={"real_quant": True, "axis": None}, weight_quant_args={"real_quant": True, "axis": 1},
                        opt_type="smooth", opt_kwargs={"alpha": 0.5}, device=DEV)
    lin.trace(x)
    lin.smooth()
    lin.calibrate(x)
    lin.finish_calibrate()
    assert np.allclose(torch.stack(lin.optimizer.s).cpu().numpy(), g["s"], rtol=1e-6)
    sx, sw = lin.optimizer.scale_tensor
    assert np.allclose(sx.cpu().numpy(), g["sx"], rtol=1e-6) and np.allclose(sw.cpu().numpy(), g["sw"], rtol=1e-6)
    x0 = x.clone()
    y = lin(x).cpu().numpy()
    assert torch.equal(x, x0)
    want = g["y"]
    assert max_rel(y, want) <= 1e-2                     # stated tolerance against the reference's fake-quant output
    cos = float((y * want).sum() / (np.linalg.norm(y) * np.linalg.norm(want)))
    assert cos >= 0.9999
    # the un-summed reference contract gives the same numbers
    parts = lin(x, chunked=True)
    y2 = (parts.sum(0) if mode == "input" else parts.movedim(0, -2).reshape(x.shape[0], -1)) + lin.bias_data
    assert max_rel(y2.cpu().numpy(), y) <= 1e-5
    assert ops.device_status() == 0


# ---------------------------------------------------------------------------------------------
# skinny-M path (M <= 4): CUDA-core weight streaming, same arithmetic as the tensor-core kernels
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind,M,N,K,bounds,group,dual,per_token", [
    ("i8", 2, 9216, 1536, None, 0, True, False),            # the adaLN projection of the MMDiT step
    ("i8", 1, 50, 96, None, 0, False, False),               # N not a multiple of the 4 columns a warp owns
    ("i8", 3, 260, 1024, [0, 256, 1024], 0, False, False),  # unequal segments
    ("i8", 4, 128, 1024, None, 128, False, True),           # groups of 128 + per-token activation scales
    ("i8", 4, 96, 3072, [0, 1024, 2048, 3072], 512, True, False),
    ("f8", 2, 300, 1536, None, 0, True, False),
    ("f8", 3, 64, 512, [0, 256, 512], 0, False, True),
])
def test_skinny_m_path_matches_oracle_and_tensor_core_path(kind, M, N, K, bounds, group, dual, per_token):
    gk = {"i8": L.SQ_GEMM_W8A8_I8, "f8": L.SQ_GEMM_W8A8_F8}[kind]
    ok = {"i8": O.GEMM_I8, "f8": O.GEMM_F8}[kind]
    xq, xn, wq, _ = random_operands(kind, M, N, K, seed=11)
    bounds = bounds or [0, K]
    S = len(bounds) - 1
    rng = np.random.default_rng(5)
    sx = rng.uniform(0.5, 4.0, (S, M) if per_token else (S,)).astype(np.float32)
    sxn = rng.uniform(0.5, 4.0, (S, M) if per_token else (S,)).astype(np.float32)
    if group:
        sw = rng.uniform(50, 150, (K // group, N)).astype(np.float32)
        strides = (0, 0, N, 1)
    else:
        sw = rng.uniform(50, 150, (S, N)).astype(np.float32)
        strides = (0, N, 0, 1)
    bias = rng.standard_normal(N).astype(np.float32)
    y_ref = O.seg_gemm(ok, xq, wq, bounds, sx, sw, xq_neg=xn if dual else None, sx_neg=sxn if dual else None, group_size=group, bias=bias)

    def run():
        return ops.gemm(gk, t(xq.view(np.uint8)).unsqueeze(0), t(wq.view(np.uint8)).unsqueeze(0), N, bounds, t(sx), t(sw),
                        xq_neg=t(xn.view(np.uint8)).unsqueeze(0) if dual else None, sx_neg=t(sxn) if dual else None, per_token=per_token,
                        group_size=group, sw_strides=strides, bias=t(bias), out_dtype=torch.float32)[0].cpu().numpy()

    y_skinny = run()
    ops.set_gemm_schedule(no_gemv=1)
    try:
        y_tc = run()
    finally:
        ops.set_gemm_schedule()
    assert max_rel(y_skinny, y_ref) < 1e-5
    assert max_rel(y_tc, y_ref) < 1e-5
    if kind == "i8":
        assert np.array_equal(y_skinny, y_tc)     # integer sums are exact on both paths and the fp32 steps are the same
    assert ops.device_status() == 0


# ---------------------------------------------------------------------------------------------
# BASELINE config 3 at its stated shapes: W4A8, int4 weights with bf16 group scales (g = 128)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,N,K,bounds,dual", [
    ("qkv", 9216, 3072, [0, 1024, 3072], False),
    ("mlp_up", 12288, 3072, [0, 1024, 3072], False),
    ("mlp_down", 3072, 12288, [0, 12288], True),
])
def test_full_size_config3_w4a8_projections(name, N, K, bounds, dual):
    """M = 4608 (4096 image + 512 text tokens), X bf16 with K-segments 0:1024 ~ N(0,1) and 1024:3072 ~ N(0,3) (QKV, MLP up) or
    X = SiLU(N(0,1)) with DualScale (MLP down); weights signed int4 packed two per byte, bf16 group scales of 128 along K;
    int8 activations, static per segment.  Checks: packed weight bytes and activation bytes of a row sample equal the C
    oracle's; the fp32 output of 256 rows spread over eight M-tiles (all N columns) within 1e-5 of the oracle's; the whole
    bf16 output against the fp32 fake-quant path (oracle/fake_path.py arithmetic, evaluated with torch on the GPU):
    max rel err <= 1e-2 and cosine >= 0.9999."""
    g = torch.Generator().manual_seed(2)
    M, G = 4608, 128
    S = len(bounds) - 1
    if dual:
        x = torch.nn.functional.silu(torch.randn(M, K, generator=g)).to(torch.bfloat16)
    else:
        x = torch.randn(M, K, generator=g)
        x[:, 1024:] *= 3.0
        x = x.to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    xd, wd = x.to(DEV), w.to(DEV)
    # weights: group scales 7 / amax, kept in bf16 (what the kernel's epilogue reads), packed by the native kernel
    sw16 = (7.0 / wd.float().view(N, K // G, G).abs().amax(-1)).to(torch.bfloat16).contiguous()            # (N, K/G)
    sw32 = sw16.float().contiguous()
    wq = torch.empty(N * K // 2, dtype=torch.uint8, device=DEV)
    ops.quantize_weight(wd, wq, sw32, L.SQ_Q_INT4, group_size=G)
    nrows = 64
    want_w = O.quantize_weight(w[:nrows].float().numpy(), sw32[:nrows].cpu().numpy(), O.Q_INT4, group_size=G)
    assert np.array_equal(wq[:nrows * K // 2].cpu().numpy(), want_w.reshape(-1))
    # activations
    xf = xd.float()
    if dual:
        sp, sn = F.dual_scales(x.float(), 127.0, 128.0)
        sx, sxn = np.array([sp], np.float32), np.array([sn], np.float32)
    else:
        sx = np.array([127.0 / xf[:, bounds[s]:bounds[s + 1]].abs().max().item() for s in range(S)], np.float32)
        sxn = None
    xq, xqn = ops.quantize_act(xd, bounds, t(sx), t(sxn) if dual else None, L.SQ_Q_INT8)
    rows = np.concatenate([np.arange(r0, r0 + 32) for r0 in (0, 577, 1154, 1731, 2308, 2885, 3462, M - 32)])
    rows_t = torch.from_numpy(rows).to(DEV)
    want_x = O.quantize_act(x[rows].float().numpy(), bounds, sx, sx_neg=sxn, out_kind=O.Q_INT8)
    if dual:
        assert np.array_equal(xq[0, rows_t].cpu().numpy().view(np.int8), want_x[0]) and np.array_equal(xqn[0, rows_t].cpu().numpy().view(np.int8), want_x[1])
    else:
        assert np.array_equal(xq[0, rows_t].cpu().numpy().view(np.int8), want_x)
    kw = dict(xq_neg=xqn, sx_neg=t(sxn) if dual else None, group_size=G, sw_strides=(0, 0, 1, K // G))
    wq3 = wq.view(1, N, K // 2)
    y32 = ops.gemm(L.SQ_GEMM_W4A8, xq, wq3, N, bounds, t(sx), sw16, out_dtype=torch.float32, **kw)[0]
    y16 = ops.gemm(L.SQ_GEMM_W4A8, xq, wq3, N, bounds, t(sx), sw16, out_dtype=torch.bfloat16, **kw)[0]
    assert torch.equal(y16, y32.to(torch.bfloat16))
    # (1) row sample against the C oracle, on the very bytes the kernel consumed
    xq_rows = (want_x[0] if dual else want_x)
    y_ref = O.seg_gemm(O.GEMM_W4A8, xq_rows, wq.cpu().numpy(), bounds, sx, sw32.t().contiguous().cpu().numpy(),
                       xq_neg=want_x[1] if dual else None, sx_neg=sxn, group_size=G)
    assert max_rel(y32[rows_t].cpu().numpy(), y_ref) < 1e-5, name
    # (2) whole output against the fp32 fake-quant path
    torch.backends.cuda.matmul.allow_tf32 = False
    sw_g = sw32.unsqueeze(-1)
    w_fake = (torch.clamp(torch.round(wd.float().view(N, K // G, G) * sw_g), -8, 7) / sw_g).view(N, K)
    if dual:
        want = F.seg_linear_fake(xf, w_fake, None, bounds, act="int8", sx_pos=[float(sx[0])], sx_neg=[float(sxn[0])])
    else:
        want = F.seg_linear_fake(xf, w_fake, None, bounds, act="int8", sx=[float(v) for v in sx])
    got, want = y16.float().cpu().numpy(), want.cpu().numpy()
    assert max_rel(got, want) <= 1e-2 and cosine(got, want) >= 0.9999, (name, max_rel(got, want), cosine(got, want))
    assert ops.device_status() == 0
