"""CPU: the oracle (oracle/) against the fixtures produced by the reference's own code
(tests/golden/make_golden.py).  These tests pin the checker, they do not touch the product."""
import numpy as np
import pytest
import torch

from oracle import fake_path as F
from oracle import oracle as O


def rel_fro(a, b):
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def cosine(a, b):
    a, b = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def test_e4m3_roundtrip_matches_reference_extension(golden):
    g = golden("quantizers")
    got = O.e4m3_roundtrip(g["e4m3_grid"])
    assert np.array_equal(got, g["e4m3_roundtrip"])


def test_e4m3_encode_all_codes_roundtrip():
    codes = np.arange(256, dtype=np.uint8)
    vals = O.e4m3_decode(codes)
    finite = ~np.isnan(vals)
    back = O.e4m3_encode(vals[finite])
    assert np.array_equal(back, codes[finite])
    # saturation and ties-to-even
    assert O.e4m3_encode(np.array([1e9, -1e9, 448.0, 464.0, 465.0], np.float32)).tolist() == [0x7E, 0xFE, 0x7E, 0x7E, 0x7E]
    assert O.e4m3_encode(np.array([17.0, 19.0], np.float32)).tolist() == O.e4m3_encode(np.array([16.0, 20.0], np.float32)).tolist()


def test_e4m3_matches_torch_cast():
    g = torch.Generator().manual_seed(5)
    x = torch.cat([torch.randn(50000, generator=g) * 50, torch.randn(50000, generator=g) * 0.01])
    want = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x.numpy()), want)


def test_scale_definitions(golden):
    g = golden("quantizers")
    assert np.isclose(O.calibrate_sym(g["int8_x"], 127.0), g["int8_scale"], rtol=1e-6)
    assert np.allclose(O.calibrate_sym(g["int8_x"], 127.0, axis=1), g["int8_axis1_scale"], rtol=1e-6)
    pos, neg = O.calibrate_dual(g["dual_x"], 127.0, 128.0)
    assert np.isclose(pos, g["dual_int8_pos"], rtol=1e-6) and np.isclose(neg, g["dual_int8_neg"], rtol=1e-6)
    pos, neg = O.calibrate_dual(g["dual_x"], 448.0, 448.0)
    assert np.isclose(pos, g["dual_fp8_pos"], rtol=1e-6) and np.isclose(neg, g["dual_fp8_neg"], rtol=1e-6)
    assert np.isclose(O.calibrate_sym(g["int8_x"], 448.0), g["fp8_scale"], rtol=1e-6)


def test_int8_quantise_then_dequantise_equals_reference_fake(golden):
    g = golden("quantizers")
    x, s = g["int8_x"], float(g["int8_scale"])
    q = O.quantize_act(x, [0, x.shape[1]], [s], out_kind=O.Q_INT8)
    assert q.dtype == np.int8
    assert np.array_equal((q.astype(np.float32) / np.float32(s)), g["int8_fake"])


def test_dual_int8_and_fp8_quantise_equal_reference_fake(golden):
    g = golden("quantizers")
    x = g["dual_x"]
    K = x.shape[1]
    qp, qn = O.quantize_act(x, [0, K], [float(g["dual_int8_pos"])], sx_neg=[float(g["dual_int8_neg"])], out_kind=O.Q_INT8)
    deq = qp.astype(np.float32) / np.float32(g["dual_int8_pos"]) + qn.astype(np.float32) / np.float32(g["dual_int8_neg"])
    assert np.allclose(deq, g["dual_int8_fake"], rtol=0, atol=1e-7)
    assert not np.any((qp != 0) & (qn != 0)), "an element may live on one side only"
    qp, qn = O.quantize_act(x, [0, K], [float(g["dual_fp8_pos"])], sx_neg=[float(g["dual_fp8_neg"])], out_kind=O.Q_E4M3)
    deq = O.e4m3_decode(qp) / np.float32(g["dual_fp8_pos"]) + O.e4m3_decode(qn) / np.float32(g["dual_fp8_neg"])
    assert np.allclose(deq, g["dual_fp8_fake"], rtol=0, atol=1e-7)


def test_int4_group_weights_and_packing(golden):
    g = golden("quantizers")
    w, scale = g["int4_w"], g["int4_group_scale"]          # scale (N, K/128)
    packed = O.quantize_weight(w, scale, O.Q_INT4, group_size=128)
    assert packed.dtype == np.uint8 and packed.size == w.size // 2
    vals = O.unpack_int4(packed, w.size).reshape(w.shape).astype(np.float32)
    assert vals.min() >= -8 and vals.max() <= 7
    deq = vals / np.repeat(scale, 128, axis=1)
    assert np.allclose(deq, g["int4_group_fake"], rtol=0, atol=1e-7)
    # nibble order: element 2j in the low nibble
    first = O.unpack_int4(packed[:1], 2)
    assert first[0] == vals.reshape(-1)[0] and first[1] == vals.reshape(-1)[1]
    assert (packed[0] & 0xF) == (int(vals.reshape(-1)[0]) & 0xF)


def test_dynamic_per_token_scales(golden):
    g = golden("quantizers")
    x = torch.from_numpy(g["int8_x"])
    s = F.amax_scale(x, 127.0, axis=-1)
    assert np.allclose(s.numpy(), g["dyn_scale"], rtol=1e-6)
    sb = F.amax_scale(x.to(torch.bfloat16), 127.0, axis=-1)
    assert sb.dtype == torch.bfloat16 and np.array_equal(sb.float().numpy(), g["dyn_scale_bf16"])
    q = O.quantize_act(g["int8_x"], [0, x.shape[1]], s.numpy().reshape(1, -1), out_kind=O.Q_INT8)
    assert np.allclose(q.astype(np.float32) / s.numpy()[:, None], g["dyn_fake"], rtol=0, atol=1e-6)


def test_real_path_restatement_vs_reference_layer_int8(golden):
    g = golden("input_seg_int8")
    bounds = g["bounds"].tolist()
    wq = O.quantize_weight(g["w"], g["sw"][0], O.Q_INT8)
    assert np.allclose(wq.astype(np.float32) / g["sw"][0][:, None], g["w_fake"], rtol=0, atol=1e-8)
    xq = O.quantize_act(g["x"], bounds, g["sx"], out_kind=O.Q_INT8)
    y, acc = O.seg_gemm(O.GEMM_I8, xq, wq, bounds, g["sx"], g["sw"], bias=g["b"], want_acc=True)
    assert acc.shape[0] == 4 and np.abs(acc).max() < 2 ** 24
    assert rel_fro(y, g["y"]) < 2e-6 and cosine(y, g["y"]) > 0.999999
    # the pybind-contract form: (S, M, K/S) inputs, (S, N, K/S) weights, un-summed outputs
    S, seg = 4, bounds[1]
    xin = g["x"].reshape(-1, S, seg).transpose(1, 0, 2)
    win = wq.reshape(-1, S, seg).transpose(1, 0, 2)
    parts = O.real_quantized_gemm_scaled("Wint8Aint8", xin, win, g["sx"], g["sw"])
    assert parts.shape == (S, g["x"].shape[0], wq.shape[0])
    assert np.allclose(parts.sum(0) + g["b"], y, rtol=1e-6, atol=1e-6)


def test_real_path_restatement_vs_reference_layer_dual_fp8(golden):
    g = golden("dual_fp8")
    K = g["x"].shape[1]
    wq = O.quantize_weight(g["w"], g["sw"][0], O.Q_E4M3)
    xp, xn = O.quantize_act(g["x"], [0, K], g["sx_pos"], sx_neg=g["sx_neg"], out_kind=O.Q_E4M3)
    y = O.seg_gemm(O.GEMM_F8, xp, wq, [0, K], g["sx_pos"], g["sw"][0], xq_neg=xn, sx_neg=g["sx_neg"], bias=g["b"])
    assert rel_fro(y, g["y"]) < 2e-6 and cosine(y, g["y"]) > 0.999999


def test_real_path_restatement_vs_reference_layer_weight_seg_dual(golden):
    g = golden("weight_seg_dual_int8")
    S = int(g["chunks"])
    N, K = g["w"].shape
    per = N // S
    outs = []
    for s in range(S):
        wq = O.quantize_weight(g["w"][s * per:(s + 1) * per], float(g["sw"][s]), O.Q_INT8)
        xp, xn = O.quantize_act(g["x"], [0, K], g["sx_pos"][s:s + 1], sx_neg=g["sx_neg"][s:s + 1], out_kind=O.Q_INT8)
        outs.append(O.seg_gemm(O.GEMM_I8, xp, wq, [0, K], g["sx_pos"][s:s + 1], np.full(per, g["sw"][s], np.float32),
                               xq_neg=xn, sx_neg=g["sx_neg"][s:s + 1]))
    y = np.concatenate(outs, axis=1) + g["b"]
    assert rel_fro(y, g["y"]) < 2e-6


def test_fake_path_port_equals_reference_layer(golden):
    g = golden("input_seg_int8")
    x, wf, b = (torch.from_numpy(g[k]) for k in ("x", "w_fake", "b"))
    y = F.seg_linear_fake(x, wf, b, g["bounds"].tolist(), act="int8", sx=[float(s) for s in g["sx"]])
    assert torch.allclose(y, torch.from_numpy(g["y"]), rtol=1e-6, atol=1e-6)
    g = golden("dual_fp8")
    x, w, b = (torch.from_numpy(g[k]) for k in ("x", "w", "b"))
    wf, sw = F.fake_weight_fp8(w)
    assert np.allclose(sw.numpy(), g["sw"][0], rtol=1e-6) and np.allclose(wf.numpy(), g["w_fake"], atol=1e-8)
    sp, sn = F.dual_scales(x, 448.0, 448.0)
    assert np.isclose(sp, g["sx_pos"][0], rtol=1e-6) and np.isclose(sn, g["sx_neg"][0], rtol=1e-6)
    y = F.seg_linear_fake(x, wf, b, [0, x.shape[1]], act="fp8", sx_pos=[sp], sx_neg=[sn])
    assert torch.allclose(y, torch.from_numpy(g["y"]), rtol=1e-5, atol=1e-6)


def test_group_and_segment_units_cross():
    """K=384 cut into 2 segments of 192 and weight groups of 128: 4 accumulation units."""
    rng = np.random.default_rng(0)
    xq = rng.integers(-128, 128, (8, 384)).astype(np.int8)
    wq = rng.integers(-128, 128, (16, 384)).astype(np.int8)
    sw = rng.uniform(1, 2, (3, 16)).astype(np.float32)
    y, acc = O.seg_gemm(O.GEMM_I8, xq, wq, [0, 192, 384], [2.0, 3.0], sw, group_size=128, want_acc=True)
    assert acc.shape[0] == 4
    cuts = [(0, 128, 0, 0), (128, 192, 0, 1), (192, 256, 1, 1), (256, 384, 1, 2)]
    want = np.zeros((8, 16), np.float64)
    for u, (a, b_, s, gi) in enumerate(cuts):
        ref = xq[:, a:b_].astype(np.int64) @ wq[:, a:b_].astype(np.int64).T
        assert np.array_equal(acc[u, 0], ref)
        want += ref / (np.float64([2.0, 3.0][s]) * sw[gi].astype(np.float64))
    assert np.allclose(y, want, rtol=1e-5, atol=1e-2)  # fp32 sums of 4 units of magnitude 1e4-1e5
