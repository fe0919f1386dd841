"""GPU tests of the pieces the synthetic MMDiT step adds on top of the layer: writing a layer's output into a slice of
a joint token buffer (out=), and the quantised step against its own fp32 calibration pass."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(K, N, kind, dual, seed):
    from segquant_b200.mmdit import QLinear
    g = torch.Generator().manual_seed(seed)
    q = "int8" if kind == "Wint8Aint8" else "fpe4m3"
    return QLinear(K, N, g, "cuda", torch.bfloat16, dual=dual, act=q, wq=q)


@pytest.mark.parametrize("kind", ["Wint8Aint8", "Wfpe4m3Afpe4m3"])
@pytest.mark.parametrize("dual", [False, True])
def test_out_slice_matches_plain_forward(kind, dual):
    torch.manual_seed(3)
    B, T1, T2, K, N = 2, 320, 77, 256, 384
    lay = _layer(K, N, kind, dual, 5)
    x1 = torch.randn(B, T1, K, device="cuda", dtype=torch.bfloat16)
    x2 = torch.randn(B, T2, K, device="cuda", dtype=torch.bfloat16)
    lay.calibrate_forward(x1)
    lay.finish()
    joint = torch.full((B, T1 + T2, N), 7.0, device="cuda", dtype=torch.bfloat16)
    lay(x1, out=joint[:, :T1])
    assert torch.equal(joint[:, :T1], lay(x1))
    assert torch.all(joint[:, T1:] == 7.0)          # rows outside the slice are untouched
    lay(x2, out=joint[:, T1:])
    assert torch.equal(joint[:, T1:], lay(x2))
    assert torch.equal(joint[:, :T1], lay(x1))


def test_small_step_close_to_calibration_pass():
    from segquant_b200.mmdit import SyntheticMMDiT, synthetic_inputs
    model = SyntheticMMDiT("cuda", blocks=2, hidden=256, heads=4, img_tokens=256, txt_tokens=40, seed=0)
    inp = synthetic_inputs(2, "cuda", img_tokens=256, txt_tokens=40, hidden=256, seed=1)
    ref = model.calibrate(*inp)
    out = model(*inp)
    assert out.shape == ref.shape
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), ref.float().flatten(), dim=0)
    assert cos > 0.99
    from segquant_b200 import ops
    assert ops.device_status() == 0


def _ref_norm_quant(x, shift, scale, bounds, sx, sx_neg, kind):
    """fp32 restatement of the fused kernel: LayerNorm (eps 1e-6, biased variance), modulation, static quantise."""
    from segquant_b200 import ops
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(-1, keepdim=True)
    n = (xf - mean) / torch.sqrt(var + 1e-6)
    if shift is not None:
        n = n * (1 + scale.float().unsqueeze(1)) + shift.float().unsqueeze(1)
    B, T, K = x.shape
    q, qn = ops.quantize_act(n.reshape(B * T, K).contiguous(), bounds, sx, sx_neg, out_kind=kind)
    return q.view(B, T, K), None if qn is None else qn.view(B, T, K)


def _as_values(q, kind):
    from segquant_b200 import _lib as L
    return q.view(torch.int8).float() if kind == L.SQ_Q_INT8 else q.view(torch.float8_e4m3fn).float()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("kind_name", ["int8", "e4m3"])
@pytest.mark.parametrize("dual,mod,segs", [(False, True, 1), (True, True, 3), (False, False, 2)])
def test_norm_quantize_act_matches_unfused(dtype, kind_name, dual, mod, segs):
    from segquant_b200 import _lib as L, ops
    kind = L.SQ_Q_INT8 if kind_name == "int8" else L.SQ_Q_E4M3
    torch.manual_seed(11)
    B, T, K = 2, 77, 1024 if dtype == torch.float32 else 1536
    x = (torch.randn(B, T, K, device="cuda") * 3 + 0.5).to(dtype)
    modt = (torch.randn(B, 6 * K, device="cuda") * 0.3).to(dtype)          # shift / scale are strided views, as in a block
    shift, scale = (modt[:, :K], modt[:, K:2 * K]) if mod else (None, None)
    bounds = [0, K] if segs == 1 else ([0, K // 2, K] if segs == 2 else [0, 256, 768, K])
    qmax = 127.0 if kind == L.SQ_Q_INT8 else 448.0
    sx = (torch.rand(segs, device="cuda") * 2 + 3) / qmax
    sxn = (torch.rand(segs, device="cuda") * 2 + 2) / qmax if dual else None
    q, qn = ops.norm_quantize_act(x, bounds, sx, sxn, out_kind=kind, shift=shift, scale=scale)
    rq, rqn = _ref_norm_quant(x, shift, scale, bounds, sx, sxn, kind)
    for got, want in ((q, rq), (qn, rqn)):
        if want is None:
            assert got is None
            continue
        # both sides round the same fp32 value up to the last ulp of the normalisation, so a value that sits on a
        # rounding boundary may land on the neighbouring code: allow that for a small fraction, and nothing larger
        diff = got != want
        assert diff.float().mean() < 2e-3
        g, w = _as_values(got, kind)[diff], _as_values(want, kind)[diff]
        if kind == L.SQ_Q_INT8:
            assert torch.all((g - w).abs() <= 1)
        else:
            assert torch.all((g - w).abs() <= 0.126 * torch.maximum(g.abs(), w.abs()) + 2 ** -9)
    assert ops.device_status() == 0


def test_norm_quantize_act_rejects_long_rows():
    from segquant_b200 import ops
    x = torch.randn(1, 4, 4096, device="cuda", dtype=torch.bfloat16)
    sx = torch.ones(1, device="cuda")
    with pytest.raises(Exception):
        ops.norm_quantize_act(x, [0, 4096], sx)


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("kind_name,dual", [("int8", True), ("e4m3", True), ("int8", False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quantize_act_with_fused_activation(act, kind_name, dual, dtype):
    """quantize_act(pre_act=...) against the activation evaluated by torch in fp32 followed by the plain quantise
    kernel: the hardware exp2 / reciprocal approximations move a value by about 2^-22 of itself, so a very small
    fraction of codes may land on the neighbouring step, none further."""
    from segquant_b200 import _lib as L, ops
    kind = L.SQ_Q_INT8 if kind_name == "int8" else L.SQ_Q_E4M3
    torch.manual_seed(5)
    B, T, K = 2, 130, 1024
    x = (torch.randn(B, T, K, device="cuda") * 2.5).to(dtype)
    fn = (lambda t: torch.nn.functional.gelu(t, approximate="tanh")) if act == "gelu_tanh" else torch.nn.functional.silu
    y = fn(x.float())
    qmax = 127.0 if kind == L.SQ_Q_INT8 else 448.0
    bounds = [0, 512, K]
    sx = qmax / torch.stack([y[..., :512].max(), y[..., 512:].max()])
    sxn = (qmax / torch.stack([y[..., :512].min().abs(), y[..., 512:].min().abs()])) if dual else None
    q, qn = ops.quantize_act(x, bounds, sx, sxn, kind, shared_scales=True, pre_act=act)
    rq, rqn = ops.quantize_act(y, bounds, sx, sxn, kind, shared_scales=True)
    for got, want in ((q, rq), (qn, rqn)):
        if want is None:
            assert got is None
            continue
        gv, wv = _as_values(got, kind), _as_values(want, kind)
        diff = gv != wv                                  # by value: an e4m3 -0 (a tiny negative input) equals +0
        assert diff.float().mean() < 0.005
        g, w = gv[diff], wv[diff]
        if kind == L.SQ_Q_INT8:
            assert torch.all((g - w).abs() <= 1)
        else:
            assert torch.all((g - w).abs() <= 0.126 * torch.maximum(g.abs(), w.abs()) + 2 ** -9)
    with pytest.raises(Exception):      # a fused activation cannot be combined with the smoothing vector
        ops.quantize_act(x, bounds, sx, sxn, kind, shared_scales=True, pre_act=act, smooth=torch.ones(K, device="cuda"))
    assert ops.device_status() == 0


def test_fused_norm_step_matches_unfused_step():
    """The step with one normalise + modulate + quantise kernel per norm and the GELU / SiLU evaluated inside the
    quantise kernel, against the same model running torch's layer_norm, modulation and activations in bf16 followed
    by the plain quantise kernel: same weights and scales, so the only difference is that the fused kernels do not
    round the intermediate tensor to bf16 before quantising."""
    from segquant_b200.mmdit import SyntheticMMDiT, synthetic_inputs
    model = SyntheticMMDiT("cuda", blocks=2, hidden=256, heads=4, img_tokens=256, txt_tokens=40, seed=0)
    inp = synthetic_inputs(2, "cuda", img_tokens=256, txt_tokens=40, hidden=256, seed=1)
    model.calibrate(*inp)
    fused = model(*inp).float()
    assert any(v is not None for v in model.fused_norm.plan.values())       # the fused kernel really ran
    assert any(isinstance(k, tuple) and k and k[0] == "merged" and v is not None for k, v in model.fused_norm.plan.items())
    model.fused_norm.merge_gemms = False        # q / k / v as three GEMMs instead of one: integer accumulation, same epilogue
    separate = model(*inp).float()
    model.fused_norm.merge_gemms = True
    assert torch.equal(fused, separate)
    model.fused_norm.fuse_residual = False      # gated residual as its own kernel: same arithmetic, same roundings
    separate = model(*inp).float()
    model.fused_norm.fuse_residual = True
    assert torch.equal(fused, separate)
    from segquant_b200.mmdit import QLinear
    keep, model.fused_norm = model.fused_norm, None
    QLinear.fuse_activation = False
    try:
        plain = model(*inp).float()
    finally:
        model.fused_norm = keep
        QLinear.fuse_activation = True
    cos = torch.nn.functional.cosine_similarity(fused.flatten(), plain.flatten(), dim=0)
    assert cos > 0.999
    from segquant_b200 import ops
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gated_residual_is_bit_identical_to_addcmul(dtype):
    from segquant_b200 import ops
    torch.manual_seed(2)
    B, T, K = 2, 333, 1536
    x = torch.randn(B, T, K, device="cuda").to(dtype)
    y = (torch.randn(B, T + 5, K, device="cuda") * 3).to(dtype)[:, 5:]          # a token slice: batch stride != T * K
    mod = torch.randn(B, 6 * K, device="cuda").to(dtype)
    gate = mod[:, 2 * K:3 * K]                                                  # a chunk of the modulation, read in place
    want = torch.addcmul(x, gate.unsqueeze(1), y)
    got = ops.gated_residual(x, gate, y)
    assert torch.equal(got, want)
    xc = x.clone()
    ops.gated_residual(xc, gate, y, out=xc)                                     # in place
    assert torch.equal(xc, want)
    with pytest.raises(Exception):
        ops.gated_residual(x[..., :20], gate[:, :20], y[..., :20])
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype,dual", [(torch.bfloat16, False), (torch.bfloat16, True), (torch.float16, False)])
def test_norm_quantize_act_with_residual(dtype, dual):
    """residual=(gate, y): the updated stream is bit-identical to torch.addcmul and the codes are those of the plain
    kernel run on that updated stream."""
    from segquant_b200 import _lib as L, ops
    torch.manual_seed(9)
    B, T, K = 2, 150, 1024 if dtype == torch.float32 else 1536
    x = torch.randn(B, T, K, device="cuda").to(dtype)
    y = (torch.randn(B, T, K, device="cuda") * 2).to(dtype)
    mod = (torch.randn(B, 6 * K, device="cuda") * 0.3).to(dtype)
    shift, scale, gate = mod[:, :K], mod[:, K:2 * K], mod[:, 2 * K:3 * K]
    sx = torch.tensor([127.0 / 4.0], device="cuda")
    sxn = torch.tensor([127.0 / 3.0], device="cuda") if dual else None
    q, qn, x_new = ops.norm_quantize_act(x, [0, K], sx, sxn, shift=shift, scale=scale, residual=(gate, y))
    want_x = torch.addcmul(x, gate.unsqueeze(1), y)
    assert torch.equal(x_new, want_x)
    rq, rqn = ops.norm_quantize_act(want_x, [0, K], sx, sxn, shift=shift, scale=scale)
    assert torch.equal(q, rq)
    assert (qn is None and rqn is None) or torch.equal(qn, rqn)
    assert ops.device_status() == 0
