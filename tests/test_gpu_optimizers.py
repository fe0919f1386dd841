"""GPU: the optimizers beyond `default` on the real-quant path -- SVDOptimizer's low-rank branch (the W4A8 recipe of
the reference, config/flux/dit/intw4a8.yaml:49-75) and smoothing inside the dynamic per-token quantise kernel --
against fixtures produced by the reference's own Python (tests/golden/svd_*.npz).

Tolerance, stated: max rel err <= 1e-2 and cosine >= 0.9999 against the expected real-path result rebuilt from the
reference's factors; measured values are printed by the assertions' messages when they fail."""
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


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    yield
    assert ops.device_status() == 0


def max_rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def cosine(a, b):
    a, b = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def build_svd(g, mode, chunks, dynamic, dtype=torch.float32):
    x, w, b = (torch.from_numpy(g[k]).to(DEV) for k in "xwb")
    in_args = {"real_quant": True, "axis": -1, "dynamic": True} if dynamic else {"real_quant": True, "axis": None}
    lin = SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode=mode, chunks=chunks, custom_weight_tensor=w, custom_bias_tensor=b,
                        input_quant_type="int8", weight_quant_type="int4", input_quant_args=in_args,
                        weight_quant_args={"real_quant": True, "axis": 1}, opt_type="svd",
                        opt_kwargs={"alpha": 0.5, "low_rank": int(g["low_rank"]), "precision": "float64"}, device=DEV)
    lin.trace(x)
    lin.smooth()
    lin.calibrate(x)
    lin.finish_calibrate()
    return lin, x


def expected_real_path(g, mode, dynamic):
    """What the real-quant path computes, from the reference's own ingredients: Q(x / s) Q(R)^T + (x / s) L1 L2 + b,
    with the low-rank branch on the UNQUANTISED smoothed activations."""
    x, b, s, wf = (torch.from_numpy(g[k]).double() for k in ("x", "b", "s", "w_fake"))
    l1, l2 = torch.from_numpy(g["l1s"]).double(), torch.from_numpy(g["l2s"]).double()
    S = int(g["chunks"])
    M, K = x.shape
    N = wf.shape[0]
    y = torch.zeros(M, N, dtype=torch.float64)
    for i in range(S):
        if mode == "input":
            cols, rows = slice(i * K // S, (i + 1) * K // S), slice(0, N)
        else:
            cols, rows = slice(0, K), slice(i * N // S, (i + 1) * N // S)
        xs = (x[:, cols].float() / s[i].float()).double()
        if dynamic:
            sc = (127.0 / xs.float().abs().amax(dim=-1).clamp(min=F.EPS)).double().unsqueeze(1)
        else:
            sc = float(np.atleast_1d(g["sx"]).reshape(-1)[i])
        xq = torch.clamp(torch.round(xs * sc), -128, 127) / sc
        y[:, rows] += xq @ wf[rows, cols].t() + xs @ l1[i] @ l2[i]
    return (y + b).numpy()


@pytest.mark.parametrize("name,mode,dynamic", [("svd_w4a8_input_seg", "input", False), ("svd_w4a8_dynamic", "weight", True),
                                               ("svd_w4a8_weight_seg", "weight", False)])
def test_svd_optimizer_real_path(golden, name, mode, dynamic):
    g = golden(name)
    lin, x = build_svd(g, mode, int(g["chunks"]), dynamic)
    opt = lin.optimizer
    assert opt.weight_manager.packed and opt.weight_manager.weight_tensor.dtype == torch.uint8
    assert np.allclose(torch.stack(opt.s).cpu().numpy(), g["s"], rtol=1e-5)
    want_prod = np.matmul(g["l1s"], g["l2s"])
    assert np.abs(torch.bmm(opt.l1s, opt.l2s).cpu().numpy() - want_prod).max() <= 1e-5 * np.abs(want_prod).max()
    # the packed int4 residual equals the reference's fake-quantised residual: unpack * 1/scale
    N, K = g["w"].shape
    S = int(g["chunks"])
    un = ops.unpack_int4(opt.weight_manager.weight_tensor.reshape(-1)).cpu().numpy().astype(np.float32)
    sw = opt.scale_tensor[-1].cpu().numpy()
    if mode == "input":
        wq = un.reshape(N, K)
        deq = np.concatenate([wq[:, i * K // S:(i + 1) * K // S] / sw[i][:, None] for i in range(S)], axis=1)
    else:
        deq = un.reshape(S, N // S, K) / sw[:, :, None]
        deq = deq.reshape(N, K)
    assert np.abs(deq - g["w_fake"]).max() <= 1e-6
    x0 = x.clone()
    y = lin(x).cpu().numpy()
    assert torch.equal(x, x0)
    want = expected_real_path(g, mode, dynamic)
    assert max_rel(y, want) <= 1e-2 and cosine(y, want) >= 0.9999, (max_rel(y, want), cosine(y, want))
    assert max_rel(y, want) <= 5e-5, max_rel(y, want)               # fp32 in / out: in fact equal up to fp32 rounding
    # against the reference's CPU output itself (its low-rank branch reads fake-quantised activations): same layer, so
    # close, but only to the size of the activation quantisation error times the low-rank part
    assert cosine(y, g["y"]) >= 0.999
    if not dynamic:
        parts = lin(x, chunked=True)                                   # un-summed reference contract + low-rank per chunk
        y2 = (parts.sum(0) if mode == "input" else parts.movedim(0, -2).reshape(x.shape[0], -1)) + lin.bias_data
        assert max_rel(y2.cpu().numpy(), want) <= 5e-5
    # bf16 activations: one output rounding (plus the bf16 low-rank GEMMs) away
    yb = lin(x.to(torch.bfloat16))
    assert yb.dtype == torch.bfloat16
    assert max_rel(yb.float().cpu().numpy(), want) <= 2e-2 and cosine(yb.float().cpu().numpy(), want) >= 0.9999


@pytest.mark.parametrize("dtype,M,K,bounds", [(torch.float32, 70, 768, [0, 256, 768]), (torch.bfloat16, 70, 768, [0, 256, 768]),
                                              (torch.bfloat16, 600, 4096, [0, 1024, 4096])])
@pytest.mark.parametrize("dual", [False, True])
def test_act_quant_dynamic_with_smoothing(dtype, dual, M, K, bounds):
    """Per-token dynamic scales on x / s: the kernel calibrates and quantises round_dtype(x / round_dtype(s)), the tensor the
    reference's optimizers hand to the quantiser; scales equal the reference definition bit for bit, bytes equal the oracle."""
    # (the large bf16 case has 2.4 M elements: a few hundred of them land within a few fp32 ulps of a bf16 rounding boundary,
    # where the kernel's reciprocal-multiply shortcut must hand over to the exact division)
    g = torch.Generator().manual_seed(21)
    x = (torch.randn(M, K, generator=g) * 3).to(dtype)
    if dual:
        x = torch.nn.functional.silu(x.float()).to(dtype)
    s = (torch.rand(K, generator=g) * 4 + 0.1)
    s_t = s.to(dtype)
    xs = x / s_t                                                     # torch: division in fp32, one rounding to dtype
    xq, xqn, sx, sxn = ops.quantize_act_dynamic(x.to(DEV), bounds, L.SQ_Q_INT8, dual=dual, smooth=s_t.float().to(DEV))
    sx_ref, sxn_ref = [], []
    for i in range(2):
        seg = xs[:, bounds[i]:bounds[i + 1]]
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
        want = O.quantize_act(xs.float().numpy(), bounds, sx_ref.numpy(), sx_neg=sxn_ref.numpy(), out_kind=O.Q_INT8)
        assert np.array_equal(xq.cpu().numpy().view(np.int8), want[0]) and np.array_equal(xqn.cpu().numpy().view(np.int8), want[1])
    else:
        want = O.quantize_act(xs.float().numpy(), bounds, sx_ref.numpy(), out_kind=O.Q_INT8)
        assert np.array_equal(xq.cpu().numpy().view(np.int8), want)
