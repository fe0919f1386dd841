"""torch-CPU restatement of the reference's FAKE-quant SegmentLinear forward -- TEST INFRASTRUCTURE.

This is the path the reference itself runs on a CPU (`real_quant=False`):
segquant/layers/SegmentLinear.py:228-241 -> segquant/optimum/optimizer.py:119-123 ->
IntQuantizer._fake_quantize / FloatQuantizer._fake_quantize (segquant/quantizers/quantizer.py:250-281,
:484-528) -> segmented_matmul (segquant/layers/segment_tensor_manager.py:83-94).  It is the timed
CPU baseline of bench.py (kind "port") and the tolerance reference of the parity tests; it is
checked against outputs of the reference itself in tests/golden/.  Only tests/, smoke() and
bench.py's baseline legs may import it.
"""
import torch

EPS = 1.0 / (1 << 24)


def e4m3_roundtrip(x):
    """fake_e4m3fy: saturating fp32 -> e4m3 -> fp32 (segquant/src/fake_quant/quantizer_fp8.cpp:25-39).
    torch's own cast yields NaN above 464, so clamp to +-448 first."""
    return x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(x.dtype)


def fake_quant_int(x, scale, qmin=-128, qmax=127):
    """IntQuantizer._fake_quantize, symmetric single scale (quantizer.py:266-281)."""
    x_int = torch.clamp(torch.round(x * scale), qmin, qmax)
    return (x_int / scale).to(x.dtype)


def fake_quant_int_dual(x, pos_scale, neg_scale, qmin=-128, qmax=127):
    """IntQuantizer._fake_quantize, DualScale (quantizer.py:251-264)."""
    xq = torch.where(x >= 0, torch.clamp(torch.round(x * pos_scale), 0, qmax),
                     torch.clamp(torch.round(x * neg_scale), qmin, 0))
    return torch.where(x >= 0, xq / pos_scale, xq / neg_scale).to(x.dtype)


def fake_quant_fp8(x, scale):
    """FloatQuantizer._fake_quantize, single scale (quantizer.py:485, :514-528)."""
    zero_mask = x.abs() < EPS
    out = e4m3_roundtrip(x * scale) / scale
    out[zero_mask] = 0.0
    return out.to(x.dtype)


def fake_quant_fp8_dual(x, pos_scale, neg_scale):
    """FloatQuantizer._fake_quantize, DualScale (quantizer.py:487-512)."""
    zero_mask = x.abs() < EPS
    xs = torch.where(x >= 0, x * pos_scale, x * neg_scale)
    xq = e4m3_roundtrip(xs)
    out = torch.where(x >= 0, xq / pos_scale, xq / neg_scale)
    out[zero_mask] = 0.0
    return out.to(x.dtype)


def amax_scale(x, qmax, axis=None):
    """qmax / amax with the epsilon guard (quantizer.py:204-217, :441-452)."""
    if axis is None:
        amax = x.abs().max().item()
        return qmax / amax if amax > EPS else 1.0
    return qmax / x.abs().amax(dim=axis).clamp(min=EPS)


def dual_scales(x, qmax, qmin_abs):
    """Per-tensor DualScale calibration (quantizer.py:170-186, :407-421)."""
    neg = x[x < 0].abs()
    pos = x[x > 0].abs()
    neg_amax = neg.max().item() if neg.numel() else 0.0
    pos_amax = pos.max().item() if pos.numel() else 0.0
    return (qmax / pos_amax if pos_amax > EPS else 1.0), (qmin_abs / neg_amax if neg_amax > EPS else 1.0)


def seg_linear_fake(x, w_fake, bias, bounds, act="int8", sx=None, sx_pos=None, sx_neg=None):
    """Fake-quant forward of a K-segmented layer: quantise-dequantise every K segment of x with its
    own scale(s), multiply by the (already fake-quantised) weight segment, sum, add bias.
    x [M, K]; w_fake [N, K]; sx: list of per-segment scales, or sx_pos/sx_neg for DualScale."""
    S = len(bounds) - 1
    out = None
    for s in range(S):
        xs = x[:, bounds[s]:bounds[s + 1]]
        if sx_pos is not None:
            xs = (fake_quant_int_dual(xs, sx_pos[s], sx_neg[s]) if act == "int8"
                  else fake_quant_fp8_dual(xs, sx_pos[s], sx_neg[s]))
        else:
            xs = fake_quant_int(xs, sx[s]) if act == "int8" else fake_quant_fp8(xs, sx[s])
        part = xs @ w_fake[:, bounds[s]:bounds[s + 1]].t()
        out = part if out is None else out + part
    return out + bias if bias is not None else out


def fake_weight_int(w, qmax, axis=1, group_size=0):
    """Weight fake-quant with per-output-channel (axis=1) or per-(row, K-group) symmetric scales.
    Returns (w_fake, scale).  Group-wise: the reference's IntQuantizer applied to W.view(N, K/g, g)
    with axis=-1 (quantizer.py:209-217)."""
    N, K = w.shape
    if group_size:
        wg = w.view(N, K // group_size, group_size)
        scale = qmax / wg.abs().amax(dim=-1).clamp(min=EPS)
        wq = torch.clamp(torch.round(wg * scale.unsqueeze(-1)), -qmax - 1, qmax)
        return (wq / scale.unsqueeze(-1)).view(N, K), scale
    scale = qmax / w.abs().amax(dim=axis).clamp(min=EPS)
    wq = torch.clamp(torch.round(w * scale.unsqueeze(1)), -qmax - 1, qmax)
    return wq / scale.unsqueeze(1), scale


def fake_weight_fp8(w):
    scale = 448.0 / w.abs().amax(dim=1).clamp(min=EPS)
    return e4m3_roundtrip(w * scale.unsqueeze(1)) / scale.unsqueeze(1), scale
