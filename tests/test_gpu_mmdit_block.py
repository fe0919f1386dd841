"""GPU: one MMDiT joint block at BASELINE config 4's real size (hidden 1536, 24 heads, 4096 image + 333 text tokens,
batch 2, every linear W8A8 INT8 SegLinear, adaLN as 6 N-chunks with DualScale, MLP down-projections DualScale after
tanh-GELU) against a FAKE-QUANT torch restatement of the same block.

The restatement follows the reference's block (backend/torch/layers/attention.py:586-679: norm1 / norm1_context ->
joint attention -> gated residual -> norm2 + modulation -> MLP -> gated residual, for both streams) and its
AdaLayerNormZero (backend/torch/layers/normalization.py:322-380: SiLU -> Linear -> chunk(6)), with every linear replaced
by the reference's fake-quant arithmetic as restated in oracle/fake_path.py (quantise-dequantise the input with the
layer's calibrated scale(s), multiply by the fake-quantised weight), all glue in fp32.  It shares nothing with
segquant_b200.mmdit but the weights and the calibrated scales.

Bars: the unfused quantised block (separate layer_norm / modulation / GELU / quantise kernels) cosine >= 0.9999 and the
fused block (LayerNorm + modulation + quantise in one kernel, GELU inside the quantise kernel, residual folded into the
next normalisation) cosine >= 0.9999 too, per stream; max-rel errors are printed in the assertion messages.  The
quantised block runs bf16 glue and rounds every linear's output to bf16, the restatement is fp32 throughout, so the
difference is bf16 rounding noise (about 2^-9 relative per op), not quantisation error: both sides quantise alike."""
import pytest
import torch
import torch.nn.functional as Fn

pytestmark = pytest.mark.gpu

from oracle import fake_path as FP

DEV = "cuda"
H, HEADS, TI, TT, B = 1536, 24, 4096, 333, 2


def _fake_linear(q, w, b, x):
    """The reference's fake-quant forward of the calibrated layer q.layer on fp32 input x [..., K]."""
    opt = q.layer.optimizer
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    wf, _ = FP.fake_weight_int(w.float(), 127.0)                       # per-output-channel int8
    K = x2.shape[-1]
    if opt.dual_scale:
        pos, neg, _ = opt.scale_tensor
        y = FP.seg_linear_fake(x2, wf, b.float(), [0, K], act="int8", sx_pos=[pos.reshape(-1)[0]], sx_neg=[neg.reshape(-1)[0]])
    else:
        sx, _ = opt.scale_tensor
        y = FP.seg_linear_fake(x2, wf, b.float(), [0, K], act="int8", sx=[sx.reshape(-1)[0]])
    return y.reshape(*lead, -1)


def _ln(x):
    return Fn.layer_norm(x, (x.shape[-1],), eps=1e-6)


def _restated_block(blk, W, img, txt, c_act):
    """fp32 fake-quant joint block (not the last one): returns (img, txt) after both residual updates."""
    lin = lambda name, x: _fake_linear(getattr(blk, name), *W[name], x)   # noqa: E731
    m = lin("norm1", c_act).chunk(6, dim=-1)
    mc = lin("norm1_context", c_act).chunk(6, dim=-1)
    n_img = _ln(img) * (1 + m[1][:, None]) + m[0][:, None]
    n_txt = _ln(txt) * (1 + mc[1][:, None]) + mc[0][:, None]
    q = torch.cat([lin("to_q", n_img), lin("add_q", n_txt)], dim=1)
    k = torch.cat([lin("to_k", n_img), lin("add_k", n_txt)], dim=1)
    v = torch.cat([lin("to_v", n_img), lin("add_v", n_txt)], dim=1)
    heads = lambda t: t.view(B, TI + TT, HEADS, H // HEADS).transpose(1, 2)   # noqa: E731
    a = Fn.scaled_dot_product_attention(heads(q), heads(k), heads(v)).transpose(1, 2).reshape(B, TI + TT, H)
    img = img + m[2][:, None] * lin("to_out", a[:, :TI])
    txt = txt + mc[2][:, None] * lin("to_add_out", a[:, TI:])
    n2 = _ln(img) * (1 + m[4][:, None]) + m[3][:, None]
    img = img + m[5][:, None] * lin("ff2", Fn.gelu(lin("ff0", n2), approximate="tanh"))
    n2c = _ln(txt) * (1 + mc[4][:, None]) + mc[3][:, None]
    txt = txt + mc[5][:, None] * lin("ffc2", Fn.gelu(lin("ffc0", n2c), approximate="tanh"))
    return img, txt


def test_joint_block_real_size_against_fake_quant_restatement(native_lib):
    from segquant_b200 import ops
    from segquant_b200.mmdit import FusedNorm, JointBlock, _gated_add, calibration_calls, quantized_calls
    torch.backends.cuda.matmul.allow_tf32 = False
    gen = torch.Generator().manual_seed(4)
    blk = JointBlock(H, HEADS, gen, DEV, torch.bfloat16, last=False, out_proj_segments=1)
    names = ["norm1", "norm1_context", "to_q", "to_k", "to_v", "add_q", "add_k", "add_v", "to_out", "to_add_out", "ff0", "ff2", "ffc0", "ffc2"]
    W = {n: (getattr(blk, n).w.clone(), getattr(blk, n).b.clone()) for n in names}       # float weights, before they are dropped
    g = torch.Generator().manual_seed(5)
    img = torch.randn(B, TI, H, generator=g).to(torch.bfloat16).to(DEV)
    txt = torch.randn(B, TT, H, generator=g).to(torch.bfloat16).to(DEV)
    c_act = Fn.silu(torch.randn(B, H, generator=g)).to(torch.bfloat16).to(DEV)

    def run(call, norm_call):
        i2, t2, pend_i, pend_t, _ = blk.forward(img, txt, c_act, call, norm_call)
        return _gated_add(i2, *pend_i).float(), _gated_add(t2, *pend_t).float()      # apply the residuals the block left pending

    with torch.no_grad():
        run(*calibration_calls())
        for lay in blk.linears():
            lay.finish()
        want_img, want_txt = _restated_block(blk, W, img.float(), txt.float(), c_act.float())
        n0 = ops.launch_count
        got_unfused = run(*quantized_calls(None))
        assert ops.launch_count > n0
        got_fused = run(*quantized_calls(FusedNorm()))

    def cos(a, b):
        return float(Fn.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0))

    def rel(a, b):
        return float((a - b).abs().max() / b.abs().max())

    for label, (gi, gt) in (("unfused", got_unfused), ("fused", got_fused)):
        ci, ct = cos(gi, want_img), cos(gt, want_txt)
        assert ci >= 0.9999 and ct >= 0.9999, (label, ci, ct, rel(gi, want_img), rel(gt, want_txt))
        assert rel(gi, want_img) <= 5e-2 and rel(gt, want_txt) <= 5e-2, (label, rel(gi, want_img), rel(gt, want_txt))
    # the block's own contribution (output minus input stream), where an error cannot hide behind the residual stream
    for label, (gi, gt) in (("unfused", got_unfused), ("fused", got_fused)):
        di, dt = cos(gi - img.float(), want_img - img.float()), cos(gt - txt.float(), want_txt - txt.float())
        assert di >= 0.999 and dt >= 0.999, (label, di, dt)
    assert ops.device_status() == 0
