"""One fake-quant MMDiT joint block on the CPU -- TEST / BASELINE INFRASTRUCTURE (timed by bench.py as the CPU
baseline of the synthetic denoise step: one block, extrapolated x 24 and labelled as such).

Structure of the reference's JointTransformerBlock.forward (backend/torch/layers/attention.py:586-679) with
AdaLayerNormZero (backend/torch/layers/normalization.py:322-380): adaLN projections (SiLU -> Linear(H, 6H) -> chunk 6)
for the image and the text stream, LayerNorm + modulation, q / k / v projections of both streams, joint attention,
gated residual, LayerNorm + modulation, MLP (Linear -> tanh-GELU -> Linear), gated residual.  Every linear is a
fake-quant W8A8 INT8 layer: the REFERENCE's own SegmentLinear(real_quant=False) when the reference package can be
imported (oracle/reference_loader.py), else the restatement in oracle/fake_path.py.  adaLN projections are 6 N-chunks
with DualScale, MLP down-projections DualScale, as the reference's pattern detector assigns them.
"""
import torch
import torch.nn.functional as F

from . import fake_path as FP

NAMES = ["norm1", "norm1_context", "to_q", "to_k", "to_v", "add_q", "add_k", "add_v", "to_out", "to_add_out", "ff0", "ff2", "ffc0", "ffc2"]


class _PortLinear:
    """fake_path restatement of a calibrated fake-quant layer (per-tensor int8 activations, per-channel int8 weights)."""

    def __init__(self, w, b, dual):
        self.w, self.b, self.dual = w, b, dual
        self.wf = None

    def calibrate(self, x):
        x2 = x.reshape(-1, x.shape[-1])
        self.scales = FP.dual_scales(x2, 127.0, 128.0) if self.dual else (FP.amax_scale(x2, 127.0),)
        self.wf = FP.fake_weight_int(self.w, 127.0)[0]

    def __call__(self, x):
        x2 = x.reshape(-1, x.shape[-1])
        K = x2.shape[-1]
        if self.dual:
            y = FP.seg_linear_fake(x2, self.wf, self.b, [0, K], act="int8", sx_pos=[self.scales[0]], sx_neg=[self.scales[1]])
        else:
            y = FP.seg_linear_fake(x2, self.wf, self.b, [0, K], act="int8", sx=[self.scales[0]])
        return y.reshape(*x.shape[:-1], -1)


class _RefLinear:
    """The reference's own SegmentLinear on its CPU (fake-quant) path."""

    def __init__(self, ref, w, b, dual, chunks):
        self.lin = ref.SegmentLinear(w.shape[1], w.shape[0], bias=True, seg_mode="weight", chunks=chunks, custom_weight_tensor=w,
                                     custom_bias_tensor=b, input_quant_type="int8", weight_quant_type="int8",
                                     input_quant_args={"real_quant": False, "axis": None, "dual_scale": dual},
                                     weight_quant_args={"real_quant": False, "axis": 1}, opt_type="default", opt_kwargs={},
                                     calib_type="amax", calib_kwargs={}, device="cpu")

    def calibrate(self, x):
        self.lin.calibrate(x.clone())
        self.lin.finish_calibrate()

    def __call__(self, x):
        return self.lin(x.clone())          # the reference's fake forward writes into its input


class FakeQuantJointBlock:
    def __init__(self, hidden=1536, heads=24, seed=0, ref=None):
        g = torch.Generator().manual_seed(seed)
        self.hidden, self.heads = hidden, heads
        self.kind = "reference" if ref is not None else "port"
        shapes = {"norm1": (6 * hidden, hidden), "norm1_context": (6 * hidden, hidden), "ff0": (4 * hidden, hidden),
                  "ffc0": (4 * hidden, hidden), "ff2": (hidden, 4 * hidden), "ffc2": (hidden, 4 * hidden)}
        dual = {"norm1", "norm1_context", "ff2", "ffc2"}
        self.float_w, self.lin = {}, {}
        for n in NAMES:
            o, i = shapes.get(n, (hidden, hidden))
            w = torch.randn(o, i, generator=g) * 0.02
            b = torch.randn(o, generator=g) * 0.01
            self.float_w[n] = (w, b)
            chunks = 6 if n.startswith("norm1") else 1
            self.lin[n] = _RefLinear(ref, w.clone(), b.clone(), n in dual, chunks) if ref is not None else _PortLinear(w, b, n in dual)

    def _run(self, img, txt, c_act, lin):
        H, B = self.hidden, img.shape[0]
        T = img.shape[1] + txt.shape[1]
        ln = lambda t: F.layer_norm(t, (H,), eps=1e-6)   # noqa: E731
        m = lin("norm1", c_act).chunk(6, dim=-1)
        mc = lin("norm1_context", c_act).chunk(6, dim=-1)
        n_img = ln(img) * (1 + m[1][:, None]) + m[0][:, None]
        n_txt = ln(txt) * (1 + mc[1][:, None]) + mc[0][:, None]
        q = torch.cat([lin("to_q", n_img), lin("add_q", n_txt)], dim=1)
        k = torch.cat([lin("to_k", n_img), lin("add_k", n_txt)], dim=1)
        v = torch.cat([lin("to_v", n_img), lin("add_v", n_txt)], dim=1)
        hd = lambda t: t.view(B, T, self.heads, H // self.heads).transpose(1, 2)   # noqa: E731
        a = F.scaled_dot_product_attention(hd(q), hd(k), hd(v)).transpose(1, 2).reshape(B, T, H)
        Ti = img.shape[1]
        img = img + m[2][:, None] * lin("to_out", a[:, :Ti])
        txt = txt + mc[2][:, None] * lin("to_add_out", a[:, Ti:])
        img = img + m[5][:, None] * lin("ff2", F.gelu(lin("ff0", ln(img) * (1 + m[4][:, None]) + m[3][:, None]), approximate="tanh"))
        txt = txt + mc[5][:, None] * lin("ffc2", F.gelu(lin("ffc0", ln(txt) * (1 + mc[4][:, None]) + mc[3][:, None]), approximate="tanh"))
        return img, txt

    def calibrate(self, img, txt, c_act):
        """One float pass; every layer is calibrated (AMax) on the input it sees."""
        def lin(n, x):
            self.lin[n].calibrate(x)
            w, b = self.float_w[n]
            return F.linear(x, w, b)
        with torch.no_grad():
            return self._run(img, txt, c_act, lin)

    def __call__(self, img, txt, c_act):
        with torch.no_grad():
            return self._run(img, txt, c_act, lambda n, x: self.lin[n](x))
