"""A small transformer-style block with the linear patterns of a DiT block (adaLN projection after SiLU chunked in six,
q / k / v, an MLP with GELU, an output head), used by the golden-vector generator (where the REFERENCE's quantize()
runs on it) and by the tests of this library's quantize() (which must reproduce those outputs).  Weights and inputs come
from seeded generators so both sides build identical tensors."""
import torch
import torch.nn.functional as F
from torch import nn


class ToyBlock(nn.Module):
    def __init__(self, hidden=64, seed=0):
        super().__init__()
        self.hidden = hidden
        self.norm_lin = nn.Linear(hidden, 6 * hidden)
        self.to_q, self.to_k, self.to_v = nn.Linear(hidden, hidden), nn.Linear(hidden, hidden), nn.Linear(hidden, hidden)
        self.ff = nn.Sequential(nn.Linear(hidden, 4 * hidden), nn.GELU(approximate="tanh"), nn.Linear(4 * hidden, hidden))
        self.proj_out = nn.Linear(hidden, 16)
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * (0.05 if p.dim() == 2 else 0.01))

    def forward(self, x, c):
        h = self.hidden
        m = self.norm_lin(F.silu(c)).chunk(6, dim=-1)
        n = F.layer_norm(x, (h,)) * (1 + m[1][:, None]) + m[0][:, None]
        q, k, v = self.to_q(n), self.to_k(n), self.to_v(n)
        a = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        x = x + m[2][:, None] * a
        n2 = F.layer_norm(x, (h,)) * (1 + m[4][:, None]) + m[3][:, None]
        x = x + m[5][:, None] * self.ff(n2)
        return self.proj_out(x)


def toy_batches(n=3, batch=2, tokens=24, hidden=64, seed=1):
    """Calibration set in the form quantize() consumes: a list of (args tuple,) items."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        x = torch.randn(batch, tokens, hidden, generator=g)
        x[..., 3] *= 12.0                      # one outlier channel, so smoothing has something to move
        out.append(((x, torch.randn(batch, hidden, generator=g)),))
    return out


def toy_config(DType, Optimum, Calibrate, search=False, real_quant=False):
    """Smooth + AMax, int8 per-tensor activations, int8 per-channel weights, no segmentation, output head disabled."""
    opt = {"type": Optimum.SMOOTH, "alpha": 0.5}
    if search:
        opt["search_alpha_config"] = {"enable": True, "min": 0.3, "max": 0.7, "step": 0.2}
    return {
        "default": {"enable": True, "seglinear": False, "search_patterns": [], "real_quant": real_quant, "opt": opt,
                    "calib": {"type": Calibrate.AMAX}, "input_quant": {"type": DType.INT8, "axis": None},
                    "weight_quant": {"type": DType.INT8, "axis": 1}},
        "*proj_out": {"enable": False},
    }
