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
