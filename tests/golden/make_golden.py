"""Generate the golden fixtures in this directory by running the REFERENCE's own Python code.

    python tests/golden/make_golden.py [<reference checkout> [fixture name ...]]

The reference (OptiSys-ZJU/segquant) is imported from its read-only checkout (the argument, or the
SEGQUANT_REFERENCE environment variable) by oracle/reference_loader.py with stub extension loaders;
nothing of it is copied.  SegmentLinear then takes its fake-quant branch
(segquant/layers/SegmentLinear.py:105-113), which is the reference's CPU path.  The fp8 round trip
uses the reference's own fake_e4m3fy C++ built into oracle/_ref/ (oracle/build_ref.py).

Each fixture is an .npz with the seeded inputs, the scales the reference's calibrators produced and
the reference's outputs.  tests/test_oracle_golden.py checks the oracle against them on CPU;
tests/test_gpu_parity.py checks the CUDA path against them on the GPU.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)


def import_reference(root):
    from oracle.build_ref import load_prebuilt
    if load_prebuilt() is None:
        raise SystemExit("oracle/_ref is not built: run `python oracle/build_ref.py <reference checkout>` first")
    from oracle.reference_loader import import_reference as imp
    ref = imp("stub", root)
    return ref.SegmentLinear, ref.quantizer


def t2n(t):
    if isinstance(t, torch.Tensor):
        return t.detach().float().cpu().numpy()
    return np.float32(t)


def gen_input_seg_int8(SegmentLinear, seed=0, M=96, K=256, N=64, S=4):
    """BASELINE config-1 recipe at toy size: K-segmented W8A8 INT8, per-segment activation scales,
    per-output-channel weight scales."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    factors = [0.5, 1.0, 4.0, 16.0]
    seg = K // S
    for s in range(S):
        x[:, s * seg:(s + 1) * seg] *= factors[s % 4]
    perm = torch.randperm(K, generator=g)[: max(1, int(0.02 * K))]
    x[:, perm] *= 20.0
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    lin = SegmentLinear(K, N, bias=True, seg_mode="input", chunks=S, custom_weight_tensor=w.clone(),
                        custom_bias_tensor=b.clone(), input_quant_type="int8", weight_quant_type="int8",
                        input_quant_args={"real_quant": False, "axis": None},
                        weight_quant_args={"real_quant": False, "axis": 1},
                        opt_type="default", opt_kwargs={}, calib_type="amax", calib_kwargs={}, device="cpu")
    lin.calibrate(x.clone())
    lin.finish_calibrate()
    y = lin(x.clone())
    sx, sw = lin.optimizer.scale_tensor
    return dict(x=t2n(x), w=t2n(w), b=t2n(b), y=t2n(y), sx=t2n(sx), sw=t2n(sw),
                w_fake=t2n(lin.optimizer.weight_manager.weight_tensor), bounds=np.arange(S + 1, dtype=np.int32) * seg)


def gen_dual_fp8(SegmentLinear, seed=1, M=96, K=384, N=48):
    """BASELINE config-2 recipe at toy size: DualScale FP8 after GELU, per-output-channel weights."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(M, K, generator=g)
    x = torch.nn.functional.gelu(z)
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    lin = SegmentLinear(K, N, bias=True, seg_mode="weight", chunks=1, custom_weight_tensor=w.clone(),
                        custom_bias_tensor=b.clone(), input_quant_type="fpe4m3", weight_quant_type="fpe4m3",
                        input_quant_args={"real_quant": False, "axis": None, "dual_scale": True},
                        weight_quant_args={"real_quant": False, "axis": 1},
                        opt_type="default", opt_kwargs={}, calib_type="amax", calib_kwargs={}, device="cpu")
    lin.calibrate(x.clone())
    lin.finish_calibrate()
    y = lin(x.clone())
    sp, sn, sw = lin.optimizer.scale_tensor
    return dict(x=t2n(x), w=t2n(w), b=t2n(b), y=t2n(y), sx_pos=t2n(sp), sx_neg=t2n(sn), sw=t2n(sw),
                w_fake=t2n(lin.optimizer.weight_manager.weight_tensor), bounds=np.array([0, K], dtype=np.int32))


def gen_weight_seg_dual_int8(SegmentLinear, seed=3, M=4, K=128, N=192, S=6):
    """The adaLN pattern: SiLU -> Linear -> chunk(6): N-segmented weights, DualScale int8 activations."""
    g = torch.Generator().manual_seed(seed)
    x = torch.nn.functional.silu(torch.randn(M, K, generator=g))
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    lin = SegmentLinear(K, N, bias=True, seg_mode="weight", chunks=S, custom_weight_tensor=w.clone(),
                        custom_bias_tensor=b.clone(), input_quant_type="int8", weight_quant_type="int8",
                        input_quant_args={"real_quant": False, "axis": None, "dual_scale": True},
                        weight_quant_args={"real_quant": False, "axis": None},
                        opt_type="default", opt_kwargs={}, calib_type="amax", calib_kwargs={}, device="cpu")
    lin.calibrate(x.clone())
    lin.finish_calibrate()
    y = lin(x.clone())
    sp, sn, sw = lin.optimizer.scale_tensor
    return dict(x=t2n(x), w=t2n(w), b=t2n(b), y=t2n(y), sx_pos=t2n(sp), sx_neg=t2n(sn), sw=t2n(sw),
                w_fake=t2n(lin.optimizer.weight_manager.weight_tensor), chunks=np.int32(S))


def gen_smooth_int8(SegmentLinear, seed=6, M=80, K=256, N=64, S=4, mode="input"):
    """SmoothOptimizer recipe (config/sd3/dit/intw8a8.yaml: opt smooth, alpha 0.5) at toy size: outlier
    channels migrate into the weights; one input and one weight quantiser per chunk."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    perm = torch.randperm(K, generator=g)[:6]
    x[:, perm] *= 25.0
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    lin = SegmentLinear(K, N, bias=True, seg_mode=mode, chunks=S, custom_weight_tensor=w.clone(),
                        custom_bias_tensor=b.clone(), input_quant_type="int8", weight_quant_type="int8",
                        input_quant_args={"real_quant": False, "axis": None},
                        weight_quant_args={"real_quant": False, "axis": 1},
                        opt_type="smooth", opt_kwargs={"alpha": 0.5}, calib_type="amax", calib_kwargs={}, device="cpu")
    lin.trace(x.clone())
    lin.smooth()
    lin.calibrate(x.clone())
    lin.finish_calibrate()
    y = lin(x.clone())
    sx, sw = lin.optimizer.scale_tensor
    s = torch.stack([v.float() for v in lin.optimizer.s])
    return dict(x=t2n(x), w=t2n(w), b=t2n(b), y=t2n(y), sx=t2n(sx), sw=t2n(sw), s=t2n(s), chunks=np.int32(S),
                w_fake=t2n(lin.optimizer.weight_manager.weight_tensor))


def gen_svd_w4a8(SegmentLinear, seed=8, M=64, K=256, N=96, S=2, mode="input", dynamic=False, low_rank=16):
    """The W4A8 recipe of config/flux/dit/intw4a8.yaml:49-75 at toy size (AMax instead of GPTQ calibration): SVDOptimizer,
    int4 per-output-channel weights on the SVD residual, int8 activations (static per segment, or dynamic per token).
    `y` is the reference's CPU (fake-quant) output; l1s / l2s / s / w_fake let a test rebuild what the real-quant path
    computes (low-rank branch on the unquantised smoothed activations)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:5]] *= 15.0
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    in_args = {"real_quant": False, "axis": -1, "dynamic": True} if dynamic else {"real_quant": False, "axis": None}
    lin = SegmentLinear(K, N, bias=True, seg_mode=mode, chunks=S, custom_weight_tensor=w.clone(),
                        custom_bias_tensor=b.clone(), input_quant_type="int8", weight_quant_type="int4",
                        input_quant_args=in_args, weight_quant_args={"real_quant": False, "axis": 1},
                        opt_type="svd", opt_kwargs={"alpha": 0.5, "low_rank": low_rank, "precision": "float64"},
                        calib_type="amax", calib_kwargs={}, device="cpu")
    lin.trace(x.clone())
    lin.smooth()
    lin.calibrate(x.clone())
    lin.finish_calibrate()
    y = lin(x.clone())
    opt = lin.optimizer
    sx, sw = opt.scale_tensor
    return dict(x=t2n(x), w=t2n(w), b=t2n(b), y=t2n(y), sx=t2n(sx), sw=t2n(sw), s=t2n(torch.stack([v.float() for v in opt.s])),
                l1s=t2n(opt.l1s), l2s=t2n(opt.l2s), chunks=np.int32(S), low_rank=np.int32(low_rank),
                w_fake=t2n(opt.weight_manager.weight_tensor))


def gen_quantize_toy(root, search):
    """The reference's own quantize() (segquant/torch/quantization.py:259-425) on tests/golden/toy_model.py, CPU fake path,
    no segmentation (the pattern detector is not exercised): outputs of the quantised model plus the alphas it settled on."""
    sys.path.insert(0, HERE)
    from toy_model import ToyBlock, toy_batches, toy_config
    from segquant.config import Calibrate, DType, Optimum
    from segquant.torch.quantization import quantize
    model = ToyBlock()
    batches = toy_batches()
    x, c = batches[0][0]
    y_float = model(x, c)
    qm = quantize(model, batches, toy_config(DType, Optimum, Calibrate, search=search))
    y = qm(x.clone(), c.clone())
    alphas = np.array([qm.to_q.optimizer.alpha[0], qm.ff[2].optimizer.alpha[0], qm.norm_lin.optimizer.alpha[0]], np.float64)
    return dict(y=t2n(y), y_float=t2n(y_float), alphas=alphas, replaced=np.array(
        [type(m).__name__ == "SegmentLinear" for m in (qm.norm_lin, qm.to_q, qm.to_k, qm.to_v, qm.ff[0], qm.ff[2], qm.proj_out)]),
        sx_to_q=t2n(qm.to_q.optimizer.scale_tensor[0]), sw_ff2=t2n(qm.ff[2].optimizer.scale_tensor[1]))


def gen_quantizer_vectors(q, seed=4):
    """Scale definitions and fake-quant outputs straight from the reference's quantizer classes."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    x = torch.randn(32, 64, generator=g) * 3
    x[0, 0] = 0.0
    iq = q.IntQuantizer(num_bits=8, axis=None)
    iq.calibrate(x)
    out["int8_x"] = t2n(x); out["int8_scale"] = t2n(iq.scale); out["int8_fake"] = t2n(iq.fake_quantize(x))
    iqa = q.IntQuantizer(num_bits=8, axis=1)
    iqa.calibrate(x)
    out["int8_axis1_scale"] = t2n(iqa.scale); out["int8_axis1_fake"] = t2n(iqa.fake_quantize(x))
    xs = torch.nn.functional.silu(torch.randn(32, 64, generator=g) * 2)
    iqd = q.IntQuantizer(num_bits=8, axis=None, dual_scale=True)
    iqd.calibrate(xs)
    out["dual_x"] = t2n(xs); out["dual_int8_pos"] = t2n(iqd.pos_scale); out["dual_int8_neg"] = t2n(iqd.neg_scale)
    out["dual_int8_fake"] = t2n(iqd.fake_quantize(xs))
    fq = q.FloatQuantizer(axis=None)
    fq.calibrate(x)
    out["fp8_scale"] = t2n(fq.scale); out["fp8_fake"] = t2n(fq.fake_quantize(x))
    fqd = q.FloatQuantizer(axis=None, dual_scale=True)
    fqd.calibrate(xs)
    out["dual_fp8_pos"] = t2n(fqd.pos_scale); out["dual_fp8_neg"] = t2n(fqd.neg_scale)
    out["dual_fp8_fake"] = t2n(fqd.fake_quantize(xs))
    # int4 group-wise weights: IntQuantizer(num_bits=4, axis=-1) on W.view(N, K/g, g)
    w = torch.randn(24, 256, generator=g) * 0.02
    i4 = q.IntQuantizer(num_bits=4, axis=-1)
    wg = w.view(24, 2, 128)
    i4.calibrate(wg)
    out["int4_w"] = t2n(w); out["int4_group_scale"] = t2n(i4.scale); out["int4_group_fake"] = t2n(i4.fake_quantize(wg).view(24, 256))
    # dynamic per-token int8: IntQuantizer(axis=-1, dynamic=True).quantize
    dq = q.IntQuantizer(num_bits=8, axis=-1, dynamic=True)
    out["dyn_fake"] = t2n(dq.quantize(x)); out["dyn_scale"] = t2n(dq.scale)
    xb = x.to(torch.bfloat16)
    dqb = q.IntQuantizer(num_bits=8, axis=-1, dynamic=True)
    dqb.quantize(xb)
    out["dyn_scale_bf16"] = t2n(dqb.scale)
    # fp8 round trip on a grid of values (the reference's compiled fake_e4m3fy)
    grid = torch.cat([torch.linspace(-500, 500, 4001), torch.logspace(-12, 3, 600), -torch.logspace(-12, 3, 600)]).float()
    out["e4m3_grid"] = t2n(grid)
    out["e4m3_roundtrip"] = t2n(q.load_fake_quant_fp8_ext().fake_e4m3fy(grid.contiguous()))
    return out


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SEGQUANT_REFERENCE")
    if not root:
        raise SystemExit("usage: make_golden.py <reference checkout>  (or set SEGQUANT_REFERENCE)")
    torch.set_num_threads(1)  # deterministic reductions
    SegmentLinear, q = import_reference(root)
    fixtures = {
        "input_seg_int8": gen_input_seg_int8(SegmentLinear),
        "dual_fp8": gen_dual_fp8(SegmentLinear),
        "weight_seg_dual_int8": gen_weight_seg_dual_int8(SegmentLinear),
        "quantizers": gen_quantizer_vectors(q),
        "smooth_input_seg_int8": gen_smooth_int8(SegmentLinear, mode="input"),
        "smooth_weight_seg_int8": gen_smooth_int8(SegmentLinear, seed=7, S=2, mode="weight"),
        "svd_w4a8_input_seg": gen_svd_w4a8(SegmentLinear),
        "svd_w4a8_dynamic": gen_svd_w4a8(SegmentLinear, seed=9, S=1, mode="weight", dynamic=True),
        "svd_w4a8_weight_seg": gen_svd_w4a8(SegmentLinear, seed=10, N=128, S=2, mode="weight"),
        "quantize_toy_smooth": gen_quantize_toy(root, search=False),
        "quantize_toy_search": gen_quantize_toy(root, search=True),
    }
    only = set(sys.argv[2:])
    for name, d in fixtures.items():
        if only and name not in only:
            continue
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **d)
        print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KB): {sorted(d)}")


if __name__ == "__main__":
    main()
