"""SegmentLinear: a linear layer whose activations (K-segments, seg_mode="input") or weights
(N-segments, seg_mode="weight") are quantised per segment, optionally with DualScale
(separate scales for the negative and the positive part of a post-GELU/SiLU input).

Constructor signature, method names and the calibrate -> finish_calibrate -> forward life cycle are
those of the reference's segquant/layers/SegmentLinear.py:11-241, so layers built by the
reference's quantize() recipes can be built the same way here.  What differs:

* real_quant=True never degrades to fake quantisation: an unknown kernel type raises
  (the reference prints a warning and falls back, :105-113);
* forward() on the real path is the fused quantise + tcgen05 GEMM of ops.seg_linear: segment sum,
  bias add and output cast happen in the GEMM epilogue (the reference sums S partial outputs and
  adds the bias in torch, :233-241);
* unequal `chunksizes` are accepted for seg_mode="input" (the reference raises, :80-82).
"""
from typing import Literal

import torch
import torch.nn as nn

from ..calibrator.calibrator import CalibratorRegistry
from ..config import Calibrate, DType, Optimum
from ..optimum.optimizer import OptimizerRegistry
from . import ext_dict
from .segment_tensor_manager import InputSegmentTensorManager, WeightSegmentTensorManager


def _even_split(total, parts):
    base, rem = divmod(total, parts)
    return [base + (1 if i < rem else 0) for i in range(parts)]


class SegmentLinear(nn.Module):
    def __init__(self, in_features, out_features, bias=True, seg_mode: Literal["input", "weight"] = "weight",
                 chunks=1, chunksizes=None, custom_weight_tensor=None, custom_bias_tensor=None,
                 input_quant_type=None, weight_quant_type=None, input_quant_args=None, weight_quant_args=None,
                 opt_type: Literal["default", "smooth", "svd"] = "default", opt_kwargs=None,
                 calib_type: Literal["amax", "gptq"] = "amax", calib_kwargs=None, device="cuda:0"):
        super().__init__()
        if seg_mode not in ("input", "weight"):
            raise ValueError("seg_mode not found")
        self.in_features, self.out_features = in_features, out_features
        self.seg_mode, self.chunks = seg_mode, chunks
        input_quant_args = dict(input_quant_args or {})
        weight_quant_args = dict(weight_quant_args or {})
        opt_kwargs, calib_kwargs = dict(opt_kwargs or {}), dict(calib_kwargs or {})

        if custom_weight_tensor is not None:
            if tuple(custom_weight_tensor.shape) != (out_features, in_features):
                raise AssertionError(f"Mismatched custom_weight_tensor shape! Expected ({out_features}, {in_features}), "
                                     f"but got {tuple(custom_weight_tensor.shape)}.")
            self.origin_device = custom_weight_tensor.device
            weight = custom_weight_tensor.to(device).clone()
        else:
            self.origin_device = torch.device("cpu")
            weight = torch.randn(out_features, in_features)
        self.bias = bias
        self.bias_data = None
        if bias:
            self.bias_data = (custom_bias_tensor.to(device).clone() if custom_bias_tensor is not None
                              else torch.zeros(out_features, device=device))

        target = in_features if seg_mode == "input" else out_features
        if chunksizes is None:
            self.chunksizes = _even_split(target, chunks)
        else:
            assert len(chunksizes) == chunks and sum(chunksizes) == target
            self.chunksizes = list(chunksizes)
        uniform = len(set(self.chunksizes)) == 1
        if not uniform and seg_mode == "weight":
            raise NotImplementedError("Only support equal chunksizes for seg_mode='weight'.")

        real_quant = bool(input_quant_args.get("real_quant", False)) if input_quant_type is not None else False
        dual_scale = bool(input_quant_args.get("dual_scale", False)) if input_quant_type is not None else False
        if weight_quant_type is not None:
            if "real_quant" in weight_quant_args:
                assert real_quant == weight_quant_args["real_quant"], \
                    f"Mismatch: real_quant={real_quant}, weight_quant_args['real_quant']={weight_quant_args['real_quant']}"
            if "dual_scale" in weight_quant_args:
                raise ValueError("Dual scale is not supported for weight quantizer in DefaultSegmentLinear.")
        kernel_type = f"W{weight_quant_type}A{input_quant_type}"
        if real_quant:
            if kernel_type not in ext_dict or None in ext_dict[kernel_type].values():
                raise RuntimeError(f"SegmentLinear needs the real-quant kernel [{kernel_type}], which this build does not "
                                   f"provide (available: {sorted(ext_dict.keys())}); there is no fake-quant fallback")
        input_quant_args["real_quant"] = real_quant
        weight_quant_args["real_quant"] = real_quant

        self.opt_type = opt_type
        if opt_type == "default":
            n_in, n_w = (chunks, 1) if seg_mode == "input" else (1, chunks)
        elif opt_type in ("smooth", "svd"):
            n_in, n_w = chunks, chunks
        else:
            raise ValueError(f"Optimizer '{opt_type}' not found in registry.")

        manager = WeightSegmentTensorManager(weight, seg_mode=seg_mode, segments=chunks, segment_size=self.chunksizes[0],
                                             segment_sizes=self.chunksizes)
        self.optimizer = OptimizerRegistry.create(
            opt_type, seg_mode=seg_mode, chunks=chunks, chunksizes=self.chunksizes, weight_manager=manager,
            input_calibrators=[CalibratorRegistry.create("amax", data_type="input", quant_type=input_quant_type,
                                                         quant_args=input_quant_args, **calib_kwargs) for _ in range(n_in)],
            weight_calibrators=[CalibratorRegistry.create(calib_type, data_type="weight", quant_type=weight_quant_type,
                                                          quant_args=weight_quant_args, **calib_kwargs) for _ in range(n_w)],
            real_quant=real_quant, dual_scale=dual_scale, kernel_type=kernel_type, **opt_kwargs)

    # ---- helpers ------------------------------------------------------------------------------
    def _inputs(self, x):
        return InputSegmentTensorManager(x, seg_mode=self.seg_mode, segments=self.chunks, segment_size=self.chunksizes[0],
                                         segment_sizes=self.chunksizes)

    def __repr__(self):
        return (f"SegmentLinear(\n  in_features={self.in_features}, out_features={self.out_features}, seg_mode={self.seg_mode},\n"
                f"  chunks={self.chunks}, chunksize={self.chunksizes},\n  opt={self.optimizer!r}\n)")

    # ---- calibration life cycle -------------------------------------------------------------------
    def trace(self, input_data):
        self.optimizer.trace(self._inputs(input_data))

    def smooth(self):
        self.optimizer.smooth()

    def calibrate(self, input_data):
        self.optimizer.calibrate(self._inputs(input_data))

    def finish_calibrate(self):
        self.optimizer.finish_calibrate()

    def segment_forward(self, x, weight):
        """Un-quantised per-segment products (used by the reference's alpha search)."""
        xs = self._inputs(x).iter_view()
        ws = WeightSegmentTensorManager(weight, seg_mode=self.seg_mode, segments=self.chunks,
                                        segment_size=self.chunksizes[0], segment_sizes=self.chunksizes).iter_view()
        return xs @ ws.unsqueeze(1).transpose(-1, -2)

    # ---- device moves --------------------------------------------------------------------------------
    def to(self, device):
        device = torch.device(device) if isinstance(device, str) else device
        if device.type == "cuda":
            self.to_cuda(device)
        elif device.type == "cpu":
            self.to_cpu()
        else:
            raise ValueError(f"Unsupported device type: {device.type}")
        return self

    def to_cpu(self):
        self.optimizer.to_cpu()
        if self.bias_data is not None:
            self.bias_data = self.bias_data.to("cpu")

    def to_cuda(self, device=None):
        device = self.origin_device if device is None else device
        self.optimizer.to_cuda(device)
        if self.bias_data is not None:
            self.bias_data = self.bias_data.to(device)

    # ---- forward ---------------------------------------------------------------------------------------
    def forward(self, x, chunked=False, out=None, peer_outputs=None):
        """out (real-quant path only): a (B, M, N) view to write into, e.g. a slice of a larger buffer.
        peer_outputs (with out=, B = 1): (pointers, row stride, column offset) of peer GPUs' buffers that receive the
        same tiles straight from the GEMM epilogue (column-sharded layers, segquant_b200/sharded.py)."""
        opt = self.optimizer
        if opt.real_quant and not chunked:
            if peer_outputs is not None:
                return opt.fused_forward(x, self.bias_data if self.bias else None, out=out, peer_outputs=peer_outputs)
            return opt.fused_forward(x, self.bias_data if self.bias else None, out=out)
        if out is not None:
            raise ValueError("out= is served by the fused real-quant forward only")
        parts = opt.forward(self._inputs(x))
        if chunked:
            return parts
        if self.seg_mode == "weight":
            out = parts.movedim(0, -2).reshape(*parts.shape[1:-1], -1)
        else:
            out = parts.sum(dim=0)
        return out + self.bias_data if self.bias else out


    def forward_quantized(self, xq, xq_neg=None, out=None, out_dtype=torch.bfloat16):
        """The layer's GEMM + epilogue on activations the caller has already quantised with
        `self.optimizer.input_quant_params()` (e.g. ops.norm_quantize_act); xq (B, M, K) uint8."""
        return self.optimizer.fused_gemm(xq, xq_neg, self.bias_data if self.bias else None, out=out, out_dtype=out_dtype)


def create_segment_linear(input_dtype: DType, weight_dtype: DType, opt: Optimum, calib: Calibrate, in_features,
                          out_features, opt_kwargs, calib_kwargs, input_quant_args, weight_quant_args, **kwargs):
    return SegmentLinear(in_features, out_features, input_quant_type=input_dtype.value,
                         weight_quant_type=weight_dtype.value, opt_type=opt.value, calib_type=calib.value,
                         opt_kwargs=opt_kwargs, calib_kwargs=calib_kwargs, input_quant_args=input_quant_args,
                         weight_quant_args=weight_quant_args, **kwargs)


def DualScale(in_features, out_features, **kwargs):
    """A SegmentLinear whose activation quantiser keeps separate negative / positive scales: the
    `dual_scale=True` flag of input_quant_args (segquant/layers/SegmentLinear.py:84-101), which the
    reference's quantize() sets for linears that follow an activation function."""
    args = dict(kwargs.pop("input_quant_args", None) or {})
    args["dual_scale"] = True
    return SegmentLinear(in_features, out_features, input_quant_args=args, **kwargs)
