"""Zero-copy segment views of activations and weights.

Same view conventions as the reference (segquant/layers/segment_tensor_manager.py:15-23, :45-80):
K-segmentation ("input" mode) views x[..., K] as (S, ..., K/S); N-segmentation ("weight" mode)
expands x to (S, ..., K) with stride 0 and views the weight as (S, N/S, K).  Unlike the reference
the managers also carry explicit segment bounds, so unequal K-segments are allowed.
"""
import torch


def bounds_from_sizes(sizes):
    out = [0]
    for s in sizes:
        out.append(out[-1] + int(s))
    return out


class SegmentTensorManager:
    def __init__(self, seg_mode, segments, segment_size, segment_sizes=None):
        if seg_mode not in ("input", "weight"):
            raise ValueError("seg_mode not found")
        self.seg_mode, self.segments, self.segment_size = seg_mode, segments, segment_size
        self.segment_sizes = list(segment_sizes) if segment_sizes is not None else [segment_size] * segments
        self.bounds = bounds_from_sizes(self.segment_sizes)
        self.uniform = len(set(self.segment_sizes)) == 1

    def _need_uniform(self):
        if not self.uniform:
            raise NotImplementedError("a stacked segment view needs equal segment sizes; use iter_list()")


class InputSegmentTensorManager(SegmentTensorManager):
    def __init__(self, input_tensor, seg_mode, segments, segment_size, segment_sizes=None):
        super().__init__(seg_mode, segments, segment_size, segment_sizes)
        self.input_tensor = input_tensor

    def iter_view(self):
        """(S, ..., K/S) strided view, or the stride-0 (S, ..., K) expand in weight mode."""
        x = self.input_tensor
        if self.seg_mode == "weight":
            return x.unsqueeze(0).expand(self.segments, *x.shape)
        self._need_uniform()
        return x.unflatten(-1, (self.segments, self.segment_size)).movedim(-2, 0)

    def iter_list(self):
        """Per-segment views as a list (also valid for unequal K-segments)."""
        x = self.input_tensor
        if self.seg_mode == "weight":
            return [x] * self.segments
        return [x[..., self.bounds[s]:self.bounds[s + 1]] for s in range(self.segments)]

    def total_view(self):
        return self.input_tensor.unsqueeze(0)


class WeightSegmentTensorManager(SegmentTensorManager):
    def __init__(self, weight_tensor, seg_mode, segments, segment_size, segment_sizes=None):
        super().__init__(seg_mode, segments, segment_size, segment_sizes)
        assert weight_tensor.ndim == 2, "weight tensor shape failed."
        self.out_features, self.in_features = weight_tensor.shape
        self.weight_tensor = weight_tensor  # (out, in); after real quantisation the low-bit storage
        self.packed = False                 # True: int4, two per byte, stored (N, K/2) row-major

    def device(self):
        return self.weight_tensor.device

    def to(self, device):
        self.weight_tensor = self.weight_tensor.to(device)
        return self

    def iter_view(self):
        """(S, N, K/S) in input mode, (S, N/S, K) in weight mode.  Packed int4 storage is returned
        as (S, bytes): contiguous per segment in weight mode, a copy gathered per K-slice in input
        mode (the reference keeps that case as (segments, bytes) too, :56-66)."""
        w = self.weight_tensor
        if self.packed:
            if self.seg_mode == "weight":
                return w.reshape(self.segments, -1)
            self._need_uniform()
            half = self.segment_size // 2
            return w.view(self.out_features, self.segments, half).permute(1, 0, 2).reshape(self.segments, -1)
        if self.seg_mode == "weight":
            return w.view(self.segments, self.segment_size, self.in_features)
        self._need_uniform()
        return w.view(self.out_features, self.segments, self.segment_size).permute(1, 0, 2)

    def iter_list(self):
        w = self.weight_tensor
        if self.seg_mode == "weight":
            return list(w.view(self.segments, self.segment_size, self.in_features))
        return [w[:, self.bounds[s]:self.bounds[s + 1]] for s in range(self.segments)]

    def total_view(self):
        return self.weight_tensor.unsqueeze(0)

    def replace_with_segments_layout(self, segmented_weights, packed=False):
        """Store per-segment results back as one (out, in) matrix (or (out, in/2) packed bytes)."""
        if packed:
            if self.seg_mode == "weight":
                self.weight_tensor = segmented_weights.reshape(self.out_features, self.in_features // 2)
            else:
                half = self.segment_size // 2
                self.weight_tensor = (segmented_weights.view(self.segments, self.out_features, half)
                                      .permute(1, 0, 2).reshape(self.out_features, self.in_features // 2).contiguous())
            self.packed = True
            return
        if self.seg_mode == "input":
            segmented_weights = segmented_weights.permute(1, 0, 2).contiguous()
        self.weight_tensor = segmented_weights.reshape(self.out_features, self.in_features)


def segmented_matmul(a, b):
    """a (S, ..., K) @ b (S, N, K)^T -> (S, ..., N)."""
    assert a.shape[0] == b.shape[0], "segments must match"
    bt = b.transpose(-1, -2)
    while bt.ndim < a.ndim:
        bt = bt.unsqueeze(1)
    return a @ bt
