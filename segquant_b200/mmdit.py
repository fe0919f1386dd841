"""Synthetic SD3.5-medium-like MMDiT denoise step built from real-quantized SegmentLinear layers.

Architecture (random-init weights ~ N(0, 0.02), no checkpoint): 24 joint blocks, hidden 1536,
24 heads of 64, MLP ratio 4, 4096 image tokens + 333 text tokens.  The block structure follows the
reference's vendored SD3 transformer: JointTransformerBlock (backend/torch/layers/attention.py:476-679),
AdaLayerNormZero (backend/torch/layers/normalization.py:322-380: SiLU -> Linear(H, 6H) -> chunk(6)),
AdaLayerNormContinuous (:271-317), the embedders of backend/torch/layers/embeddings.py:973-1071, and the
output head of backend/torch/modules/transformer_sd3.py:90-156.

Every nn.Linear is a W8A8 INT8 SegmentLinear with the segmentation the reference's pattern detector
would give it (segquant/pattern_detector.py:239-358):
  * adaLN modulation linears: N-segmented into their 6 (or 2) output chunks, DualScale input (after SiLU);
  * ff.net[2] (after GELU-tanh) and the second embedder linears (after SiLU): DualScale input;
  * attention output projections: S = 1 by default, or 24 K-segments of 64 (`out_proj_segments=24`,
    the reshape_to_linear pattern: heads x head_dim);
  * everything else: S = 1.
Attention (torch SDPA) stays bf16.  Scales are calibrated once from one forward of the float model on the
given inputs (AMax), then every layer runs the fused quantise + tcgen05 GEMM path; where a LayerNorm + adaLN
modulation feeds linears, one kernel normalises, modulates and quantises (FusedNorm below), q / k / v of a stream
run as one GEMM on those bytes, the GELU in front of the MLP down-projection is evaluated inside its quantise kernel,
and the gated residual updates use this library's vectorised kernel.
"""
import math

import torch
import torch.nn.functional as F

from .layers.SegmentLinear import SegmentLinear


class QLinear:
    """A float linear that becomes a real-quantized SegmentLinear after one calibration forward."""

    def __init__(self, in_f, out_f, gen, device, dtype, seg_mode="weight", chunks=1, dual=False, bias=True, act="int8", wq="int8"):
        self.in_f, self.out_f, self.seg_mode, self.chunks, self.dual = in_f, out_f, seg_mode, chunks, dual
        self.act, self.wq = act, wq
        self.w = (torch.randn(out_f, in_f, generator=gen, dtype=torch.float32) * 0.02).to(dtype).to(device)
        self.b = (torch.randn(out_f, generator=gen, dtype=torch.float32) * 0.01).to(dtype).to(device) if bias else None
        self.layer = None
        self.device = device

    def calibrate_forward(self, x):
        self.layer = SegmentLinear(
            self.in_f, self.out_f, bias=self.b is not None, seg_mode=self.seg_mode, chunks=self.chunks,
            custom_weight_tensor=self.w, custom_bias_tensor=self.b, input_quant_type=self.act, weight_quant_type=self.wq,
            input_quant_args={"real_quant": True, "axis": None, "dual_scale": self.dual},
            weight_quant_args={"real_quant": True, "axis": 1}, device=self.device)
        self.layer.calibrate(x)
        return F.linear(x, self.w, self.b)

    def finish(self):
        self.layer.finish_calibrate()
        self.w = None   # the float weight is no longer needed

    fuse_activation = True     # class-wide switch: False runs the activation in front of a layer as its own torch kernel

    def __call__(self, x, out=None, pre_act=None):
        """pre_act ("gelu_tanh" / "silu"): the layer's input is pre_act(x); the quantise kernel evaluates it on the fly."""
        if pre_act is None:
            return self.layer(x, out=out)
        if self.fuse_activation:
            try:
                bounds, sx, sx_neg, kind = self.layer.optimizer.input_quant_params()
            except RuntimeError:
                bounds = None
            if bounds is not None:
                from . import ops
                x3 = x if x.dim() == 3 else x.reshape(1, -1, x.shape[-1])
                xq, xq_neg = ops.quantize_act(x3, bounds, sx, sx_neg, kind, shared_scales=True, pre_act=pre_act)
                y = self.layer.forward_quantized(xq, xq_neg, out=out, out_dtype=x.dtype)
                return y if out is not None else y.reshape(*x.shape[:-1], self.out_f)
        return self.layer(_ACTS[pre_act](x), out=out)


_ACTS = {"gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "silu": F.silu}


def _layer_norm(x):
    return F.layer_norm(x, (x.shape[-1],), eps=1e-6)


def _modulate(x, shift, scale):
    """LayerNorm(x) * (1 + scale) + shift; shift / scale are (B, H) or None."""
    n = _layer_norm(x)
    return n if shift is None else torch.addcmul(shift.unsqueeze(1), n, 1 + scale.unsqueeze(1))


def _gated_add(x, gate, y):
    """x + gate[:, None, :] * y, the residual-stream update; on the GPU one vectorised kernel of this library (bit-identical
    to torch.addcmul, which takes a slow strided path for the broadcast gate)."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.stride(-1) == 1 and y.stride(-1) == 1:
        from . import ops
        return ops.gated_residual(x, gate, y)
    return torch.addcmul(x, gate.unsqueeze(1), y)


class FusedNorm:
    """Runs `layers` on LayerNorm(x) * (1 + scale) + shift.  Linears that were calibrated on the same tensor hold the
    same static input scale, so the normalisation, the modulation and the quantisation are done once, in one kernel that
    reads x once and writes bytes (ops.norm_quantize_act), and every layer's GEMM consumes those bytes.  Groups whose
    layers do not share their quantisation parameters (or whose rows are too long for the kernel) take the unfused path;
    the decision is made on the first call, outside any graph capture, and cached."""

    MAX_ROW_BYTES = 4096

    def __init__(self, merge_gemms=True, fuse_residual=True):
        self.plan = {}
        self.merge_gemms = merge_gemms
        self.fuse_residual = fuse_residual

    def _params(self, layers, x):
        key = tuple(id(l) for l in layers)
        if key not in self.plan:
            self.plan[key] = None
            try:
                ps = [l.layer.optimizer.input_quant_params() for l in layers]
            except RuntimeError:
                return None
            b0, sx0, sn0, k0 = ps[0]
            same = all(list(b) == list(b0) and k == k0 and torch.equal(sx, sx0) and (sn is None) == (sn0 is None)
                       and (sn is None or torch.equal(sn, sn0)) for b, sx, sn, k in ps[1:])
            if same and x.shape[-1] * x.element_size() <= self.MAX_ROW_BYTES:
                self.plan[key] = ps[0]
        return self.plan[key]

    def _merged(self, layers, outs):
        """Layers that share their quantised input and write side by side into one buffer (q / k / v) run as ONE GEMM over
        the concatenated weight rows: three launches of 384 tiles each (2.6 rounds of the 148 SMs, the last one 59 % full)
        become one of 1152 (7.8 rounds).  Returns the concatenated operands, or None when the layers or `outs` do not fit."""
        from . import ops
        if len(layers) < 2 or any(o is None for o in outs):
            return None
        key = ("merged",) + tuple(id(l) for l in layers)
        if key not in self.plan:
            self.plan[key] = None
            opts = [l.layer.optimizer for l in layers]
            fs = [o._fused for o in opts]
            N = fs[0]["N"]
            biases = [l.layer.bias_data if l.layer.bias else None for l in layers]
            ok = all(f["group"] == 0 and tuple(f["sw_strides"]) == (0, 0, 0, 1) and f["sw"].numel() == f["N"] == N
                     and f["wq"].shape == fs[0]["wq"].shape and f["sw"].dtype == fs[0]["sw"].dtype for f in fs)
            ok = ok and len({o.kernel_type for o in opts}) == 1 and len({b is None for b in biases}) == 1
            if ok:
                self.plan[key] = dict(
                    wq=torch.cat([f["wq"] for f in fs], dim=1).contiguous(), sw=torch.cat([f["sw"] for f in fs]).contiguous(),
                    bias=None if biases[0] is None else torch.cat(biases).contiguous(), N=N * len(layers), n=N,
                    kind=ops.KERNELS[opts[0].kernel_type][0])
        m = self.plan[key]
        if m is None:
            return None
        o0 = outs[0]
        for j, o in enumerate(outs):       # consecutive column blocks of one buffer
            if o.shape != o0.shape or o.stride() != o0.stride() or o.data_ptr() != o0.data_ptr() + j * m["n"] * o.element_size():
                return None
        if o0.dim() != 3 or o0.stride(2) != 1 or o0.stride(1) < m["N"]:
            return None
        return m

    def __call__(self, layers, x, shift, scale, outs=None, residual=None):
        """Returns (outputs, x'): residual=(gate, y) first updates the stream, x' = x + gate * y, inside the same kernel."""
        from . import ops
        outs = outs or [None] * len(layers)
        p = self._params(layers, x)
        if p is None or (residual is not None and not self.fuse_residual):
            if residual is not None:
                x = _gated_add(x, *residual)
                residual = None
        if p is None:
            n = _modulate(x, shift, scale)
            return [l(n, out=o) for l, o in zip(layers, outs)], x
        bounds, sx, sx_neg, kind = p
        if residual is None:
            xq, xq_neg = ops.norm_quantize_act(x, bounds, sx, sx_neg, out_kind=kind, shift=shift, scale=scale)
        else:
            xq, xq_neg, x = ops.norm_quantize_act(x, bounds, sx, sx_neg, out_kind=kind, shift=shift, scale=scale, residual=residual)
        m = self._merged(layers, outs) if self.merge_gemms else None
        if m is not None:
            o0 = outs[0]
            joint = torch.as_strided(o0, (o0.shape[0], o0.shape[1], m["N"]), o0.stride())
            ops.gemm(m["kind"], xq, m["wq"], m["N"], bounds, sx, m["sw"], xq_neg=xq_neg, sx_neg=sx_neg, bias=m["bias"],
                     out_dtype=joint.dtype, out=joint, y_strides=(joint.stride(0), joint.stride(1)), sx_batch_stride=0)
            return list(outs), x
        return [l.layer.forward_quantized(xq, xq_neg, out=o, out_dtype=x.dtype) for l, o in zip(layers, outs)], x


def _timestep_embedding(t, dim=256):
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class _SideStream:
    """Second CUDA stream for the text branch of a joint block.  The text stream has 333 tokens against 4096 image tokens:
    its kernels are a few CTAs each and, run in line, cost their launch and pipeline latency 20 times per block for 7 % of the
    work.  On their own stream they fill the SMs that the image branch's persistent kernels leave idle in their last round of
    tiles.  fork(): the side stream waits for everything enqueued on the current stream; join(): the current stream waits for
    the side stream.  Both are plain events, so the pattern is captured into a CUDA graph as fork / join edges."""

    def __init__(self, device):
        self.stream = torch.cuda.Stream(device)

    def fork(self):
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.stream.wait_event(ev)

    def join(self):
        ev = torch.cuda.Event()
        ev.record(self.stream)
        torch.cuda.current_stream().wait_event(ev)

    def ctx(self):
        return torch.cuda.stream(self.stream)


class _InLine:
    """Stand-in for _SideStream that runs the text branch in line (calibration pass, single-stream mode)."""

    def fork(self):
        pass

    def join(self):
        pass

    def ctx(self):
        import contextlib
        return contextlib.nullcontext()


class JointBlock:
    def __init__(self, hidden, heads, gen, device, dtype, last, out_proj_segments):
        self.heads, self.last = heads, last
        mk = lambda i, o, **kw: QLinear(i, o, gen, device, dtype, **kw)  # noqa: E731
        self.norm1 = mk(hidden, 6 * hidden, chunks=6, dual=True)
        self.norm1_context = mk(hidden, (2 if last else 6) * hidden, chunks=2 if last else 6, dual=True)
        self.to_q, self.to_k, self.to_v = mk(hidden, hidden), mk(hidden, hidden), mk(hidden, hidden)
        self.add_q, self.add_k, self.add_v = mk(hidden, hidden), mk(hidden, hidden), mk(hidden, hidden)
        seg = dict(seg_mode="input", chunks=out_proj_segments) if out_proj_segments > 1 else {}
        self.to_out = mk(hidden, hidden, **seg)
        self.ff0, self.ff2 = mk(hidden, 4 * hidden), mk(4 * hidden, hidden, dual=True)
        if not last:
            self.to_add_out = mk(hidden, hidden, **seg)
            self.ffc0, self.ffc2 = mk(hidden, 4 * hidden), mk(4 * hidden, hidden, dual=True)

    def linears(self):
        names = ["norm1", "norm1_context", "to_q", "to_k", "to_v", "add_q", "add_k", "add_v", "to_out", "ff0", "ff2"]
        if not self.last:
            names += ["to_add_out", "ffc0", "ffc2"]
        return [getattr(self, n) for n in names]

    def forward(self, img, txt, c_act, call, norm_call, pend_img=None, pend_txt=None, side=None):
        """c_act = SiLU(conditioning) [B, H]; call(layer, x, out=None, pre_act=None) runs either the calibration or the
        quantized linear on pre_act(x), writing into `out` when given; norm_call(layers, x, shift, scale, outs, residual)
        first applies the pending gated residual (gate, y) to the stream x, then runs `layers` on the normalised and
        modulated x, and returns (outputs, updated x).  pend_* are the residuals the previous block left unapplied;
        the block returns its own (of the MLP) the same way, so every residual update rides on the next normalisation.
        side: a _SideStream for the text branch (None = in line).  The fifth return value holds the tensors that cross
        between the two streams; the caller keeps it alive until the next block has joined the streams again, so the
        caching allocator cannot hand their memory out while the other stream may still use it."""
        side = side or _InLine()
        B, Ti, H = img.shape
        Tt = txt.shape[1]
        # the six projections write straight into their token range of one joint buffer, q | k | v side by side per
        # token, so the three projections of a stream can be one GEMM of 3 H columns
        qkv = torch.empty((B, Ti + Tt, 3, H), dtype=img.dtype, device=img.device)
        side.fork()                                                          # qkv's memory and c_act are the main stream's
        with side.ctx():
            mc = call(self.norm1_context, c_act).chunk(2 if self.last else 6, dim=-1)
            _, txt = norm_call((self.add_q, self.add_k, self.add_v), txt, mc[0], mc[1], [qkv[:, Ti:, j] for j in range(3)], pend_txt)
        m = call(self.norm1, c_act).chunk(6, dim=-1)                         # shift, scale, gate (msa), shift, scale, gate (mlp)
        _, img = norm_call((self.to_q, self.to_k, self.to_v), img, m[0], m[1], [qkv[:, :Ti, j] for j in range(3)], pend_img)
        side.join()

        def heads(t):
            return t.view(B, Ti + Tt, self.heads, H // self.heads).transpose(1, 2)

        a = F.scaled_dot_product_attention(heads(qkv[:, :, 0]), heads(qkv[:, :, 1]), heads(qkv[:, :, 2]))
        a = a.transpose(1, 2).reshape(B, Ti + Tt, H)
        a_img, a_txt = a[:, :Ti], a[:, Ti:]
        side.fork()

        pend_txt = None
        if not self.last:
            with side.ctx():
                (h,), txt = norm_call((self.ffc0,), txt, mc[3], mc[4], None, (mc[2], call(self.to_add_out, a_txt)))
                pend_txt = (mc[5], call(self.ffc2, h, pre_act="gelu_tanh"))
        (h,), img = norm_call((self.ff0,), img, m[3], m[4], None, (m[2], call(self.to_out, a_img)))
        pend_img = (m[5], call(self.ff2, h, pre_act="gelu_tanh"))
        return img, txt, pend_img, pend_txt, (qkv, a)


def calibration_calls():
    """(call, norm_call) for JointBlock.forward that run the FLOAT linears and let each one record its input range."""
    def calib(layer, x, out=None, pre_act=None):
        y = layer.calibrate_forward(x if pre_act is None else _ACTS[pre_act](x))
        if out is not None:
            out.copy_(y)
            return out
        return y

    def calib_norm(layers, x, shift, scale, outs=None, residual=None):
        if residual is not None:
            x = _gated_add(x, *residual)
        n = _modulate(x, shift, scale)
        return [calib(l, n, o) for l, o in zip(layers, outs or [None] * len(layers))], x
    return calib, calib_norm


def quantized_calls(fused_norm=None):
    """(call, norm_call) for JointBlock.forward that run the quantized linears; fused_norm: a FusedNorm, or None to run
    layer_norm / modulation / quantise / gated residual as separate kernels."""
    def unfused(layers, x, shift, scale, outs=None, residual=None):
        if residual is not None:
            x = _gated_add(x, *residual)
        n = _modulate(x, shift, scale)
        return [l(n, out=o) for l, o in zip(layers, outs or [None] * len(layers))], x
    return (lambda layer, x, out=None, pre_act=None: layer(x, out=out, pre_act=pre_act)), (fused_norm or unfused)


class SyntheticMMDiT:
    def __init__(self, device, blocks=24, hidden=1536, heads=24, img_tokens=4096, txt_tokens=333, seed=0,
                 dtype=torch.bfloat16, out_proj_segments=1):
        gen = torch.Generator().manual_seed(seed)
        self.device, self.dtype, self.hidden = device, dtype, hidden
        self.img_tokens, self.txt_tokens = img_tokens, txt_tokens
        mk = lambda i, o, **kw: QLinear(i, o, gen, device, dtype, **kw)  # noqa: E731
        self.context_embedder = mk(4096, hidden)
        self.t_lin1, self.t_lin2 = mk(256, hidden), mk(hidden, hidden, dual=True)
        self.p_lin1, self.p_lin2 = mk(2048, hidden), mk(hidden, hidden, dual=True)
        self.blocks = [JointBlock(hidden, heads, gen, device, dtype, last=(i == blocks - 1), out_proj_segments=out_proj_segments)
                       for i in range(blocks)]
        self.norm_out = mk(hidden, 2 * hidden, chunks=2, dual=True)
        self.proj_out = mk(hidden, 64)
        self.calibrated = False
        self.fused_norm = FusedNorm()      # set to None to run layer_norm / modulation / quantise as separate kernels
        self.two_streams = True            # text branch on a second CUDA stream (quantized path on a GPU only)
        self._side = None

    def linears(self):
        out = [self.context_embedder, self.t_lin1, self.t_lin2, self.p_lin1, self.p_lin2]
        for b in self.blocks:
            out += b.linears()
        return out + [self.norm_out, self.proj_out]

    def _forward(self, latents, text, pooled, timestep, call, norm_call, side=None):
        """latents [B, Ti, H] (already patch-embedded: the patch embedder is a Conv2d, never quantised),
        text [B, Tt, 4096], pooled [B, 2048], timestep [B]."""
        temb = call(self.t_lin2, call(self.t_lin1, _timestep_embedding(timestep).to(self.dtype)), pre_act="silu")
        pemb = call(self.p_lin2, call(self.p_lin1, pooled), pre_act="silu")
        c_act = F.silu(temb + pemb)
        txt = call(self.context_embedder, text)
        img = latents
        pend_img = pend_txt = None
        keep = None                                                          # see JointBlock.forward
        for blk in self.blocks:
            img, txt, pend_img, pend_txt, keep = blk.forward(img, txt, c_act, call, norm_call, pend_img, pend_txt, side)
        if side is not None:
            side.join()
        del keep
        mod = call(self.norm_out, c_act).chunk(2, dim=-1)                    # scale, shift
        return norm_call((self.proj_out,), img, mod[1], mod[0], None, pend_img)[0][0]

    def calibrate(self, latents, text, pooled, timestep):
        """One forward of the float model; every linear records its input range and is then quantized."""
        with torch.no_grad():
            calib, calib_norm = calibration_calls()
            y = self._forward(latents, text, pooled, timestep, calib, calib_norm)
            for lin in self.linears():
                lin.finish()
        self.calibrated = True
        return y

    def __call__(self, latents, text, pooled, timestep):
        if not self.calibrated:
            raise RuntimeError("call calibrate() once before running the quantized model")
        with torch.no_grad():
            call, norm_call = quantized_calls(self.fused_norm)
            side = None
            if self.two_streams and latents.is_cuda:
                if self._side is None:
                    self._side = _SideStream(latents.device)
                side = self._side
            return self._forward(latents, text, pooled, timestep, call, norm_call, side)

    def linear_ops(self, batch):
        """Useful operations 2*M*N*K of one step, summed over every quantized linear."""
        total = 0
        small = {id(l) for l in (self.t_lin1, self.t_lin2, self.p_lin1, self.p_lin2, self.norm_out)}
        txt_side = {id(self.context_embedder)}
        for blk in self.blocks:
            small |= {id(blk.norm1), id(blk.norm1_context)}
            txt_side |= {id(l) for l in (blk.add_q, blk.add_k, blk.add_v)}
            if not blk.last:
                txt_side |= {id(l) for l in (blk.to_add_out, blk.ffc0, blk.ffc2)}
        for lin in self.linears():
            rows = batch if id(lin) in small else batch * (self.txt_tokens if id(lin) in txt_side else self.img_tokens)
            total += 2 * rows * lin.in_f * lin.out_f
        return total


class GraphedStep:
    """The quantized denoise step captured once into a CUDA graph and replayed: a step is well over a thousand small
    launches (two per linear plus the bf16 glue), so launch overhead dominates when they are issued one by
    one from Python.  Inputs are copied into static buffers; the output tensor is reused by every replay."""

    def __init__(self, model, latents, text, pooled, timestep, warmup=2):
        self.static_in = [t.clone() for t in (latents, text, pooled, timestep)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):            # first calls build per-layer caches and set kernel attributes
                model(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from . import ops
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(self.graph):
            self.static_out = model(*self.static_in)
        self.launches_per_replay = ops.launch_count - before   # this library's kernels recorded in the graph

    def __call__(self, latents=None, text=None, pooled=None, timestep=None):
        for dst, src in zip(self.static_in, (latents, text, pooled, timestep)):
            if src is not None and src is not dst:
                dst.copy_(src, non_blocking=True)
        from . import ops
        self.graph.replay()
        ops.launch_count += self.launches_per_replay
        return self.static_out


def synthetic_inputs(batch, device, dtype=torch.bfloat16, img_tokens=4096, txt_tokens=333, hidden=1536, seed=0):
    g = torch.Generator().manual_seed(seed)
    latents = torch.randn(batch, img_tokens, hidden, generator=g).to(dtype).to(device)
    text = torch.randn(batch, txt_tokens, 4096, generator=g).to(dtype).to(device)
    pooled = torch.randn(batch, 2048, generator=g).to(dtype).to(device)
    timestep = torch.full((batch,), 500.0, device=device)
    return latents, text, pooled, timestep
