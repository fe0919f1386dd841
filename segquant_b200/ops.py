"""torch-tensor front end of the C ABI (include/segquant_b200.h).

torch is used here only for device memory and the current stream; all arithmetic happens in the
sm_100a kernels of libsegquant_b200.so.  There is no CPU implementation: every function raises if
its tensors are not on a CUDA device.

The two functions at the bottom keep the tensor contract of the reference's pybind functions
(segquant/src/real_quant/seg_utils.h:122-161, real_gemm.cu:643-894); `seg_linear` is the fused
layer forward that SegmentLinear uses.
"""
import ctypes

import torch

from . import _lib as L

_DT = {torch.float32: L.SQ_F32, torch.float16: L.SQ_F16, torch.bfloat16: L.SQ_BF16}

# kernel_type string (f"W{weight}A{input}", segquant/layers/SegmentLinear.py:103)
#   -> (GEMM kind, activation storage, weight storage)
KERNELS = {
    "Wint8Aint8": (L.SQ_GEMM_W8A8_I8, L.SQ_Q_INT8, L.SQ_Q_INT8),
    "Wfpe4m3Afpe4m3": (L.SQ_GEMM_W8A8_F8, L.SQ_Q_E4M3, L.SQ_Q_E4M3),
    "Wint4Aint8": (L.SQ_GEMM_W4A8, L.SQ_Q_INT8, L.SQ_Q_INT4),
}

launch_count = 0  # kernels of this library launched by this process (bench.py reports it)


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("segquant_b200: tensors must live on a CUDA device (there is no CPU path)")


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"segquant_b200: unsupported floating dtype {t.dtype}") from None


def _f32(t, device):
    if not isinstance(t, torch.Tensor):
        t = torch.tensor(t, dtype=torch.float32, device=device)
    return t.to(device=device, dtype=torch.float32).contiguous()


def uniform_bounds(K, segments):
    if K % segments:
        raise ValueError(f"K={K} is not divisible into {segments} equal segments")
    step = K // segments
    return [i * step for i in range(segments + 1)]


# ---------------------------------------------------------------------------------------------
# activation quantise
# ---------------------------------------------------------------------------------------------
PRE_ACTS = {None: L.SQ_ACT_NONE, "gelu_tanh": L.SQ_ACT_GELU_TANH, "silu": L.SQ_ACT_SILU}


def quantize_act(x, bounds, sx, sx_neg=None, out_kind=L.SQ_Q_INT8, per_token=False, smooth=None,
                 out=None, out_neg=None, shared_scales=False, pre_act=None):
    """x: (B, M, K) view (any batch / row stride, K contiguous) or (M, K).

    sx: (B*S,) or (B*S*M,) float32 in (batch, segment[, row]) order, or (S,) used by every batch
    when shared_scales is set.  Returns (xq, xq_neg) uint8 tensors of shape (B, M, K) (contiguous).
    `bounds` cuts K into the S segments.  pre_act ("gelu_tanh" / "silu") applies that activation to x, in fp32,
    inside the kernel, so the activation in front of a layer costs no pass over memory of its own."""
    global launch_count
    _need_cuda(x, sx, sx_neg)
    if pre_act not in PRE_ACTS:
        raise ValueError(f"pre_act must be one of {list(PRE_ACTS)}")
    if x.dim() == 2:
        x = x.unsqueeze(0)
    if x.stride(-1) != 1:
        x = x.contiguous()
    B, M, K = x.shape
    S = len(bounds) - 1
    dual = sx_neg is not None
    xq = out if out is not None else torch.empty((B, M, K), dtype=torch.uint8, device=x.device)
    xqn = (out_neg if out_neg is not None else torch.empty((B, M, K), dtype=torch.uint8, device=x.device)) if dual else None
    if x.numel() == 0:
        return xq, xqn
    a = L.ActQuantArgs()
    a.x_dev = x.data_ptr()
    a.x_dtype = _dt(x)
    a.out_kind = out_kind
    a.batch, a.M, a.K = B, M, K
    a.x_batch_stride, a.x_row_stride = (x.stride(0) if B > 1 else 0), x.stride(1)
    a.num_segs = S
    L.set_bounds(a.seg_bounds, bounds)
    a.sx_dev = sx.data_ptr()
    a.sx_neg_dev = sx_neg.data_ptr() if dual else None
    if per_token:
        a.sx_batch_stride, a.sx_seg_stride, a.sx_row_stride = S * M, M, 1
    else:
        a.sx_batch_stride, a.sx_seg_stride, a.sx_row_stride = S, 1, 0
    if shared_scales:
        a.sx_batch_stride = 0
    a.smooth_dev = smooth.data_ptr() if smooth is not None else None
    a.pre_act = PRE_ACTS[pre_act]
    a.xq_dev = xq.data_ptr()
    a.xq_neg_dev = xqn.data_ptr() if dual else None
    a.xq_batch_stride, a.xq_row_stride = M * K, K
    with torch.cuda.device(x.device):
        L.check(L.load().sq_quantize_act(ctypes.byref(a), _stream(x)), "sq_quantize_act")
    launch_count += 1
    return xq, xqn


def norm_quantize_act(x, bounds, sx, sx_neg=None, out_kind=L.SQ_Q_INT8, shift=None, scale=None, eps=1e-6, residual=None):
    """LayerNorm(x) * (1 + scale) + shift, quantised with the static per-segment scales, in one pass over x.

    x: (B, T, K) with contiguous rows; shift / scale: (B, K) in x's dtype (or both None for a plain LayerNorm);
    sx (and sx_neg for DualScale): (S,) float32 shared by all batches.  Returns (xq, xq_neg) uint8 (B, T, K).

    residual=(gate (B, K), y (B, T, K)): the stream is first updated, x' = x + gate * y (bit-identical to torch.addcmul),
    in the same pass; returns (xq, xq_neg, x') with x' a new tensor of x's dtype."""
    global launch_count
    _need_cuda(x, sx, sx_neg, shift, scale)
    if x.dim() != 3 or x.stride(-1) != 1:
        raise ValueError("norm_quantize_act needs a (B, T, K) tensor with contiguous rows")
    B, M, K = x.shape
    dual = sx_neg is not None
    xq = torch.empty((B, M, K), dtype=torch.uint8, device=x.device)
    xqn = torch.empty((B, M, K), dtype=torch.uint8, device=x.device) if dual else None
    if x.numel() == 0:
        return (xq, xqn) if residual is None else (xq, xqn, x.clone())
    a = L.ActQuantArgs()
    a.x_dev, a.x_dtype, a.out_kind = x.data_ptr(), _dt(x), out_kind
    a.batch, a.M, a.K = B, M, K
    a.x_batch_stride, a.x_row_stride = (x.stride(0) if B > 1 else 0), x.stride(1)
    a.num_segs = len(bounds) - 1
    L.set_bounds(a.seg_bounds, bounds)
    a.sx_dev = sx.data_ptr()
    a.sx_neg_dev = sx_neg.data_ptr() if dual else None
    a.sx_batch_stride, a.sx_seg_stride, a.sx_row_stride = 0, 1, 0
    a.xq_dev = xq.data_ptr()
    a.xq_neg_dev = xqn.data_ptr() if dual else None
    a.xq_batch_stride, a.xq_row_stride = M * K, K
    mod_bs = 0
    if shift is not None:
        if shift.dtype != x.dtype or scale.dtype != x.dtype or shift.shape != (B, K) or scale.shape != (B, K):
            raise ValueError("shift / scale must be (B, K) tensors of x's dtype")
        if shift.stride(-1) != 1 or scale.stride(-1) != 1 or (B > 1 and shift.stride(0) != scale.stride(0)):
            shift, scale = shift.contiguous(), scale.contiguous()     # views with one common row stride are read in place
        mod_bs = shift.stride(0) if B > 1 else 0
    res, x_new = None, None
    if residual is not None:
        gate, y = residual
        _need_cuda(gate, y)
        if y.shape != x.shape or y.dtype != x.dtype or y.stride(-1) != 1 or gate.shape != (B, K) or gate.dtype != x.dtype:
            raise ValueError("residual=(gate (B, K), y (B, T, K)) in x's dtype, rows contiguous")
        if gate.stride(-1) != 1:
            gate = gate.contiguous()
        x_new = torch.empty((B, M, K), dtype=x.dtype, device=x.device)
        res = L.NormResidual()
        res.y_dev, res.gate_dev, res.x_out_dev = y.data_ptr(), gate.data_ptr(), x_new.data_ptr()
        res.y_batch_stride, res.y_row_stride = (y.stride(0) if B > 1 else 0), y.stride(1)
        res.gate_batch_stride = gate.stride(0) if B > 1 else 0
        res.x_out_batch_stride, res.x_out_row_stride = M * K, K
    with torch.cuda.device(x.device):
        L.check(L.load().sq_residual_norm_quantize_act(ctypes.byref(a), shift.data_ptr() if shift is not None else None,
                                                       scale.data_ptr() if scale is not None else None, mod_bs, float(eps),
                                                       ctypes.byref(res) if res is not None else None, _stream(x)),
                "sq_norm_quantize_act")
    launch_count += 1
    return (xq, xqn) if residual is None else (xq, xqn, x_new)


def gated_residual(x, gate, y, out=None):
    """x + gate.unsqueeze(1) * y for 16-bit (B, T, K) tensors x, y (contiguous rows) and a (B, K) gate, bit-identical to
    torch.addcmul; `out` may be x itself."""
    global launch_count
    _need_cuda(x, gate, y)
    if x.dim() != 3 or y.shape != x.shape or gate.shape != (x.shape[0], x.shape[2]) or x.stride(-1) != 1 or y.stride(-1) != 1:
        raise ValueError("gated_residual needs (B, T, K) tensors x, y with contiguous rows and a (B, K) gate")
    if not (x.dtype == y.dtype == gate.dtype) or x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("gated_residual: x, gate and y must share a 16-bit dtype")
    if gate.stride(-1) != 1:
        gate = gate.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device) if out is None else out
    if x.numel() == 0:
        return out
    B, M, K = x.shape
    a = L.GatedResidualArgs()
    a.x_dev, a.gate_dev, a.y_dev, a.out_dev = x.data_ptr(), gate.data_ptr(), y.data_ptr(), out.data_ptr()
    a.dtype = _dt(x)
    a.batch, a.M, a.K = B, M, K
    a.x_batch_stride, a.x_row_stride = (x.stride(0) if B > 1 else 0), x.stride(1)
    a.y_batch_stride, a.y_row_stride = (y.stride(0) if B > 1 else 0), y.stride(1)
    a.out_batch_stride, a.out_row_stride = (out.stride(0) if B > 1 else 0), out.stride(1)
    a.gate_batch_stride = gate.stride(0) if B > 1 else 0
    with torch.cuda.device(x.device):
        L.check(L.load().sq_gated_residual(ctypes.byref(a), _stream(x)), "sq_gated_residual")
    launch_count += 1
    return out


def quantize_act_dynamic(x, bounds, out_kind=L.SQ_Q_INT8, dual=False, smooth=None):
    """Per-token dynamic scales + quantise in one launch.  x (M, K).  Returns
    (xq, xq_neg, sx, sx_neg) with scales of shape (S, M).  smooth: (K,) float32 divisors, already rounded
    to x's dtype; the kernel calibrates and quantises round_dtype(x / smooth)."""
    global launch_count
    _need_cuda(x, smooth)
    if x.dim() != 2 or x.stride(-1) != 1:
        x = x.reshape(-1, x.shape[-1]).contiguous()
    M, K = x.shape
    S = len(bounds) - 1
    xq = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    xqn = torch.empty((M, K), dtype=torch.uint8, device=x.device) if dual else None
    sx = torch.empty((S, M), dtype=torch.float32, device=x.device)
    sxn = torch.empty((S, M), dtype=torch.float32, device=x.device) if dual else None
    a = L.ActQuantArgs()
    a.x_dev = x.data_ptr()
    a.x_dtype = _dt(x)
    a.out_kind = out_kind
    a.batch, a.M, a.K = 1, M, K
    a.x_batch_stride, a.x_row_stride = 0, x.stride(0)
    a.num_segs = S
    L.set_bounds(a.seg_bounds, bounds)
    a.xq_dev = xq.data_ptr()
    a.xq_neg_dev = xqn.data_ptr() if dual else None
    a.xq_batch_stride, a.xq_row_stride = M * K, K
    a.smooth_dev = smooth.data_ptr() if smooth is not None else None
    with torch.cuda.device(x.device):
        L.check(L.load().sq_quantize_act_dynamic(ctypes.byref(a), ctypes.c_void_p(sx.data_ptr()),
                                                 ctypes.c_void_p(sxn.data_ptr()) if dual else None, _stream(x)),
                "sq_quantize_act_dynamic")
    launch_count += 1
    return xq, xqn, sx, sxn


# ---------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------
def quantize_weight(w, out, scale, out_kind, group_size=0):
    """real_quantized_quantize_weights(weights, outputs, scale_w): scale is a python float, a
    (N,) tensor or, with group_size, a (N, K/group_size) tensor.  Writes into `out`."""
    global launch_count
    _need_cuda(w, out)
    if w.dim() != 2:
        raise ValueError("weights must be [N, K]")
    w = w.contiguous()
    N, K = w.shape
    if isinstance(scale, torch.Tensor):
        sc = _f32(scale, w.device)
        if group_size and sc.dim() == 2:
            mode = 2
            if sc.shape != (N, K // group_size):
                raise ValueError(f"group scale shape {tuple(sc.shape)} != {(N, K // group_size)}")
        else:
            mode = 1
            if sc.numel() != N:
                raise ValueError(f"per-channel scale has {sc.numel()} elements, expected {N}")
        scalar, ptr = 0.0, sc.data_ptr()
    else:
        mode, scalar, ptr, sc = 0, float(scale), None, None
    with torch.cuda.device(w.device):
        L.check(L.load().sq_quantize_weight(w.data_ptr(), _dt(w), N, K, mode, scalar, ptr, int(group_size or 0), out_kind,
                                            out.data_ptr(), _stream(w)), "sq_quantize_weight")
    launch_count += 1
    return out


def unpack_int4(packed, numel=None):
    global launch_count
    _need_cuda(packed)
    packed = packed.contiguous()
    numel = packed.numel() * 2 if numel is None else numel
    out = torch.empty(numel, dtype=torch.int8, device=packed.device)
    with torch.cuda.device(packed.device):
        L.check(L.load().sq_unpack_int4(packed.data_ptr(), out.data_ptr(), numel, _stream(packed)), "sq_unpack_int4")
    launch_count += 1
    return out


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def num_units(bounds, group_size=0):
    arr = (ctypes.c_int32 * len(bounds))(*[int(b) for b in bounds])
    return L.check(L.load().sq_gemm_num_units(len(bounds) - 1, arr, int(group_size or 0)), "sq_gemm_num_units")


def gemm(kind, xq, wq, N, bounds, sx, sw, *, xq_neg=None, sx_neg=None, per_token=False, group_size=0,
         sw_strides=(0, 0, 0, 1), bias=None, out_dtype=torch.float32, out=None, x_batched=True, w_seg_as_batch=False,
         y_strides=None, sx_batch_stride=None, want_acc=False, peer_outputs=None):
    """xq: (B, M, K) uint8 contiguous (or B == 1 shared by `batch` problems when x_batched=False).

    wq: weights, (Bw, N, K) bytes or (Bw, N, K/2) packed int4, contiguous.
    sw_strides = (batch, segment, group, column) element strides into `sw`."""
    global launch_count
    _need_cuda(xq, wq, sx, sw, bias)
    Bx, M, K = xq.shape
    Bw = wq.shape[0]
    batch = 1 if w_seg_as_batch else max(Bx, Bw)
    S = len(bounds) - 1
    w4 = kind == L.SQ_GEMM_W4A8
    a = L.GemmArgs()
    a.kind = kind
    a.out_dtype = _DT[out_dtype]
    a.batch, a.M, a.N, a.K = batch, M, N, K
    a.xq_dev = xq.data_ptr()
    a.xq_neg_dev = xq_neg.data_ptr() if xq_neg is not None else None
    a.xq_batch_stride = M * K if (x_batched and Bx > 1) else 0
    a.xq_row_stride = K
    a.wq_dev = wq.data_ptr()
    Kw = (bounds[1] - bounds[0]) if w_seg_as_batch else K
    a.wq_row_stride = Kw // 2 if w4 else Kw
    a.wq_batch_stride = N * a.wq_row_stride if Bw > 1 else 0
    a.w_seg_as_batch = 1 if w_seg_as_batch else 0
    a.num_segs = S
    L.set_bounds(a.seg_bounds, bounds)
    a.group_size = int(group_size or 0)
    a.sw_is_bf16 = 1 if sw.dtype == torch.bfloat16 else 0
    if sw.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("weight scales must be float32 or bfloat16")
    a.sx_dev = sx.data_ptr()
    a.sx_neg_dev = sx_neg.data_ptr() if sx_neg is not None else None
    if per_token:
        a.sx_batch_stride, a.sx_seg_stride, a.sx_row_stride = S * M, M, 1
    else:
        a.sx_batch_stride, a.sx_seg_stride, a.sx_row_stride = S, 1, 0
    if sx_batch_stride is not None:
        a.sx_batch_stride = sx_batch_stride
    a.sw_dev = sw.data_ptr()
    a.sw_batch_stride, a.sw_seg_stride, a.sw_group_stride, a.sw_col_stride = sw_strides
    if bias is not None:
        a.bias_dev = bias.data_ptr()
        a.bias_dtype = _dt(bias)
    a.bias_batch_stride = 0
    y = out if out is not None else torch.empty((batch, M, N), dtype=out_dtype, device=xq.device)
    a.y_dev = y.data_ptr()
    a.y_batch_stride, a.y_row_stride = y_strides if y_strides is not None else (M * N, N)
    if peer_outputs is not None:
        # fused all-gather: (device pointers of the peers' [M, *] buffers, row stride, column offset) in elements
        ptrs, prs, pco = peer_outputs
        if len(ptrs) > L.SQ_MAX_PEERS:
            raise ValueError(f"at most {L.SQ_MAX_PEERS} peer outputs")
        a.num_peer_outputs = len(ptrs)
        for j, ptr in enumerate(ptrs):
            a.peer_y_dev[j] = int(ptr)
        a.peer_row_stride, a.peer_col_offset = int(prs), int(pco)
    acc = None
    if want_acc:
        units = num_units(bounds, group_size)
        sides = 2 if xq_neg is not None else 1
        acc = torch.zeros((batch, units, sides, M, N), dtype=torch.int32, device=xq.device)
        a.acc_dump_dev = acc.data_ptr()
    with torch.cuda.device(xq.device):
        L.check(L.load().sq_gemm(ctypes.byref(a), _stream(xq)), "sq_gemm")
    launch_count += 1
    return (y, acc) if want_acc else y


def device_status():
    """Synchronise and return the word kernels write when a bounded wait gave up (0 = fine)."""
    return int(L.load().sq_device_status())


def push_columns(block, peer_ptrs, peer_row_stride_bytes):
    """Copy the 2-D view `block` ([rows, width], a column block inside this rank's result matrix, last dim contiguous) to
    the device addresses peer_ptrs (the block's position inside each peer GPU's matrix, mapped into this process)."""
    global launch_count
    _need_cuda(block)
    if block.dim() != 2 or block.stride(1) != 1:
        raise ValueError("push_columns needs a [rows, width] view with a contiguous last dim")
    if not peer_ptrs:
        return
    esz = block.element_size()
    arr = (ctypes.c_void_p * len(peer_ptrs))(*[int(p) for p in peer_ptrs])
    with torch.cuda.device(block.device):
        L.check(L.load().sq_push_columns(block.data_ptr(), block.shape[0], block.shape[1] * esz, block.stride(0) * esz, len(peer_ptrs),
                                         arr, int(peer_row_stride_bytes), _stream(block)), "sq_push_columns")
    launch_count += 1


def peer_barrier(rank, flag_ptrs, epoch, device):
    """Stream-ordered barrier over flag words in peer-mapped memory (sq_peer_barrier): flag_ptrs[j] = device address of
    rank j's array of len(flag_ptrs) uint32 words, epoch = number of this collective call (1, 2, ...)."""
    global launch_count
    world = len(flag_ptrs)
    if world == 1:
        return
    arr = (ctypes.c_void_p * world)(*[int(p) for p in flag_ptrs])
    with torch.cuda.device(device):
        L.check(L.load().sq_peer_barrier(int(rank), world, arr, int(epoch) & 0xFFFFFFFF,
                                         ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)), "sq_peer_barrier")
    launch_count += 1


def check_device():
    """Synchronise and raise SegQuantError(SQ_ERR_DEVICE_TIMEOUT) if a kernel reported a bounded wait that ran out."""
    L.check(L.load().sq_check_device(), "sq_check_device")


def set_gemm_schedule(bn=0, two_cta=-1, ksub=0, no_gemv=0):
    """Force the GEMM schedule process-wide (0 / -1 = automatic); results do not depend on it.  Test and tuning aid."""
    L.check(L.load().sq_set_gemm_schedule(int(bn), int(two_cta), int(ksub), int(no_gemv)), "sq_set_gemm_schedule")


# ---------------------------------------------------------------------------------------------
# fused layer forward
# ---------------------------------------------------------------------------------------------
def seg_linear(kernel_type, x, wq, N, bounds, sx, sw, *, sx_neg=None, dynamic=False, group_size=0,
               sw_strides=(0, 0, 0, 1), bias=None, smooth=None, w_seg_as_batch=False, out_dtype=None, out=None,
               peer_outputs=None):
    """SegmentLinear.forward on the real-quant path in two launches: quantise x [.., K] with the
    per-K-segment (or DualScale, or dynamic per-token) scales, then one GEMM that sums the
    segments in fp32 registers, adds the bias and casts.  Returns [.., N] in x.dtype."""
    kind, a_kind, _ = KERNELS[kernel_type]
    lead = x.shape[:-1]
    K = x.shape[-1]
    out_dtype = out_dtype or x.dtype
    dual = sx_neg is not None
    if out is not None:
        # write straight into a caller-provided (B, M, N) view (any batch / row stride, N contiguous), e.g. a slice of
        # a joint token buffer: one problem per batch entry, all sharing the weight matrix
        if dynamic or x.dim() != 3 or out.dim() != 3 or out.stride(-1) != 1 or out.shape[:2] != x.shape[:2] or out.shape[2] != N:
            raise ValueError("out= needs a static-scale (B, M, K) input and a (B, M, N) output view with a contiguous last dim")
        xq, xqn = quantize_act(x if x.stride(-1) == 1 else x.contiguous(), bounds, sx, sx_neg, a_kind, smooth=smooth, shared_scales=True)
        gemm(kind, xq, wq, N, bounds, sx, sw, xq_neg=xqn, sx_neg=sx_neg, group_size=group_size, sw_strides=sw_strides, bias=bias,
             out_dtype=out.dtype, out=out, y_strides=(out.stride(0), out.stride(1)), sx_batch_stride=0, w_seg_as_batch=w_seg_as_batch,
             peer_outputs=peer_outputs)
        return out
    if peer_outputs is not None:
        raise ValueError("peer_outputs needs out= (a (1, M, N) view of this rank's own buffer)")
    if x.dim() == 3 and x.stride(-1) == 1 and not x.is_contiguous() and not dynamic:
        # a strided (B, M, K) view (e.g. a token slice of a joint sequence): the quantise kernel reads it
        # in place and writes contiguous bytes, so no copy of x is made
        xq, xqn = quantize_act(x, bounds, sx, sx_neg, a_kind, smooth=smooth, shared_scales=True)
        rows = xq.shape[0] * xq.shape[1]
        y = gemm(kind, xq.view(1, rows, K), wq, N, bounds, sx, sw, xq_neg=None if xqn is None else xqn.view(1, rows, K),
                 sx_neg=sx_neg, group_size=group_size, sw_strides=sw_strides, bias=bias, out_dtype=out_dtype,
                 w_seg_as_batch=w_seg_as_batch)
        return y.reshape(*lead, N)
    x2 = x.reshape(-1, K)
    if dynamic:
        xq, xqn, sxd, sxnd = quantize_act_dynamic(x2, bounds, a_kind, dual=dual, smooth=smooth)
        y = gemm(kind, xq.unsqueeze(0), wq, N, bounds, sxd, sw, xq_neg=xqn, sx_neg=sxnd, per_token=True,
                 group_size=group_size, sw_strides=sw_strides, bias=bias, out_dtype=out_dtype,
                 w_seg_as_batch=w_seg_as_batch)
    else:
        xq, xqn = quantize_act(x2, bounds, sx, sx_neg, a_kind, smooth=smooth)
        y = gemm(kind, xq, wq, N, bounds, sx, sw, xq_neg=xqn, sx_neg=sx_neg, group_size=group_size,
                 sw_strides=sw_strides, bias=bias, out_dtype=out_dtype, w_seg_as_batch=w_seg_as_batch)
    return y.reshape(*lead, N)


# ---------------------------------------------------------------------------------------------
# the reference's pybind functions
# ---------------------------------------------------------------------------------------------
def _segment_batches(inputs):
    """Classify the (S, ..., M, K) input of the reference contract without copying it.
    Returns (x3 (B, M, K) view, shared) where shared=True means all S batches are the same
    (a stride-0 expand, segquant/layers/segment_tensor_manager.py:21-23)."""
    S, K = inputs.shape[0], inputs.shape[-1]
    if inputs.stride(0) == 0 and S >= 1:
        first = inputs[0]
        first = first.reshape(-1, K) if first.is_contiguous() else first.contiguous().view(-1, K)
        return first.unsqueeze(0), True
    if inputs.dim() == 3 and inputs.stride(-1) == 1:
        return inputs, False  # (S, M, K) with arbitrary batch / row stride: the kernel takes it as is
    if inputs.dim() > 3 and inputs.stride(-1) == 1:
        try:
            return inputs.view(S, -1, K), False
        except RuntimeError:
            pass
    return inputs.contiguous().view(S, -1, K), False


def real_quantized_gemm_scaled(kernel_type, inputs, weights, scale_x, scale_w, neg_scale_x=None):
    """`{P}_real_quantized_gemm_scaled(inputs, weights, scale_x, scale_w)` and, when neg_scale_x is
    given (scale_x then being the positive scale), `{P}_real_quantized_gemm_dual_scaled`.

    inputs (S, ..., M, K) float; weights (S, N, K) int8 / uint8-as-e4m3 or (S, N*K/2) packed int4;
    scales float32 with S or S*M (x) and S or S*N (w) elements.  Returns a new (S, ..., M, N)
    tensor in the input dtype, un-summed and without bias (real_gemm.cu:644-687)."""
    kind, a_kind, _ = KERNELS[kernel_type]
    _need_cuda(inputs, weights)
    S, K = inputs.shape[0], inputs.shape[-1]
    lead = tuple(inputs.shape[1:-1])
    x3, shared = _segment_batches(inputs)
    M = x3.shape[1]
    if weights.shape[0] != S:
        raise RuntimeError(f"weights have {weights.shape[0]} segments, inputs {S}")
    weights = weights.contiguous()
    if kind == L.SQ_GEMM_W4A8:
        N = weights.shape[1] * 2 // K   # real_gemm.cu:670
        w3 = weights.view(S, N, K // 2)
    else:
        N = weights.shape[1]
        w3 = weights.view(S, N, K)
    dev = inputs.device
    sx = _f32(scale_x, dev).reshape(-1)
    sxn = _f32(neg_scale_x, dev).reshape(-1) if neg_scale_x is not None else None
    sw = _f32(scale_w, dev).reshape(-1)
    per_token = sx.numel() != S          # real_gemm.cu:703
    if per_token and sx.numel() != S * M:
        raise RuntimeError(f"scale_x has {sx.numel()} elements, expected {S} or {S * M}")
    w_scalar = sw.numel() == S           # real_gemm.cu:743
    if not w_scalar and sw.numel() != S * N:
        raise RuntimeError(f"scale_w has {sw.numel()} elements, expected {S} or {S * N}")
    sw_strides = (1, 0, 0, 0) if w_scalar else (N, 0, 0, 1)
    bounds = [0, K]
    if shared:
        # a stride-0 expand: every batch re-reads the same rows (its scales may differ), nothing is copied
        x3 = x3.expand(S, M, K)
    xq, xqn = quantize_act(x3, bounds, sx, sxn, a_kind, per_token=per_token)
    y = gemm(kind, xq, w3, N, bounds, sx, sw, xq_neg=xqn, sx_neg=sxn, per_token=per_token, sw_strides=sw_strides,
             out_dtype=inputs.dtype)
    return y.view(S, *lead, N)
