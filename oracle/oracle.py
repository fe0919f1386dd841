"""numpy front end of the CPU oracle (oracle/segquant_oracle.c) -- TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may import
this module.  It restates, on the CPU, what the reference's native layer computes:

* quantize_act / quantize_weight / unpack_int4   -- segquant/src/real_quant/quantizer.cuh:13-206
* seg_gemm                                       -- segquant/src/real_quant/real_gemm.cu:643-894 with
                                                    dequantizer.cuh:8-73 and SegmentLinear.py:238-241
* real_quantized_gemm_scaled / _dual_scaled      -- the pybind functions of seg_utils.h:122-161, with
                                                    their (S, ..., M, K) / (S, N, K) tensor contract
* calibrate_* (scale definitions)                -- segquant/quantizers/quantizer.py:161-248, :398-452

Parity pin: see the header of segquant_oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

Q_INT8, Q_E4M3, Q_INT4 = 0, 1, 2
GEMM_I8, GEMM_F8, GEMM_W4A8 = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    """Compile oracle/liboracle.so with gcc if it is missing or older than its source."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "segquant_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return so


def _lib():
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(build())
        lib.sqo_e4m3_from_float.restype = ctypes.c_uint8
        lib.sqo_e4m3_from_float.argtypes = [ctypes.c_float]
        lib.sqo_e4m3_to_float.restype = ctypes.c_float
        lib.sqo_e4m3_to_float.argtypes = [ctypes.c_uint8]
        lib.sqo_seg_gemm.restype = ctypes.c_int
        lib.sqo_num_threads.restype = ctypes.c_int
        _LIB = lib
    return _LIB


def num_threads():
    return _lib().sqo_num_threads()


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _bounds(bounds):
    return np.ascontiguousarray(bounds, dtype=np.int32)


def e4m3_encode(x):
    """float32 array -> e4m3 bytes (saturating RN-even)."""
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint8)
    _lib().sqo_e4m3_encode(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


_E4M3_TABLE = None


def e4m3_decode(b):
    """e4m3 bytes -> float32 array."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        lib = _lib()
        _E4M3_TABLE = np.array([lib.sqo_e4m3_to_float(i) for i in range(256)], dtype=np.float32)
    return _E4M3_TABLE[np.asarray(b, dtype=np.uint8)]


def e4m3_roundtrip(x):
    """fake_e4m3fy on a float32 array (segquant/src/fake_quant/quantizer_fp8.cpp:25-39)."""
    x = _f32(x)
    out = np.empty_like(x)
    _lib().sqo_e4m3_roundtrip(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def quantize_act(x, bounds, sx, sx_neg=None, out_kind=Q_INT8, smooth=None):
    """x [M, K] -> quantised bytes [M, K] (and the negative-side tensor with DualScale).

    sx / sx_neg: shape (S,) for per-segment scales or (S, M) for per-token scales."""
    x = _f32(x)
    M, K = x.shape
    bounds = _bounds(bounds)
    S = len(bounds) - 1
    sx = _f32(sx).reshape(S, -1)
    per_token = sx.shape[1] != 1
    assert sx.shape[1] in (1, M)
    sxn = None if sx_neg is None else _f32(sx_neg).reshape(S, -1)
    xq = np.empty((M, K), dtype=np.uint8)
    xqn = None if sx_neg is None else np.empty((M, K), dtype=np.uint8)
    sm = _f32(smooth)
    _lib().sqo_quantize_act(_p(x), ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int(S), _p(bounds), _p(sx), _p(sxn),
                            ctypes.c_int64(sx.shape[1]), ctypes.c_int64(1 if per_token else 0), _p(sm),
                            ctypes.c_int(out_kind), _p(xq), _p(xqn))
    if out_kind == Q_INT8:
        xq = xq.view(np.int8)
        xqn = None if xqn is None else xqn.view(np.int8)
    return (xq, xqn) if sx_neg is not None else xq


def quantize_weight(w, scale, out_kind=Q_INT8, group_size=0):
    """w [N, K] -> int8 [N, K] / e4m3 bytes [N, K] / packed int4 bytes [N*K/2].

    scale: python float (scalar overload), array (N,) (per row) or (N, K/group_size) (per group)."""
    w = _f32(w)
    N, K = w.shape
    if np.isscalar(scale) or np.ndim(scale) == 0:
        mode, sc, sarr = 0, float(scale), None
    else:
        sarr = _f32(scale)
        mode = 2 if (group_size and sarr.ndim == 2) else 1
        sc = 0.0
    nbytes = (N * K + 1) // 2 if out_kind == Q_INT4 else N * K
    out = np.empty(nbytes, dtype=np.uint8)
    _lib().sqo_quantize_weight(_p(w), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(mode), ctypes.c_float(sc),
                               _p(sarr), ctypes.c_int(group_size), ctypes.c_int(out_kind), _p(out))
    if out_kind == Q_INT4:
        return out
    out = out.reshape(N, K)
    return out.view(np.int8) if out_kind == Q_INT8 else out


def unpack_int4(packed, numel):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(numel, dtype=np.int8)
    _lib().sqo_unpack_int4(_p(packed), _p(out), ctypes.c_int64(numel))
    return out


def seg_gemm(kind, xq, wq, bounds, sx, sw, xq_neg=None, sx_neg=None, group_size=0, bias=None, want_acc=False):
    """Segmented GEMM + de-quantise.  Returns y float32 [M, N] (and the per-unit accumulators).

    xq [M, K] bytes; wq [N, K] bytes or packed int4 [N*K/2]; sx (S,) or (S, M);
    sw: (N,) shared by all units, (S, N) per segment, (G, N) per K-group (group_size > 0),
        or (S,) one scalar per segment."""
    xq = np.ascontiguousarray(xq).view(np.uint8)
    M, K = xq.shape
    wq = np.ascontiguousarray(wq).view(np.uint8)
    N = wq.size * 2 // K if kind == GEMM_W4A8 else wq.shape[0]
    bounds = _bounds(bounds)
    S = len(bounds) - 1
    sx = _f32(sx).reshape(S, -1)
    per_token = sx.shape[1] != 1
    sxn = None if sx_neg is None else _f32(sx_neg).reshape(S, -1)
    xqn = None if xq_neg is None else np.ascontiguousarray(xq_neg).view(np.uint8)
    sw = _f32(sw)
    if group_size:
        assert sw.shape == (K // group_size, N), sw.shape
        sw_ss, sw_gs, sw_cs = 0, N, 1
    elif sw.ndim == 1 and sw.size == N:
        sw_ss, sw_gs, sw_cs = 0, 0, 1
    elif sw.ndim == 2 and sw.shape == (S, N):
        sw_ss, sw_gs, sw_cs = N, 0, 1
    elif sw.size == S:
        sw_ss, sw_gs, sw_cs = 1, 0, 0
    else:
        raise ValueError(f"unsupported sw shape {sw.shape}")
    units = 0
    for s in range(S):
        k = int(bounds[s])
        while k < bounds[s + 1]:
            ke = int(bounds[s + 1])
            if group_size:
                ke = min(ke, (k // group_size + 1) * group_size)
            units += 1
            k = ke
    sides = 2 if xqn is not None else 1
    y = np.empty((M, N), dtype=np.float32)
    acc = np.empty((units, sides, M, N), dtype=np.int32) if want_acc else None
    b = _f32(bias)
    got = _lib().sqo_seg_gemm(ctypes.c_int(kind), ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K), _p(xq), _p(xqn),
                              _p(wq), ctypes.c_int(S), _p(bounds), ctypes.c_int(group_size), _p(sx), _p(sxn),
                              ctypes.c_int64(sx.shape[1]), ctypes.c_int64(1 if per_token else 0), _p(sw),
                              ctypes.c_int64(sw_ss), ctypes.c_int64(sw_gs), ctypes.c_int64(sw_cs), _p(b), _p(y), _p(acc))
    assert got == units, (got, units)
    if want_acc:
        if kind == GEMM_F8:
            acc = acc.view(np.float32)
        return y, acc
    return y


# ---- scale definitions ---------------------------------------------------------------------------

_EPS = 1.0 / (1 << 24)


def calibrate_sym(x, qmax, axis=None):
    """scale = qmax / amax with the 2^-24 guard (IntQuantizer.calibrate, quantizer.py:204-217;
    FloatQuantizer.calibrate :441-452; qmax = 127, 7 or 448)."""
    x = np.asarray(x, dtype=np.float32)
    if axis is None:
        amax = float(np.abs(x).max()) if x.size else 0.0
        return qmax / amax if amax > _EPS else 1.0
    amax = np.abs(x).max(axis=axis)
    return (qmax / np.maximum(amax, _EPS)).astype(np.float32)


def calibrate_dual(x, qmax, qmin_abs):
    """DualScale per-tensor scales (quantizer.py:170-186 for int: pos = qmax/pos_amax,
    neg = qmin/(-neg_amax); :407-421 for e4m3: 448 on both sides)."""
    x = np.asarray(x, dtype=np.float32)
    neg = -x[x < 0]
    pos = x[x > 0]
    neg_amax = float(neg.max()) if neg.size else 0.0
    pos_amax = float(pos.max()) if pos.size else 0.0
    pos_scale = qmax / pos_amax if pos_amax > _EPS else 1.0
    neg_scale = qmin_abs / neg_amax if neg_amax > _EPS else 1.0
    return pos_scale, neg_scale


# ---- the reference's pybind functions, restated -------------------------------------------------------

_KIND_OF_PREFIX = {"Wint8Aint8": (GEMM_I8, Q_INT8), "Wfpe4m3Afpe4m3": (GEMM_F8, Q_E4M3), "Wint4Aint8": (GEMM_W4A8, Q_INT8)}


def real_quantized_gemm_scaled(prefix, inputs, weights, scale_x, scale_w, pos_neg=None):
    """`{prefix}_real_quantized_gemm_scaled(inputs, weights, scale_x, scale_w)` and, with
    pos_neg=(pos_scale_x, neg_scale_x), `{prefix}_real_quantized_gemm_dual_scaled`
    (real_gemm.cu:643-894).  inputs (S, ..., M, K) float32; weights (S, N, K) bytes or (S, N*K/2)
    packed int4; scales with S or S*M (x) / S or S*N (w) elements.  Returns float32 (S, ..., M, N)
    -- the caller rounds to the input dtype as the reference does (real_gemm.cu:684-687)."""
    kind, qk = _KIND_OF_PREFIX[prefix]
    inputs = np.asarray(inputs, dtype=np.float32)
    S = inputs.shape[0]
    K = inputs.shape[-1]
    M = int(np.prod(inputs.shape[1:-1]))
    x = inputs.reshape(S, M, K)
    weights = np.asarray(weights)
    N = weights.shape[1] * 2 // K if kind == GEMM_W4A8 else weights.shape[1]
    scale_w = _f32(scale_w).reshape(-1)
    outs = []
    for s in range(S):
        sw = scale_w[s:s + 1].repeat(N) if scale_w.size == S else scale_w[s * N:(s + 1) * N]  # real_gemm.cu:743
        if pos_neg is None:
            sx = _f32(scale_x).reshape(-1)
            sxs = sx[s:s + 1] if sx.size == S else sx[s * M:(s + 1) * M]  # real_gemm.cu:703
            xq = quantize_act(x[s], [0, K], sxs, out_kind=qk)
            outs.append(seg_gemm(kind, xq, weights[s], [0, K], sxs, sw))
        else:
            sp, sn = (_f32(t).reshape(-1) for t in pos_neg)
            sps = sp[s:s + 1] if sp.size == S else sp[s * M:(s + 1) * M]
            sns = sn[s:s + 1] if sn.size == S else sn[s * M:(s + 1) * M]
            xq, xqn = quantize_act(x[s], [0, K], sps, sx_neg=sns, out_kind=qk)
            outs.append(seg_gemm(kind, xq, weights[s], [0, K], sps, sw, xq_neg=xqn, sx_neg=sns))
    return np.stack(outs).reshape(*inputs.shape[:-1], N)
