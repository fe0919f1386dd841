"""GPU: sq_seg_linear_static -- the fused layer forward whose scratch is a fixed array inside the
library, for callers that are not allowed to allocate device memory (a plugin in a serving
process with a frozen memory budget, a loop barred from the allocator).

Called through the C ABI and compared with sq_seg_linear (caller-provided scratch) on the same
inputs, twice in a row with different shapes so that bytes left behind by the first call cannot
help the second.  Both entry points run the same kernels, so the outputs must be identical; the
comparison still uses the 1e-5 relative bound of the other GPU tests.  The result is also held against
the CPU oracle (bf16 output within one rounding step), and the property in the entry point's name is
checked directly: once the first call on the device has been made, the free device memory the driver
reports does not move across further calls.  Collected last so a run that stops at the first failure
has already run everything else; passes alone in a fresh process too.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import oracle as O
from segquant_b200 import _lib as L

DEV = "cuda:0"


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _blocks(x, wq, sx, sxn, sw, bias, y, bounds, kind, a_kind):
    M, K = x.shape
    N = wq.shape[0]
    q = L.ActQuantArgs()
    q.x_dev, q.x_dtype, q.out_kind = x.data_ptr(), L.SQ_BF16, a_kind
    q.batch, q.M, q.K = 1, M, K
    q.x_batch_stride, q.x_row_stride = 0, K
    q.num_segs = len(bounds) - 1
    L.set_bounds(q.seg_bounds, bounds)
    q.sx_dev = sx.data_ptr()
    q.sx_neg_dev = sxn.data_ptr() if sxn is not None else None
    q.sx_batch_stride, q.sx_seg_stride, q.sx_row_stride = 0, 1, 0
    q.xq_batch_stride, q.xq_row_stride = M * K, K
    g = L.GemmArgs()
    g.kind, g.out_dtype = kind, L.SQ_BF16
    g.batch, g.M, g.N, g.K = 1, M, N, K
    g.xq_row_stride = K
    g.wq_dev, g.wq_row_stride = wq.data_ptr(), K
    g.num_segs = len(bounds) - 1
    L.set_bounds(g.seg_bounds, bounds)
    g.sx_dev = sx.data_ptr()
    g.sx_neg_dev = sxn.data_ptr() if sxn is not None else None
    g.sx_seg_stride = 1
    g.sw_dev, g.sw_col_stride = sw.data_ptr(), 1
    g.bias_dev, g.bias_dtype = bias.data_ptr(), L.SQ_F32
    g.y_dev, g.y_row_stride = y.data_ptr(), N
    return q, g


def _case(seed, M, K, N, bounds, dual, kind, a_kind):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=gen)
    if dual:
        x = torch.nn.functional.gelu(x)
    x = x.to(torch.bfloat16).to(DEV)
    if kind == L.SQ_GEMM_W8A8_I8:
        wq = torch.randint(-128, 128, (N, K), generator=gen, dtype=torch.int8).to(DEV)
    else:
        wq = (torch.randn(N, K, generator=gen) * 40).to(torch.float8_e4m3fn).view(torch.uint8).to(DEV)
    S = len(bounds) - 1
    sx = (torch.rand(S, generator=gen) * 20 + 20).to(DEV)
    sxn = (torch.rand(S, generator=gen) * 200 + 400).to(DEV) if dual else None
    sw = (torch.rand(N, generator=gen) * 100 + 50).to(DEV)
    bias = torch.randn(N, generator=gen).to(DEV)
    return x, wq, sx, sxn, sw, bias


def test_static_scratch_forward_matches_caller_scratch_forward(native_lib):
    lib = native_lib
    cases = [
        (21, 700, 1536, 520, [0, 384, 768, 1152, 1536], False, L.SQ_GEMM_W8A8_I8, L.SQ_Q_INT8),
        (22, 300, 1024, 264, [0, 1024], True, L.SQ_GEMM_W8A8_F8, L.SQ_Q_E4M3),     # smaller, DualScale: reuses the array
    ]
    for seed, M, K, N, bounds, dual, kind, a_kind in cases:
        x, wq, sx, sxn, sw, bias = _case(seed, M, K, N, bounds, dual, kind, a_kind)
        y_ref = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        y_new = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        xq = torch.empty((M, K), dtype=torch.uint8, device=DEV)
        xqn = torch.empty((M, K), dtype=torch.uint8, device=DEV) if dual else None
        q, g = _blocks(x, wq, sx, sxn, sw, bias, y_ref, bounds, kind, a_kind)
        q.xq_dev = xq.data_ptr()
        q.xq_neg_dev = xqn.data_ptr() if dual else None
        L.check(lib.sq_seg_linear(ctypes.byref(q), ctypes.byref(g), _stream()), "sq_seg_linear")
        q2, g2 = _blocks(x, wq, sx, sxn, sw, bias, y_new, bounds, kind, a_kind)   # no scratch pointers at all
        L.check(lib.sq_seg_linear_static(ctypes.byref(q2), ctypes.byref(g2), _stream()), "sq_seg_linear_static")
        torch.cuda.synchronize()
        a, b = y_new.float().cpu().numpy(), y_ref.float().cpu().numpy()
        assert not np.isnan(a).any()
        assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max()
        # against the CPU oracle: its own quantise and exact integer / fp32 GEMM on the same inputs
        okind, oq = (O.GEMM_I8, O.Q_INT8) if kind == L.SQ_GEMM_W8A8_I8 else (O.GEMM_F8, O.Q_E4M3)
        sxn_np = sxn.cpu().numpy() if dual else None
        xq_o = O.quantize_act(x.float().cpu().numpy(), bounds, sx.cpu().numpy(), sx_neg=sxn_np, out_kind=oq)
        want = O.seg_gemm(okind, xq_o[0] if dual else xq_o, wq.cpu().numpy(), bounds, sx.cpu().numpy(), sw.cpu().numpy(),
                          xq_neg=xq_o[1] if dual else None, sx_neg=sxn_np, bias=bias.cpu().numpy())
        want16 = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
        assert np.abs(a - want16).max() <= 2.0 ** -8 * np.abs(want16).max()
        # no device allocation: free memory as the driver reports it is the same before and after further calls
        # (tensors were all created above; the first call on this device, which looks up the array's address, is behind us)
        free0, _ = torch.cuda.mem_get_info()
        for _ in range(3):
            L.check(lib.sq_seg_linear_static(ctypes.byref(q2), ctypes.byref(g2), _stream()), "sq_seg_linear_static")
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0, f"device memory moved by {free0 - free1} bytes across sq_seg_linear_static calls"
    assert lib.sq_device_status() == 0


def test_static_scratch_rejects_oversize_without_launching(native_lib):
    lib = native_lib
    M, K = 8192, 8192 + 32          # 64 MiB + 256 KiB of activations: one byte each is already too much
    x = torch.zeros(1, device=DEV)
    q, g = L.ActQuantArgs(), L.GemmArgs()
    for blk in (q, g):
        blk.batch, blk.M, blk.K = 1, M, K
    q.x_dev = q.sx_dev = x.data_ptr()
    assert lib.sq_seg_linear_static(ctypes.byref(q), ctypes.byref(g), _stream()) == L.SQ_ERR_TOO_LARGE
    msg = lib.sq_last_error().decode()
    assert "exceed the built-in" in msg and str(L.SQ_STATIC_SCRATCH_BYTES) in msg
    g.M = M - 1
    assert lib.sq_seg_linear_static(ctypes.byref(q), ctypes.byref(g), _stream()) == L.SQ_ERR_INVALID_ARG
    assert lib.sq_seg_linear_static(None, None, None) == L.SQ_ERR_INVALID_ARG
    torch.cuda.synchronize()
