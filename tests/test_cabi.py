"""CPU: the C-ABI shared library loads without a GPU, exports every symbol the header declares,
its argument structs have the layout the ctypes mirror assumes, and argument errors come back as
status codes (no compute is attempted here)."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

from segquant_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "segquant_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native_lib):
    names = declared_functions()
    assert "sq_gemm" in names and "sq_quantize_act" in names and len(names) >= 11
    for n in names:
        assert hasattr(native_lib, n), f"{n} declared in include/segquant_b200.h but not exported"
    assert set(names) == set(L.EXPORTED_SYMBOLS)


def test_version_and_status_strings(native_lib):
    assert native_lib.sq_version() == 100
    assert native_lib.sq_status_string(0) == b"SQ_OK"
    assert native_lib.sq_status_string(L.SQ_ERR_ALIGNMENT) == b"SQ_ERR_ALIGNMENT"


def test_struct_layout_matches_header(tmp_path):
    """Compile a tiny C program against the header and compare sizeof / offsetof with ctypes."""
    fields_a = [f[0] for f in L.ActQuantArgs._fields_]
    fields_g = [f[0] for f in L.GemmArgs._fields_]
    fields_r = [f[0] for f in L.GatedResidualArgs._fields_]
    fields_n = [f[0] for f in L.NormResidual._fields_]
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){",
             'printf("A %zu\\n", sizeof(sq_act_quant_args));', 'printf("G %zu\\n", sizeof(sq_gemm_args));']
    for f in fields_a:
        lines.append(f'printf("A.{f} %zu\\n", offsetof(sq_act_quant_args, {f}));')
    for f in fields_g:
        lines.append(f'printf("G.{f} %zu\\n", offsetof(sq_gemm_args, {f}));')
    lines.append('printf("R %zu\\n", sizeof(sq_gated_residual_args));')
    for f in fields_r:
        lines.append(f'printf("R.{f} %zu\\n", offsetof(sq_gated_residual_args, {f}));')
    lines.append('printf("N %zu\\n", sizeof(sq_norm_residual));')
    for f in fields_n:
        lines.append(f'printf("N.{f} %zu\\n", offsetof(sq_norm_residual, {f}));')
    lines.append("return 0;}")
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    got = dict(l.split() for l in out if l)
    assert int(got["A"]) == ctypes.sizeof(L.ActQuantArgs)
    assert int(got["G"]) == ctypes.sizeof(L.GemmArgs)
    assert int(got["R"]) == ctypes.sizeof(L.GatedResidualArgs)
    assert int(got["N"]) == ctypes.sizeof(L.NormResidual)
    for f in fields_n:
        assert int(got[f"N.{f}"]) == getattr(L.NormResidual, f).offset, f
    for f in fields_r:
        assert int(got[f"R.{f}"]) == getattr(L.GatedResidualArgs, f).offset, f
    for f in fields_a:
        assert int(got[f"A.{f}"]) == getattr(L.ActQuantArgs, f).offset, f
    for f in fields_g:
        assert int(got[f"G.{f}"]) == getattr(L.GemmArgs, f).offset, f


def test_argument_errors_are_status_codes(native_lib):
    assert native_lib.sq_gemm(None, None) == L.SQ_ERR_INVALID_ARG
    assert b"NULL" in native_lib.sq_last_error()
    assert native_lib.sq_quantize_act(None, None) == L.SQ_ERR_INVALID_ARG
    assert native_lib.sq_gated_residual(None, None) == L.SQ_ERR_INVALID_ARG
    r = L.GatedResidualArgs()
    r.batch, r.M, r.K, r.dtype = 1, 4, 20, L.SQ_BF16
    r.x_dev = r.gate_dev = r.y_dev = r.out_dev = 256
    assert native_lib.sq_gated_residual(ctypes.byref(r), None) == L.SQ_ERR_ALIGNMENT      # K not a multiple of 8
    r.K, r.dtype = 16, L.SQ_F32
    assert native_lib.sq_gated_residual(ctypes.byref(r), None) == L.SQ_ERR_UNSUPPORTED    # 16-bit tensors only
    a = L.GemmArgs()
    a.kind = 99
    assert native_lib.sq_gemm(ctypes.byref(a), None) == L.SQ_ERR_INVALID_ARG
    a.kind, a.out_dtype, a.batch, a.M, a.N, a.K = L.SQ_GEMM_W8A8_I8, L.SQ_F32, 1, 16, 16, 40
    buf = ctypes.create_string_buffer(4096)
    addr = (ctypes.addressof(buf) + 255) & ~255
    for f in ("xq_dev", "wq_dev", "sx_dev", "sw_dev", "y_dev"):
        setattr(a, f, addr)
    a.num_segs = 1
    L.set_bounds(a.seg_bounds, [0, 40])
    a.xq_row_stride = a.wq_row_stride = 48
    # K = 40 is not a multiple of 32: the reference throws std::runtime_error for K alignment
    assert native_lib.sq_gemm(ctypes.byref(a), None) == L.SQ_ERR_ALIGNMENT
    assert b"divisible" in native_lib.sq_last_error()
    with pytest.raises(L.SegQuantError) as e:
        L.check(L.SQ_ERR_ALIGNMENT, "sq_gemm")
    assert e.value.status == L.SQ_ERR_ALIGNMENT
    # fused all-gather outputs: range, batch and alignment are checked before anything is launched
    a.K = 64
    L.set_bounds(a.seg_bounds, [0, 64])
    a.xq_row_stride = a.wq_row_stride = 64
    a.y_row_stride = 16
    a.num_peer_outputs = L.SQ_MAX_PEERS + 1
    assert native_lib.sq_gemm(ctypes.byref(a), None) == L.SQ_ERR_INVALID_ARG
    a.num_peer_outputs, a.peer_row_stride, a.peer_col_offset = 1, 32, 3          # column offset not 16-byte aligned
    a.peer_y_dev[0] = addr
    assert native_lib.sq_gemm(ctypes.byref(a), None) == L.SQ_ERR_ALIGNMENT
    a.peer_col_offset, a.batch = 16, 2
    assert native_lib.sq_gemm(ctypes.byref(a), None) == L.SQ_ERR_UNSUPPORTED
    assert b"batch" in native_lib.sq_last_error()
    q = L.ActQuantArgs()
    q.x_dev = q.xq_dev = q.sx_dev = addr
    q.x_dtype, q.out_kind, q.batch, q.M, q.K, q.num_segs = L.SQ_F32, L.SQ_Q_INT4, 1, 4, 64, 1
    L.set_bounds(q.seg_bounds, [0, 64])
    assert native_lib.sq_quantize_act(ctypes.byref(q), None) == L.SQ_ERR_UNSUPPORTED   # int4 activations
    q.out_kind, q.K = L.SQ_Q_INT8, 24
    L.set_bounds(q.seg_bounds, [0, 24])
    assert native_lib.sq_quantize_act(ctypes.byref(q), None) == L.SQ_ERR_ALIGNMENT


def test_num_units(native_lib):
    def units(bounds, group):
        arr = (ctypes.c_int32 * len(bounds))(*bounds)
        return native_lib.sq_gemm_num_units(len(bounds) - 1, arr, group)
    assert units([0, 1536], 0) == 1
    assert units([0, 384, 768, 1152, 1536], 0) == 4
    assert units([0, 1024, 3072], 128) == 24
    assert units([0, 192, 384], 128) == 4       # segments of 192 straddle groups of 128
    assert units([0, 0], 0) == L.SQ_ERR_INVALID_ARG


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "_LIB", None)
    monkeypatch.setattr(L, "lib_path", lambda: str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        L.load()
