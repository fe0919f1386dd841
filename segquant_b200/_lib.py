"""ctypes binding of libsegquant_b200.so (the C ABI declared in include/segquant_b200.h).

There is no fallback: if the shared library is missing or a call fails this module raises.
The library is built in-tree by `python -m segquant_b200.build`.
"""
import ctypes
import os

SQ_MAX_SEGS = 64
SQ_MAX_PEERS = 8
SQ_STATIC_SCRATCH_BYTES = 64 * 1024 * 1024

SQ_OK = 0
SQ_ERR_INVALID_ARG = -1
SQ_ERR_ALIGNMENT = -2
SQ_ERR_UNSUPPORTED = -3
SQ_ERR_CUDA = -4
SQ_ERR_DEVICE_TIMEOUT = -5
SQ_ERR_TOO_LARGE = -6

SQ_F32, SQ_F16, SQ_BF16 = 0, 1, 2
SQ_Q_INT8, SQ_Q_E4M3, SQ_Q_INT4 = 0, 1, 2
SQ_ACT_NONE, SQ_ACT_GELU_TANH, SQ_ACT_SILU = 0, 1, 2
SQ_GEMM_W8A8_I8, SQ_GEMM_W8A8_F8, SQ_GEMM_W4A8 = 0, 1, 2

EXPORTED_SYMBOLS = (
    "sq_version", "sq_last_error", "sq_status_string", "sq_device_status",
    "sq_quantize_act", "sq_quantize_act_dynamic", "sq_norm_quantize_act", "sq_residual_norm_quantize_act", "sq_gated_residual", "sq_quantize_weight", "sq_unpack_int4",
    "sq_gemm", "sq_gemm_num_units", "sq_seg_linear", "sq_seg_linear_static",
    "sq_check_device", "sq_set_wait_limit_cycles", "sq_wait_probe", "sq_set_gemm_schedule", "sq_push_columns", "sq_peer_barrier",
)


class ActQuantArgs(ctypes.Structure):
    """struct sq_act_quant_args"""
    _fields_ = [
        ("x_dev", ctypes.c_void_p),
        ("x_dtype", ctypes.c_int32),
        ("out_kind", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("M", ctypes.c_int64), ("K", ctypes.c_int64),
        ("x_batch_stride", ctypes.c_int64), ("x_row_stride", ctypes.c_int64),
        ("num_segs", ctypes.c_int32),
        ("seg_bounds", ctypes.c_int32 * (SQ_MAX_SEGS + 1)),
        ("sx_dev", ctypes.c_void_p),
        ("sx_neg_dev", ctypes.c_void_p),
        ("sx_batch_stride", ctypes.c_int64), ("sx_seg_stride", ctypes.c_int64), ("sx_row_stride", ctypes.c_int64),
        ("smooth_dev", ctypes.c_void_p),
        ("xq_dev", ctypes.c_void_p),
        ("xq_neg_dev", ctypes.c_void_p),
        ("xq_batch_stride", ctypes.c_int64), ("xq_row_stride", ctypes.c_int64),
        ("pre_act", ctypes.c_int32), ("reserved0", ctypes.c_int32),
    ]


class NormResidual(ctypes.Structure):
    """struct sq_norm_residual"""
    _fields_ = [
        ("y_dev", ctypes.c_void_p), ("gate_dev", ctypes.c_void_p), ("x_out_dev", ctypes.c_void_p),
        ("y_batch_stride", ctypes.c_int64), ("y_row_stride", ctypes.c_int64),
        ("gate_batch_stride", ctypes.c_int64),
        ("x_out_batch_stride", ctypes.c_int64), ("x_out_row_stride", ctypes.c_int64),
    ]


class GatedResidualArgs(ctypes.Structure):
    """struct sq_gated_residual_args"""
    _fields_ = [
        ("x_dev", ctypes.c_void_p), ("gate_dev", ctypes.c_void_p), ("y_dev", ctypes.c_void_p), ("out_dev", ctypes.c_void_p),
        ("dtype", ctypes.c_int32), ("reserved0", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("M", ctypes.c_int64), ("K", ctypes.c_int64),
        ("x_batch_stride", ctypes.c_int64), ("x_row_stride", ctypes.c_int64),
        ("y_batch_stride", ctypes.c_int64), ("y_row_stride", ctypes.c_int64),
        ("out_batch_stride", ctypes.c_int64), ("out_row_stride", ctypes.c_int64),
        ("gate_batch_stride", ctypes.c_int64),
    ]


class GemmArgs(ctypes.Structure):
    """struct sq_gemm_args"""
    _fields_ = [
        ("kind", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
        ("xq_dev", ctypes.c_void_p),
        ("xq_neg_dev", ctypes.c_void_p),
        ("xq_batch_stride", ctypes.c_int64), ("xq_row_stride", ctypes.c_int64),
        ("wq_dev", ctypes.c_void_p),
        ("wq_batch_stride", ctypes.c_int64), ("wq_row_stride", ctypes.c_int64),
        ("w_seg_as_batch", ctypes.c_int32),
        ("num_segs", ctypes.c_int32),
        ("seg_bounds", ctypes.c_int32 * (SQ_MAX_SEGS + 1)),
        ("group_size", ctypes.c_int32),
        ("sw_is_bf16", ctypes.c_int32),
        ("sx_dev", ctypes.c_void_p),
        ("sx_neg_dev", ctypes.c_void_p),
        ("sx_batch_stride", ctypes.c_int64), ("sx_seg_stride", ctypes.c_int64), ("sx_row_stride", ctypes.c_int64),
        ("sw_dev", ctypes.c_void_p),
        ("sw_batch_stride", ctypes.c_int64), ("sw_seg_stride", ctypes.c_int64),
        ("sw_group_stride", ctypes.c_int64), ("sw_col_stride", ctypes.c_int64),
        ("bias_dev", ctypes.c_void_p),
        ("bias_dtype", ctypes.c_int32),
        ("reserved0", ctypes.c_int32),
        ("bias_batch_stride", ctypes.c_int64),
        ("y_dev", ctypes.c_void_p),
        ("y_batch_stride", ctypes.c_int64), ("y_row_stride", ctypes.c_int64),
        ("acc_dump_dev", ctypes.c_void_p),
        ("num_peer_outputs", ctypes.c_int32),
        ("reserved1", ctypes.c_int32),
        ("peer_y_dev", ctypes.c_void_p * SQ_MAX_PEERS),
        ("peer_row_stride", ctypes.c_int64),
        ("peer_col_offset", ctypes.c_int64),
    ]


class SegQuantError(RuntimeError):
    """A C-ABI call returned a negative status; mirrors the reference's std::runtime_error ->
    RuntimeError mapping (segquant/src/real_quant/real_gemm.cu:237-247, :300-304)."""

    def __init__(self, status, message):
        super().__init__(message)
        self.status = status


_LIB = None


def lib_path():
    """In-tree library, or the file named by SEGQUANT_B200_LIB (e.g. an instrumented build)."""
    return os.environ.get("SEGQUANT_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libsegquant_b200.so")


def load():
    """Load (once) and return the ctypes handle of the native library.  Raises if it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"segquant_b200: native library {path} not found; build it with `python -m segquant_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(path)
    lib.sq_version.restype = ctypes.c_int
    lib.sq_last_error.restype = ctypes.c_char_p
    lib.sq_status_string.restype = ctypes.c_char_p
    lib.sq_status_string.argtypes = [ctypes.c_int]
    lib.sq_device_status.restype = ctypes.c_int64
    lib.sq_check_device.restype = ctypes.c_int
    lib.sq_set_wait_limit_cycles.restype = ctypes.c_int
    lib.sq_set_wait_limit_cycles.argtypes = [ctypes.c_int64]
    lib.sq_wait_probe.restype = ctypes.c_int
    lib.sq_wait_probe.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.sq_set_gemm_schedule.restype = ctypes.c_int
    lib.sq_set_gemm_schedule.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.sq_peer_barrier.restype = ctypes.c_int
    lib.sq_peer_barrier.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint32, ctypes.c_void_p]
    lib.sq_push_columns.restype = ctypes.c_int
    lib.sq_push_columns.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                    ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_void_p]
    lib.sq_quantize_act.restype = ctypes.c_int
    lib.sq_quantize_act.argtypes = [ctypes.POINTER(ActQuantArgs), ctypes.c_void_p]
    lib.sq_quantize_act_dynamic.restype = ctypes.c_int
    lib.sq_residual_norm_quantize_act.restype = ctypes.c_int
    lib.sq_residual_norm_quantize_act.argtypes = [ctypes.POINTER(ActQuantArgs), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                                  ctypes.c_float, ctypes.POINTER(NormResidual), ctypes.c_void_p]
    lib.sq_gated_residual.restype = ctypes.c_int
    lib.sq_gated_residual.argtypes = [ctypes.POINTER(GatedResidualArgs), ctypes.c_void_p]
    lib.sq_norm_quantize_act.restype = ctypes.c_int
    lib.sq_norm_quantize_act.argtypes = [ctypes.POINTER(ActQuantArgs), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.c_float, ctypes.c_void_p]
    lib.sq_quantize_act_dynamic.argtypes = [ctypes.POINTER(ActQuantArgs), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.sq_quantize_weight.restype = ctypes.c_int
    lib.sq_quantize_weight.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                       ctypes.c_float, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                       ctypes.c_void_p]
    lib.sq_unpack_int4.restype = ctypes.c_int
    lib.sq_unpack_int4.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    lib.sq_gemm.restype = ctypes.c_int
    lib.sq_gemm.argtypes = [ctypes.POINTER(GemmArgs), ctypes.c_void_p]
    lib.sq_gemm_num_units.restype = ctypes.c_int
    lib.sq_gemm_num_units.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]
    lib.sq_seg_linear.restype = ctypes.c_int
    lib.sq_seg_linear.argtypes = [ctypes.POINTER(ActQuantArgs), ctypes.POINTER(GemmArgs), ctypes.c_void_p]
    lib.sq_seg_linear_static.restype = ctypes.c_int
    lib.sq_seg_linear_static.argtypes = [ctypes.POINTER(ActQuantArgs), ctypes.POINTER(GemmArgs), ctypes.c_void_p]
    _LIB = lib
    return lib


def check(status, what):
    """Turn a negative status into SegQuantError carrying the library's message."""
    if status < 0:
        lib = load()
        name = lib.sq_status_string(status).decode()
        msg = lib.sq_last_error().decode()
        raise SegQuantError(status, f"{what}: {name}: {msg}")
    return status


def set_bounds(field, bounds):
    if len(bounds) - 1 > SQ_MAX_SEGS:
        raise SegQuantError(SQ_ERR_INVALID_ARG, f"at most {SQ_MAX_SEGS} segments per call, got {len(bounds) - 1}")
    for i, v in enumerate(bounds):
        field[i] = int(v)
