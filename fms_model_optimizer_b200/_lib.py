"""ctypes binding of ``libqlin_b200.so`` (declared in ``include/qlin_b200.h``).

The structures below mirror the header field for field.  There is no fallback: if the library is
missing or a call fails, a ``RuntimeError`` with the library's own message is raised.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libqlin_b200.so"

# qlin_status
OK = 0
ERR_BAD_SHAPE, ERR_BAD_ALIGN, ERR_BAD_DTYPE, ERR_UNSUPPORTED = -1, -2, -3, -4
ERR_LAUNCH, ERR_TIMEOUT, ERR_NULL, ERR_DEVICE, ERR_TOO_LARGE = -5, -6, -7, -8, -9

# qlin_dtype
DT_NONE, DT_I8, DT_U8, DT_I32, DT_F32, DT_F16, DT_BF16, DT_F8E4M3, DT_F8E5M2 = range(9)

# qlin_epilogue
EPI_RAW, EPI_SCALE_PROD, EPI_SCALE_SEQ = 0, 1, 2

# qlin_quant_mode
(Q_I8_DYN, Q_I8_STATIC, Q_I8_STATIC_CLAMP_FIRST, Q_F8_DYN, Q_I8_GIVEN_SCALE, Q_F8_FAKE_SCALED, Q_I8_STATIC_ROUND_FIRST,
 Q_I8_AFFINE_RCP, Q_F8_TENSOR) = range(9)

# qlin_pact_variant
PACT_TWO_SIDED, PACT_ONE_SIDED, PACT_SYMMETRIC = 0, 1, 2

# qlin_wq_mode
W_SAWB, W_MAX, W_GIVEN = 0, 1, 2
PT_INT_SYM, PT_F8_SCALED, PT_F8_SAT = 0, 1, 2
BLOCK_PLAIN, BLOCK_NORM, BLOCK_SILU_MUL = 0, 1, 2
BLOCK_DYN, BLOCK_GIVEN_SCALE, BLOCK_SCALE_ONLY = 0, 1, 2

EXPORTED_SYMBOLS = (
    "qlin_version",
    "qlin_last_error_string",
    "qlin_device_supported",
    "qlin_gemm",
    "qlin_gemm_batched",
    "qlin_act_quant",
    "qlin_pact2_fwd",
    "qlin_pact2_bwd",
    "qlin_pact2_bwd_workspace_bytes",
    "qlin_pact2_bwd_noalloc",
    "qlin_pact2_bwd_noalloc_max_numel",
    "qlin_weight_fq_perch",
    "qlin_tensor_fq",
    "qlin_tensor_fq_workspace_bytes",
    "qlin_block_quant",
    "qlin_rope",
    "qlin_ipc_export",
    "qlin_ipc_open",
    "qlin_ipc_close",
    "qlin_peer_copy2d",
    "qlin_peer_barrier",
    "qlin_col_absmax",
    "qlin_shard_reduce",
)


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("c", C.c_void_p),
        ("d", C.c_void_p),
        ("row_scale", C.c_void_p),
        ("col_scale", C.c_void_p),
        ("bias", C.c_void_p),
        ("status", C.c_void_p),
        ("lda", C.c_int64),
        ("ldb", C.c_int64),
        ("ldc", C.c_int64),
        ("ldd", C.c_int64),
        ("M", C.c_int32),
        ("N", C.c_int32),
        ("K", C.c_int32),
        ("kind", C.c_int32),
        ("chunk_k", C.c_int32),
        ("trun_bits", C.c_int32),
        ("max_acc_bits", C.c_int32),
        ("trunc_then_acc", C.c_int32),
        ("clamp_dl16", C.c_int32),
        ("epilogue", C.c_int32),
        ("row_scale_stride", C.c_int32),
        ("col_scale_stride", C.c_int32),
        ("prod_round", C.c_int32),
        ("scale_round", C.c_int32),
        ("mid_round", C.c_int32),
        ("acc_round", C.c_int32),
        ("out_dtype", C.c_int32),
        ("scatter_d", C.c_void_p * 8),
        ("scatter_rows", C.c_int32),
        ("scatter_row0", C.c_int32),
        ("max_ctas", C.c_int32),
    ]


class QuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("smooth", C.c_void_p),
        ("smooth_rcp", C.c_void_p),
        ("scale_in", C.c_void_p),
        ("codes", C.c_void_p),
        ("scale_out", C.c_void_p),
        ("dq_out", C.c_void_p),
        ("status", C.c_void_p),
        ("ldx", C.c_int64),
        ("ldq", C.c_int64),
        ("lddq", C.c_int64),
        ("rows", C.c_int32),
        ("cols", C.c_int32),
        ("x_dtype", C.c_int32),
        ("mode", C.c_int32),
        ("native_chain", C.c_int32),
        ("smooth_mul", C.c_int32),
        ("clamp_codes", C.c_int32),
        ("qmax_levels", C.c_int32),
        ("dl8_flush", C.c_int32),
        ("scale_in_stride", C.c_int32),
        ("scale0", C.c_float),
        ("zp0", C.c_float),
        ("lo", C.c_float),
        ("hi", C.c_float),
        ("shift", C.c_float),
        ("add2", C.c_float),
        ("dyn_eps", C.c_float),
        ("f8_format", C.c_int32),
    ]


class Pact2Args(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("grad_out", C.c_void_p),
        ("out", C.c_void_p),
        ("clip_val", C.c_void_p),
        ("clip_valn", C.c_void_p),
        ("grad_clip", C.c_void_p),
        ("workspace", C.c_void_p),
        ("numel", C.c_int64),
        ("dtype", C.c_int32),
        ("num_bits", C.c_int32),
        ("align_zero", C.c_int32),
        ("variant", C.c_int32),
    ]


class WfqArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p),
        ("smooth", C.c_void_p),
        ("dq_out", C.c_void_p),
        ("codes", C.c_void_p),
        ("clip_io", C.c_void_p),
        ("ldw", C.c_int64),
        ("ldo", C.c_int64),
        ("ldq", C.c_int64),
        ("rows", C.c_int32),
        ("cols", C.c_int32),
        ("dtype", C.c_int32),
        ("num_bits", C.c_int32),
        ("mode", C.c_int32),
        ("native_mul", C.c_int32),
        ("clip_dtype", C.c_int32),
        ("c0", C.c_float),
        ("c1", C.c_float),
    ]


class TensorFqArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("out", C.c_void_p),
        ("clip_io", C.c_void_p),
        ("workspace", C.c_void_p),
        ("numel", C.c_int64),
        ("dtype", C.c_int32),
        ("num_bits", C.c_int32),
        ("mode", C.c_int32),
        ("kind", C.c_int32),
        ("align_zero", C.c_int32),
        ("dequantize", C.c_int32),
        ("c0", C.c_float),
        ("c1", C.c_float),
    ]


class BlockQuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("r", C.c_void_p),
        ("r_parts", C.c_int32),
        ("r_part_stride", C.c_int64),
        ("x_out", C.c_void_p),
        ("h_out", C.c_void_p),
        ("norm_w", C.c_void_p),
        ("smooth_rcp", C.c_void_p * 3),
        ("codes", C.c_void_p * 3),
        ("scale_out", C.c_void_p * 3),
        ("scale_in", C.c_void_p),
        ("scale_in_stride", C.c_int64),
        ("scale_in_parts", C.c_int32),
        ("dst_base", C.c_void_p * 8),
        ("codes_off", C.c_int64 * 3),
        ("scale_off", C.c_int64 * 3),
        ("ndst", C.c_int32),
        ("dst_row0", C.c_int32),
        ("ldx", C.c_int64),
        ("ldr", C.c_int64),
        ("ldxo", C.c_int64),
        ("ldh", C.c_int64),
        ("ldq", C.c_int64 * 3),
        ("rows", C.c_int32),
        ("cols", C.c_int32),
        ("nout", C.c_int32),
        ("prologue", C.c_int32),
        ("mode", C.c_int32),
        ("qmax_levels", C.c_int32),
        ("norm_eps", C.c_float),
        ("dyn_eps", C.c_float),
        ("max_ctas", C.c_int32),
        ("r_multimem", C.c_int32),
        ("dst_multimem", C.c_int32),
    ]


class RopeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("cos", C.c_void_p),
        ("sin", C.c_void_p),
        ("ld_token", C.c_int64),
        ("tokens", C.c_int32),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("seq_len", C.c_int32),
    ]


class ColAbsmaxArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("amax_io", C.c_void_p),
        ("ldx", C.c_int64),
        ("rows", C.c_int32),
        ("cols", C.c_int32),
        ("dtype", C.c_int32),
        ("accumulate", C.c_int32),
    ]


class ShardReduceArgs(C.Structure):
    _fields_ = [
        ("src_multicast", C.c_void_p),
        ("add", C.c_void_p),
        ("out", C.c_void_p),
        ("ld_src", C.c_int64),
        ("ld_add", C.c_int64),
        ("ld_out", C.c_int64),
        ("rows", C.c_int32),
        ("cols", C.c_int32),
        ("max_ctas", C.c_int32),
    ]


class PeerBarrierArgs(C.Structure):
    _fields_ = [
        ("local_flags", C.c_void_p),
        ("peer_flags", C.c_void_p * 8),
        ("epoch", C.c_void_p),
        ("status", C.c_void_p),
        ("rank", C.c_int32),
        ("world", C.c_int32),
        ("timeout_ns", C.c_int64),
    ]


_lib = None


def load() -> C.CDLL:
    """Loads the library once and declares the prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m fms_model_optimizer_b200.build_ext` "
            "(there is no fallback implementation)"
        )
    lib = C.CDLL(str(LIB_PATH))
    lib.qlin_version.restype = C.c_int
    lib.qlin_last_error_string.restype = C.c_char_p
    lib.qlin_device_supported.argtypes = [C.c_int]
    lib.qlin_device_supported.restype = C.c_int
    for name, struct in (
        ("qlin_gemm", GemmArgs),
        ("qlin_act_quant", QuantArgs),
        ("qlin_pact2_fwd", Pact2Args),
        ("qlin_pact2_bwd", Pact2Args),
        ("qlin_pact2_bwd_noalloc", Pact2Args),
        ("qlin_weight_fq_perch", WfqArgs),
        ("qlin_tensor_fq", TensorFqArgs),
        ("qlin_block_quant", BlockQuantArgs),
        ("qlin_rope", RopeArgs),
        ("qlin_peer_barrier", PeerBarrierArgs),
        ("qlin_col_absmax", ColAbsmaxArgs),
        ("qlin_shard_reduce", ShardReduceArgs),
    ):
        fn = getattr(lib, name)
        fn.argtypes = [C.POINTER(struct), C.c_void_p]
        fn.restype = C.c_int
    lib.qlin_gemm_batched.argtypes = [C.POINTER(GemmArgs), C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
    lib.qlin_gemm_batched.restype = C.c_int
    lib.qlin_pact2_bwd_workspace_bytes.argtypes = [C.c_int64]
    lib.qlin_pact2_bwd_workspace_bytes.restype = C.c_size_t
    lib.qlin_pact2_bwd_noalloc_max_numel.restype = C.c_int64
    lib.qlin_ipc_export.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    lib.qlin_ipc_export.restype = C.c_int
    lib.qlin_ipc_open.argtypes = [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
    lib.qlin_ipc_open.restype = C.c_int
    lib.qlin_peer_copy2d.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
    lib.qlin_peer_copy2d.restype = C.c_int
    lib.qlin_ipc_close.argtypes = [C.c_void_p]
    lib.qlin_ipc_close.restype = C.c_int
    lib.qlin_tensor_fq_workspace_bytes.argtypes = [C.c_int64]
    lib.qlin_tensor_fq_workspace_bytes.restype = C.c_int64
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    """Turns a negative qlin_status into a RuntimeError carrying the library's message."""
    if rc != OK:
        msg = load().qlin_last_error_string()
        raise RuntimeError(f"{what} failed with status {rc}: {msg.decode() if msg else ''}")
