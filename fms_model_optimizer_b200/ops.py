"""Tensor-level entry points over the C ABI of ``libqlin_b200.so``.

Every function here takes CUDA tensors, allocates its outputs with PyTorch's caching allocator,
passes raw device pointers plus the current CUDA stream to the library and returns tensors.  There
is no CPU path and no fallback kernel: a CPU tensor or a missing library is an error.

The functions are also registered as torch custom ops in the ``qlin_b200`` namespace (see the end
of the file) so that modules call ``torch.ops.qlin_b200.*`` the way the reference's modules call
``torch.ops.fms_mo.*`` (fms_mo/custom_ext_kernels/utils.py:642-802).
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence, Tuple

import torch

from . import _lib as L

_DT = {
    torch.int8: L.DT_I8,
    torch.uint8: L.DT_U8,
    torch.int32: L.DT_I32,
    torch.float32: L.DT_F32,
    torch.float16: L.DT_F16,
    torch.bfloat16: L.DT_BF16,
    torch.float8_e4m3fn: L.DT_F8E4M3,
    torch.float8_e5m2: L.DT_F8E5M2,
}
_ROUND = {None: L.DT_NONE, torch.float32: L.DT_F32, torch.float16: L.DT_F16, torch.bfloat16: L.DT_BF16}

_status_words: dict[int, torch.Tensor] = {}


# Measurement hooks used by bench.py: LAUNCHES counts kernel launches made through this module;
# when PROFILE is a list, every launch is bracketed by CUDA events on the launching stream and
# (name, start, end, work) is appended (work = operations for the GEMM, bytes for the others).
LAUNCHES = 0
PROFILE = None
# Upper bound on the CTAs of a GEMM launch (0 = one per SM).  A caller that overlaps GEMMs with a collective on another
# stream lowers it so that the collective's CTAs find free SMs.
GEMM_MAX_CTAS = 0


# QLIN_NVTX=1: every launch of this library sits inside an NVTX range named after its entry point, so that a timeline
# tool shows the library's calls among PyTorch's (off by default: a range costs a little host time per launch).
NVTX = os.environ.get("QLIN_NVTX", "0") == "1"


def _timed(name: str, work: float, dev: torch.device, call):
    global LAUNCHES
    LAUNCHES += 1
    if NVTX:
        torch.cuda.nvtx.range_push(f"qlin_{name}")
        try:
            return _timed_inner(name, work, dev, call)
        finally:
            torch.cuda.nvtx.range_pop()
    return _timed_inner(name, work, dev, call)


def _timed_inner(name: str, work: float, dev: torch.device, call):
    if PROFILE is None:
        return call()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st = torch.cuda.current_stream(dev)
    e0.record(st)
    rc = call()
    e1.record(st)
    PROFILE.append((name, e0, e1, work))
    return rc


def _require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("qlin_b200 ops run on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    if dev is None:
        raise RuntimeError("no tensor given")
    return dev


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(dev: torch.device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def status_word(dev: torch.device) -> torch.Tensor:
    """Per-device int32 status word handed to the GEMM; stays 0 unless a kernel gave up a wait."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status_words[idx]


def check_status(dev: Optional[torch.device] = None) -> None:
    """Synchronises and raises if any GEMM on ``dev`` reported a timed-out wait."""
    dev = dev if dev is not None else torch.device("cuda", torch.cuda.current_device())
    word = status_word(dev)
    val = int(word.item())
    if val != 0:
        word.zero_()
        raise RuntimeError(f"qlin_gemm reported device status {val} (a bounded wait ran out)")


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    t = t.reshape(-1)
    if t.dtype != torch.float32:
        t = t.float()
    return t.contiguous()


def _pad_k(t: torch.Tensor) -> torch.Tensor:
    """Returns a K-contiguous 2-D view/copy whose row stride and base are 16-byte aligned."""
    es = t.element_size()
    if t.stride(1) == 1 and (t.stride(0) * es) % 16 == 0 and t.data_ptr() % 16 == 0 and t.stride(0) >= t.shape[1]:
        return t
    rows, k = t.shape
    kp = (k * es + 15) // 16 * 16 // es
    buf = torch.zeros((rows, kp), dtype=t.dtype, device=t.device)
    buf[:, :k] = t
    return buf[:, :k]


# --------------------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------------------
def gemm(
    a: torch.Tensor,
    b_nk: torch.Tensor,
    *,
    c: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    chunk_k: int = 0,
    trun_bits: int = 0,
    max_acc_bits: int = 32,
    trunc_then_acc: bool = True,
    clamp_dl16: bool = False,
    epilogue: int = L.EPI_RAW,
    row_scale: Optional[torch.Tensor] = None,
    col_scale: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    prod_round: Optional[torch.dtype] = None,
    scale_round: Optional[torch.dtype] = None,
    mid_round: Optional[torch.dtype] = None,
    acc_round: Optional[torch.dtype] = None,
    scatter: Optional[Tuple[Sequence[int], int, int]] = None,
    max_ctas: Optional[int] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """``D[M,N] = epilogue(C + sum_chunks f(A_c @ B_c^T))`` with A ``[M,K]`` and B ``[N,K]`` (both
    K-contiguous, int8 or float8_e4m3fn).  See ``qlin_gemm`` in include/qlin_b200.h for the
    chunk and epilogue semantics (tl_matmul_chunk_truncate, fms_mo/custom_ext_kernels/triton_kernels.py:468)."""
    dev = _require_cuda(a, b_nk, c, out, row_scale, col_scale, bias)
    if a.dim() != 2 or b_nk.dim() != 2 or a.shape[1] != b_nk.shape[1]:
        raise RuntimeError(f"incompatible shapes {tuple(a.shape)} x {tuple(b_nk.shape)}^T")
    if a.dtype != b_nk.dtype or a.dtype not in (torch.int8, torch.float8_e4m3fn, torch.float8_e5m2):
        raise RuntimeError(f"operands must both be int8, float8_e4m3fn or float8_e5m2, got {a.dtype} and {b_nk.dtype}")
    f8 = a.dtype != torch.int8
    M, K = a.shape
    N = b_nk.shape[0]
    raw_dtype = torch.float32 if f8 else torch.int32
    if epilogue == L.EPI_RAW:
        out_dtype = raw_dtype
    elif out_dtype is None:
        out_dtype = torch.float32
    ldd = N
    if scatter is not None:
        # (base addresses, rows per destination, first row in each destination[, leading dimension]): the epilogue
        # stores row block m // rows to its own buffer, possibly another GPU's; nothing is returned
        if out is not None or c is not None:
            raise RuntimeError("scatter excludes out and c")
        ldd = int(scatter[3]) if len(scatter) > 3 else N
    elif out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    elif out.dtype != out_dtype or out.shape != (M, N) or out.stride(1) != 1:
        raise RuntimeError("out has the wrong dtype, shape or layout")
    else:
        ldd = out.stride(0)
    if M == 0 or N == 0:
        return out
    if K == 0:
        raise RuntimeError("K must be positive")
    a = _pad_k(a)
    b_nk = _pad_k(b_nk)
    if c is not None:
        if c.dtype != raw_dtype or c.shape != (M, N):
            raise RuntimeError("c must be an [M,N] tensor of the accumulator dtype")
        if c.stride(1) != 1:
            c = c.contiguous()
    rs, cs, bs = _f32(row_scale), _f32(col_scale), _f32(bias)
    if rs is not None and rs.numel() not in (1, M):
        raise RuntimeError("row_scale must have 1 or M elements")
    if cs is not None and cs.numel() not in (1, N):
        raise RuntimeError("col_scale must have 1 or N elements")
    if bs is not None and bs.numel() != N:
        raise RuntimeError("bias must have N elements")
    args = L.GemmArgs(
        a=_ptr(a), b=_ptr(b_nk), c=_ptr(c), d=_ptr(out),
        row_scale=_ptr(rs), col_scale=_ptr(cs), bias=_ptr(bs), status=_ptr(status_word(dev)),
        lda=a.stride(0), ldb=b_nk.stride(0), ldc=(c.stride(0) if c is not None else 0), ldd=ldd,
        M=M, N=N, K=K, kind=_DT[a.dtype],
        chunk_k=int(chunk_k), trun_bits=int(trun_bits), max_acc_bits=int(max_acc_bits),
        trunc_then_acc=int(bool(trunc_then_acc)), clamp_dl16=int(bool(clamp_dl16)), epilogue=int(epilogue),
        row_scale_stride=(0 if rs is None or rs.numel() == 1 else 1),
        col_scale_stride=(0 if cs is None or cs.numel() == 1 else 1),
        prod_round=_ROUND[prod_round], scale_round=_ROUND[scale_round], mid_round=_ROUND[mid_round], acc_round=_ROUND[acc_round],
        out_dtype=_DT[out_dtype], max_ctas=int(GEMM_MAX_CTAS if max_ctas is None else max_ctas),
    )  # fmt: skip
    if scatter is not None:
        bases = list(scatter[0]) + [None] * (8 - len(scatter[0]))
        args.scatter_d = (C.c_void_p * 8)(*bases)
        args.scatter_rows, args.scatter_row0 = int(scatter[1]), int(scatter[2])
    with torch.cuda.device(dev):
        rc = _timed("gemm", 2.0 * M * N * K, dev, lambda: L.load().qlin_gemm(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_gemm")
    return out


def bmm_i8(a: torch.Tensor, b_nk: torch.Tensor) -> torch.Tensor:
    """Batched int8 product: ``a [B, M, K]`` times ``b_nk [B, N, K]`` (both K-contiguous) -> int32 ``[B, M, N]``, exact.
    One ``qlin_gemm_batched`` call (include/qlin_b200.h); the integer product QBmmINT8Deploy stands for
    (fms_mo/modules/bmm.py:741-752 simulates it with a float matmul)."""
    if a.dim() != 3 or b_nk.dim() != 3 or a.shape[0] != b_nk.shape[0] or a.shape[2] != b_nk.shape[2]:
        raise RuntimeError("bmm_i8 takes a [B,M,K] and b_nk [B,N,K]")
    if a.dtype != torch.int8 or b_nk.dtype != torch.int8 or not a.is_cuda or a.device != b_nk.device:
        raise RuntimeError("bmm_i8 takes int8 CUDA tensors on one device")
    B, M, K = a.shape
    N = b_nk.shape[1]
    dev = a.device
    out = torch.empty((B, M, N), dtype=torch.int32, device=dev)
    if B == 0 or M == 0 or N == 0:
        return out
    if K % 16 != 0:  # rows of the operands must start on 16-byte boundaries: zero columns add nothing
        pad = 16 - K % 16
        a, b_nk = torch.nn.functional.pad(a, (0, pad)), torch.nn.functional.pad(b_nk, (0, pad))
    a, b_nk = a.contiguous(), b_nk.contiguous()
    Kp = a.shape[2]
    args = L.GemmArgs(
        a=_ptr(a), b=_ptr(b_nk), c=None, d=_ptr(out), row_scale=None, col_scale=None, bias=None, status=_ptr(status_word(dev)),
        lda=Kp, ldb=Kp, ldc=0, ldd=N, M=M, N=N, K=Kp, kind=L.DT_I8, chunk_k=0, trun_bits=0, max_acc_bits=32, trunc_then_acc=1,
        clamp_dl16=0, epilogue=L.EPI_RAW, row_scale_stride=0, col_scale_stride=0, prod_round=_ROUND[None], scale_round=_ROUND[None],
        mid_round=_ROUND[None], acc_round=_ROUND[None], out_dtype=L.DT_I32, max_ctas=int(GEMM_MAX_CTAS),
    )  # fmt: skip
    with torch.cuda.device(dev):
        rc = _timed("gemm", 2.0 * B * M * N * K, dev,
                    lambda: L.load().qlin_gemm_batched(C.byref(args), B, M * Kp, N * Kp, M * N, _stream(dev)))
        L.check(rc, "qlin_gemm_batched")
    return out


def _as_nk(m2: torch.Tensor) -> torch.Tensor:
    """The reference passes B as a ``[k,n]`` tensor, normally the ``.t()`` view of a row-major
    ``[n,k]`` weight.  Returns the ``[n,k]`` K-contiguous operand, copying only when ``m2`` is not
    such a view."""
    nk = m2.t()
    return nk if nk.stride(1) == 1 else nk.contiguous()


def imatmul(m1: torch.Tensor, m2: torch.Tensor) -> torch.Tensor:
    """``fms_mo::imatmul`` contract (fms_mo/custom_ext_kernels/utils.py:690-720): int8 ``m1 [..,k]``
    times int8 ``m2 [k,n]`` -> int32 ``[..,n]``."""
    lead = m1.shape[:-1]
    out = gemm(m1.reshape(-1, m1.shape[-1]), _as_nk(m2))
    return out.reshape(*lead, m2.shape[1])


_MIN_CHUNK_8BIT = 32


def tl_matmul_chunk_truncate(
    a,
    b,
    c=None,
    activation="",
    chunk_trun_bits=0,
    chunk_size=16,
    max_acc_bits=32,
    truncate_then_accumulate=True,
    cast_output_to_input_dtype=None,
    clamp_acc_to_dl16=False,
):
    """Drop-in for ``tl_matmul_chunk_truncate`` (fms_mo/custom_ext_kernels/triton_kernels.py:468-621)
    for int8 and float8_e4m3fn operands: ``a [m,k]`` contiguous, ``b [k,n]``; returns int32 for int8
    and float32 for fp8 (the reference does not cast 8-bit results back).  ``c``, if given, is the
    initial accumulator.  The chunk size is normalised exactly as the reference does: a power of
    two is raised to at least 32, anything else becomes 32; ``chunk_size == 8`` is emulated there by
    zero-interleaving both operands and is reproduced here the same way."""
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.is_contiguous(), "Matrix A must be contiguous"
    assert a.dtype == b.dtype, "Input dtypes inconsistent"
    if a.dtype not in (torch.int8, torch.float8_e4m3fn):
        raise RuntimeError(
            f"tl_matmul_chunk_truncate on B200 takes int8 or float8_e4m3fn operands, got {a.dtype}"
        )
    if activation not in ("", None):
        raise RuntimeError(f"activation {activation!r} is not supported")
    if cast_output_to_input_dtype:
        raise RuntimeError("8-bit results are returned in the accumulator dtype")
    f8 = a.dtype == torch.float8_e4m3fn
    if chunk_size == 8:
        ratio = _MIN_CHUNK_8BIT // chunk_size
        a_p = torch.zeros(a.shape[0], a.shape[1] * ratio, dtype=a.dtype, device=a.device)
        a_p.view(torch.int8)[:, ::ratio] = a.view(torch.int8)
        b_nk = _as_nk(b)
        b_p = torch.zeros(b_nk.shape[0], b_nk.shape[1] * ratio, dtype=b.dtype, device=b.device)
        b_p.view(torch.int8)[:, ::ratio] = b_nk.view(torch.int8)
        a, b_nk = a_p, b_p
        chunk_size = _MIN_CHUNK_8BIT
    else:
        b_nk = _as_nk(b)
        pow2 = chunk_size > 0 and (chunk_size & (chunk_size - 1)) == 0
        chunk_size = max(chunk_size, _MIN_CHUNK_8BIT) if pow2 else _MIN_CHUNK_8BIT
    if f8:
        assert chunk_trun_bits < 23, "FP32 accumulator only has 23 mantissa bits"
        if clamp_acc_to_dl16:
            chunk_trun_bits = 14
    acc_dtype = torch.float32 if f8 else torch.int32
    c_in = None
    if c is not None:
        assert c.shape[0] == a.shape[0] and c.shape[1] == b.shape[1], "C shape is inconsistent with A B."
        c_in = c.to(acc_dtype)
    return gemm(
        a,
        b_nk,
        c=c_in,
        chunk_k=chunk_size,
        trun_bits=chunk_trun_bits,
        max_acc_bits=max_acc_bits,
        trunc_then_acc=truncate_then_accumulate,
        clamp_dl16=bool(clamp_acc_to_dl16) and f8,
    )


# --------------------------------------------------------------------------------------------------
# Row-wise quantisation
# --------------------------------------------------------------------------------------------------
def smooth_reciprocal(smooth_f32: torch.Tensor) -> torch.Tensor:
    """The ``smooth_rcp`` operand of qlin_act_quant: the IEEE fp32 reciprocal of every smoothing scale,
    NaN where the kernel's three-operation exact division is not proven (significand all ones, or a
    magnitude outside [1e-15, 1e15]) so that those columns take the ordinary division."""
    s = smooth_f32.float().reshape(-1).contiguous()
    r = torch.reciprocal(s)
    bad = ((s.view(torch.int32) & 0x7FFFFF) == 0x7FFFFF) | ~((s.abs() > 1e-15) & (s.abs() < 1e15))
    return torch.where(bad, torch.full_like(r, float("nan")), r).contiguous()


def act_quant(
    x: torch.Tensor,
    *,
    mode: int = L.Q_I8_DYN,
    smooth: Optional[torch.Tensor] = None,
    smooth_rcp: Optional[torch.Tensor] = None,
    smooth_mul: bool = False,
    native_chain: int = 0,
    clamp_codes: bool = False,
    levels: int = 127,
    want_codes: bool = True,
    want_dq: bool = False,
    scale_in: Optional[torch.Tensor] = None,
    dl8_flush: bool = False,
    scale0: float = 1.0,
    zp0: float = 0.0,
    lo: float = 0.0,
    hi: float = 0.0,
    shift: float = 0.0,
    add2: float = 0.0,
    dyn_eps: float = 1e-5,
    f8_e5m2: bool = False,
) -> Tuple[Optional[torch.Tensor], torch.Tensor, Optional[torch.Tensor]]:
    """Row-wise 8-bit quantisation of a 2-D tensor; returns ``(codes, scale[rows], dq)``.
    See ``qlin_act_quant`` in include/qlin_b200.h for the modes."""
    dev = _require_cuda(x, smooth, scale_in)
    if x.dim() != 2:
        raise RuntimeError("act_quant takes a 2-D tensor")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"unsupported activation dtype {x.dtype}")
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    code_dtype = torch.int8
    if mode == L.Q_F8_DYN or (mode == L.Q_F8_TENSOR and not f8_e5m2):
        code_dtype = torch.float8_e4m3fn
    elif mode == L.Q_F8_TENSOR:
        code_dtype = torch.float8_e5m2
    codes = torch.empty((rows, cols), dtype=code_dtype, device=dev) if want_codes else None
    dq = torch.empty((rows, cols), dtype=x.dtype, device=dev) if want_dq else None
    scale = torch.empty((rows,), dtype=torch.float32, device=dev)
    sm = _f32(smooth)
    if sm is not None and sm.numel() != cols:
        raise RuntimeError("smooth must have one entry per column")
    rsm = None
    if sm is not None and not smooth_mul:
        rsm = _f32(smooth_rcp) if smooth_rcp is not None else smooth_reciprocal(sm)
    si = _f32(scale_in)
    if rows == 0 or cols == 0:
        return codes, scale, dq
    args = L.QuantArgs(
        x=_ptr(x), smooth=_ptr(sm), smooth_rcp=_ptr(rsm), scale_in=_ptr(si), codes=_ptr(codes), scale_out=_ptr(scale), dq_out=_ptr(dq),
        status=None, ldx=x.stride(0), ldq=cols, lddq=cols, rows=rows, cols=cols, x_dtype=_DT[x.dtype], mode=mode,
        native_chain=int(native_chain), smooth_mul=int(bool(smooth_mul)), clamp_codes=int(bool(clamp_codes)),
        qmax_levels=int(levels), dl8_flush=int(bool(dl8_flush)),
        scale_in_stride=(0 if si is None or si.numel() == 1 else 1),
        scale0=scale0, zp0=zp0, lo=lo, hi=hi, shift=shift, add2=add2, dyn_eps=dyn_eps, f8_format=int(bool(f8_e5m2)),
    )  # fmt: skip
    nbytes = rows * cols * (x.element_size() + (1 if want_codes else 0) + (x.element_size() if want_dq else 0)) + 4 * rows
    nbytes += 4 * cols if sm is not None else 0
    with torch.cuda.device(dev):
        rc = _timed("act_quant", float(nbytes), dev, lambda: L.load().qlin_act_quant(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_act_quant")
    return codes, scale, dq


def weight_fq_perch(
    w: torch.Tensor,
    *,
    num_bits: int = 8,
    mode: int = L.W_SAWB,
    clip: Optional[torch.Tensor] = None,
    smooth: Optional[torch.Tensor] = None,
    native_mul: bool = True,
    clip_dtype: Optional[torch.dtype] = None,
    want_dq: bool = True,
    want_codes: bool = False,
    c0: float = 0.0,
    c1: float = 0.0,
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], torch.Tensor]:
    """Per-output-channel symmetric fake quantisation of ``w [rows, cols]``; returns
    ``(dq, codes, clip[rows])``.  See ``qlin_weight_fq_perch`` in include/qlin_b200.h."""
    dev = _require_cuda(w, clip, smooth)
    if w.dim() != 2:
        w = w.reshape(w.shape[0], -1)
    if w.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"unsupported weight dtype {w.dtype}")
    if w.stride(1) != 1:
        w = w.contiguous()
    rows, cols = w.shape
    if mode == L.W_GIVEN:
        if clip is None or clip.numel() != rows:
            raise RuntimeError("W_GIVEN needs one clip value per row")
        clip_io = _f32(clip).clone()
    else:
        clip_io = torch.empty((rows,), dtype=torch.float32, device=dev)
    dq = torch.empty((rows, cols), dtype=w.dtype, device=dev) if want_dq else None
    codes = torch.empty((rows, cols), dtype=torch.int8, device=dev) if want_codes else None
    sm = _f32(smooth)
    if rows == 0 or cols == 0:
        return dq, codes, clip_io
    args = L.WfqArgs(
        w=_ptr(w), smooth=_ptr(sm), dq_out=_ptr(dq), codes=_ptr(codes), clip_io=_ptr(clip_io),
        ldw=w.stride(0), ldo=cols, ldq=cols, rows=rows, cols=cols, dtype=_DT[w.dtype], num_bits=int(num_bits),
        mode=int(mode), native_mul=int(bool(native_mul)), clip_dtype=(0 if clip_dtype is None or clip_dtype == w.dtype else _DT[clip_dtype]), c0=float(c0), c1=float(c1),
    )  # fmt: skip
    nbytes = rows * cols * (w.element_size() * (2 if want_dq else 1) + (1 if want_codes else 0)) + 4 * rows
    with torch.cuda.device(dev):
        rc = _timed("weight_fq", float(nbytes), dev, lambda: L.load().qlin_weight_fq_perch(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_weight_fq_perch")
    return dq, codes, clip_io


def tensor_fq(
    x: torch.Tensor,
    *,
    kind: int = L.PT_INT_SYM,
    mode: int = L.W_SAWB,
    num_bits: int = 8,
    clip: Optional[torch.Tensor] = None,
    align_zero: bool = True,
    dequantize: bool = True,
    want_out: bool = True,
    c0: float = 0.0,
    c1: float = 0.0,
) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """Per-tensor fake quantisation; returns ``(out, clip[1] fp32)``.  See ``qlin_tensor_fq`` in
    include/qlin_b200.h."""
    dev = _require_cuda(x, clip)
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"unsupported dtype {x.dtype}")
    xc = x if x.is_contiguous() else x.contiguous()
    if mode == L.W_GIVEN:
        if kind != L.PT_F8_SAT and (clip is None or clip.numel() != 1):
            raise RuntimeError("W_GIVEN needs one clip value")
        clip_io = _clip_f32(clip, dev).clone() if clip is not None else torch.zeros(1, dtype=torch.float32, device=dev)
        ws = None
    else:
        clip_io = torch.empty((1,), dtype=torch.float32, device=dev)
        ws = torch.empty((L.load().qlin_tensor_fq_workspace_bytes(xc.numel()) // 4,), dtype=torch.float32, device=dev)
    out = torch.empty_like(xc) if want_out else None
    if xc.numel() == 0:
        return out, clip_io
    args = L.TensorFqArgs(
        x=_ptr(xc), out=_ptr(out), clip_io=_ptr(clip_io), workspace=_ptr(ws), numel=xc.numel(), dtype=_DT[xc.dtype],
        num_bits=int(num_bits), mode=int(mode), kind=int(kind), align_zero=int(bool(align_zero)),
        dequantize=int(bool(dequantize)), c0=float(c0), c1=float(c1),
    )  # fmt: skip
    nbytes = xc.numel() * xc.element_size() * ((1 if mode != L.W_GIVEN else 0) + (2 if want_out else 0))
    with torch.cuda.device(dev):
        rc = _timed("tensor_fq", float(nbytes), dev, lambda: L.load().qlin_tensor_fq(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_tensor_fq")
    return (out.view_as(x) if out is not None else None), clip_io


# --------------------------------------------------------------------------------------------------
# PACT+ two-sided fake quantisation
# --------------------------------------------------------------------------------------------------
def _clip_f32(t: torch.Tensor, dev: torch.device) -> torch.Tensor:
    t = t.detach().reshape(-1)[:1]
    if t.dtype != torch.float32 or t.device != dev:
        t = t.to(device=dev, dtype=torch.float32)
    return t.contiguous()


def pact2_fwd(x: torch.Tensor, clip_val: torch.Tensor, clip_valn: Optional[torch.Tensor], num_bits: int, align_zero: bool,
              variant: int = L.PACT_TWO_SIDED) -> torch.Tensor:
    """PACTplus2STE.forward with dequantize=True (fms_mo/quant/quantizers.py:1949-2055); ``variant`` selects the
    one-sided (PACTplusSTE, :1016) or symmetric (PACTplusSymSTE_rev1, :1073) member of the family."""
    dev = _require_cuda(x)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    cv = _clip_f32(clip_val, dev)
    cvn = _clip_f32(clip_valn, dev) if clip_valn is not None else None
    args = L.Pact2Args(
        x=_ptr(xc), grad_out=None, out=_ptr(out), clip_val=_ptr(cv), clip_valn=_ptr(cvn), grad_clip=None,
        workspace=None, numel=xc.numel(), dtype=_DT[xc.dtype], num_bits=int(num_bits), align_zero=int(bool(align_zero)),
        variant=int(variant),
    )  # fmt: skip
    with torch.cuda.device(dev):
        rc = _timed("pact2_fwd", 2.0 * xc.numel() * xc.element_size(), dev, lambda: L.load().qlin_pact2_fwd(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_pact2_fwd")
    return out


def pact2_bwd(
    x: torch.Tensor, grad_out: torch.Tensor, clip_val: torch.Tensor, clip_valn: Optional[torch.Tensor], num_bits: int,
    align_zero: bool, variant: int = L.PACT_TWO_SIDED,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """PACTplus2STE.backward (fms_mo/quant/quantizers.py:2058-2102): returns ``(grad_x, [grad_cv, grad_cvn])``."""
    dev = _require_cuda(x, grad_out)
    xc = x.contiguous()
    gc = grad_out.contiguous()
    if gc.dtype != xc.dtype:
        gc = gc.to(xc.dtype)
    gx = torch.empty_like(xc)
    cv = _clip_f32(clip_val, dev)
    cvn = _clip_f32(clip_valn, dev) if clip_valn is not None else None
    lib = L.load()
    ws = torch.empty((max(1, lib.qlin_pact2_bwd_workspace_bytes(xc.numel()) // 4),), dtype=torch.float32, device=dev)
    grads = torch.empty((2,), dtype=torch.float32, device=dev)
    args = L.Pact2Args(
        x=_ptr(xc), grad_out=_ptr(gc), out=_ptr(gx), clip_val=_ptr(cv), clip_valn=_ptr(cvn), grad_clip=_ptr(grads),
        workspace=_ptr(ws), numel=xc.numel(), dtype=_DT[xc.dtype], num_bits=int(num_bits),
        align_zero=int(bool(align_zero)), variant=int(variant),
    )  # fmt: skip
    with torch.cuda.device(dev):
        rc = _timed("pact2_bwd", 3.0 * xc.numel() * xc.element_size(), dev, lambda: lib.qlin_pact2_bwd(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_pact2_bwd")
    return gx, grads


# --------------------------------------------------------------------------------------------------
# Decoder-block fusions: (residual add +) RMSNorm / SiLU * up, then per-token quantisation for up to
# three Linears that share the input; rotary embedding.
# --------------------------------------------------------------------------------------------------
def block_quant(
    x: torch.Tensor,
    *,
    prologue: int = L.BLOCK_PLAIN,
    r: Optional[torch.Tensor] = None,
    norm_w: Optional[torch.Tensor] = None,
    smooth_rcps: Sequence[Optional[torch.Tensor]] = (None,),
    mode: int = L.BLOCK_DYN,
    scale_in: Optional[torch.Tensor] = None,
    scale_in_parts: int = 0,
    scale_in_stride: int = 0,
    store_sum: bool = False,
    sum_into: Optional[torch.Tensor] = None,
    r_parts: int = 0,
    r_part_stride: int = 0,
    dst: Optional[Tuple[Sequence[int], Sequence[int], Sequence[int], int]] = None,
    want_h: bool = False,
    max_ctas: int = 0,
    r_multimem: bool = False,
    dst_multimem: bool = False,
    r_ptr: Optional[int] = None,
    levels: int = 127,
    norm_eps: float = 1e-5,
    dyn_eps: float = 1e-5,
):
    """See ``qlin_block_quant`` in include/qlin_b200.h.  ``x`` (and ``r``) are 2-D bf16 with unit column
    stride; ``smooth_rcps`` holds one fp32 reciprocal vector (or None) per Linear that consumes the row.
    Returns ``(codes list, scales list, x_plus_r or None, h or None)``; with ``BLOCK_SCALE_ONLY`` the codes are None.
    ``r_ptr`` gives the addend as a raw device address with the row pitch of ``x`` (a multicast mapping when
    ``r_multimem``); ``dst_multimem`` says that ``dst[0][0]`` is a multicast address."""
    dev = _require_cuda(x, r, norm_w, scale_in, *smooth_rcps)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise RuntimeError("block_quant takes a 2-D bf16 tensor with contiguous rows")
    if r is not None and (r.dtype != torch.bfloat16 or r.shape != x.shape or r.stride(1) != 1):
        raise RuntimeError("r must match x")
    rows, cols = x.shape
    nout = len(smooth_rcps)
    if dst is not None:
        # (base address per destination, byte offset of each output's codes, of each output's scales, first row):
        # every destination (this GPU's buffer or a peer's) receives the codes and scales of these rows
        codes, scales = [None] * nout, [None] * nout
    else:
        codes = [None if mode == L.BLOCK_SCALE_ONLY else torch.empty((rows, cols), dtype=torch.int8, device=dev) for _ in range(nout)]
        given_as_is = mode == L.BLOCK_GIVEN_SCALE and scale_in_parts <= 1
        scales = [scale_in if given_as_is else torch.empty((rows,), dtype=torch.float32, device=dev) for _ in range(nout)]
    x_out = None
    has_r = r is not None or r_ptr is not None
    if has_r and sum_into is not None:
        x_out = sum_into
    elif has_r and store_sum:
        x_out = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
    h_out = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev) if want_h else None
    if rows == 0 or cols == 0:
        return codes, scales, x_out, h_out
    p3 = C.c_void_p * 3
    i3 = C.c_int64 * 3
    pad = [None] * (3 - nout)
    args = L.BlockQuantArgs(
        x=_ptr(x), r=(int(r_ptr) if r_ptr is not None else _ptr(r)), r_parts=int(r_parts), r_part_stride=int(r_part_stride), x_out=_ptr(x_out), h_out=_ptr(h_out),
        norm_w=_ptr(norm_w),
        smooth_rcp=p3(*[_ptr(t) for t in list(smooth_rcps) + pad]), codes=p3(*[_ptr(t) for t in codes + pad]),
        scale_out=p3(*[(_ptr(t) if (mode != L.BLOCK_GIVEN_SCALE or scale_in_parts > 1) else None) for t in scales + pad]), scale_in=_ptr(scale_in), scale_in_parts=int(scale_in_parts), scale_in_stride=int(scale_in_stride),
        ldx=x.stride(0), ldr=(r.stride(0) if r is not None else (cols if r_ptr is not None else 0)), ldxo=(x_out.stride(0) if x_out is not None else cols),
        ldh=cols, ldq=i3(cols, cols, cols),
        rows=rows, cols=cols, nout=nout, prologue=int(prologue), mode=int(mode), qmax_levels=int(levels),
        norm_eps=float(norm_eps), dyn_eps=float(dyn_eps), max_ctas=int(max_ctas),
        r_multimem=int(bool(r_multimem)), dst_multimem=int(bool(dst_multimem)),
    )  # fmt: skip
    ndst = 1
    if dst is not None:
        ndst = len(dst[0])
        args.dst_base = (C.c_void_p * 8)(*(list(dst[0]) + [None] * (8 - ndst)))
        args.codes_off = i3(*(list(dst[1]) + [0] * (3 - nout)))
        args.scale_off = i3(*(list(dst[2]) + [0] * (3 - nout)))
        args.ndst, args.dst_row0 = ndst, int(dst[3])
    nbytes = rows * cols * (2 * (1 + (max(1, r_parts) if has_r else 0) + (x_out is not None) + (h_out is not None))
                            + (0 if mode == L.BLOCK_SCALE_ONLY else nout * ndst))
    with torch.cuda.device(dev):
        rc = _timed("block_quant", float(nbytes), dev, lambda: L.load().qlin_block_quant(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_block_quant")
    return codes, scales, x_out, h_out


def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int) -> torch.Tensor:
    """Rotary embedding in place on ``x [tokens, heads, head_dim]`` bf16 (``qlin_rope``)."""
    dev = _require_cuda(x, cos, sin)
    if x.dtype != torch.bfloat16 or x.dim() != 3 or x.stride(2) != 1 or x.stride(1) != x.shape[2]:
        raise RuntimeError("rope_ takes [tokens, heads, head_dim] bf16 with contiguous heads")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or not cos.is_contiguous() or not sin.is_contiguous():
        raise RuntimeError("cos / sin are contiguous fp32 [seq_len, head_dim / 2]")
    args = L.RopeArgs(x=_ptr(x), cos=_ptr(cos), sin=_ptr(sin), ld_token=x.stride(0), tokens=x.shape[0], heads=x.shape[1],
                      head_dim=x.shape[2], seq_len=int(seq_len))  # fmt: skip
    with torch.cuda.device(dev):
        rc = _timed("rope", 4.0 * x.numel(), dev, lambda: L.load().qlin_rope(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_rope")
    return x


def shard_reduce_(x: torch.Tensor, src_multicast: int, max_ctas: int = 0) -> torch.Tensor:
    """``x += sum over GPUs of their partial outputs`` for this GPU's block of rows, read through the multicast mapping at
    ``src_multicast`` (row pitch = the row length of ``x``); in place on the bf16 ``x`` (``qlin_shard_reduce``)."""
    dev = _require_cuda(x)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise RuntimeError("shard_reduce_ takes a 2-D bf16 tensor with contiguous rows")
    rows, cols = x.shape
    args = L.ShardReduceArgs(src_multicast=int(src_multicast), add=_ptr(x), out=_ptr(x), ld_src=cols, ld_add=x.stride(0), ld_out=x.stride(0),
                             rows=rows, cols=cols, max_ctas=int(max_ctas))  # fmt: skip
    with torch.cuda.device(dev):
        rc = _timed("shard_reduce", float(rows * cols * 2 * 3), dev, lambda: L.load().qlin_shard_reduce(C.byref(args), _stream(dev)))
        L.check(rc, "qlin_shard_reduce")
    return x


# --------------------------------------------------------------------------------------------------
# Calibration statistics
# --------------------------------------------------------------------------------------------------
def col_absmax(x: torch.Tensor, running: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-input-channel absolute maximum of ``x`` viewed as ``[-1, x.shape[-1]]`` (``qlin_col_absmax``): the statistic of
    activation_stats (fms_mo/quant/ptq.py:2586-2596).  With ``running`` (fp32 ``[channels]``, on the device) the result
    is folded into it in place -- the maximum over all batches seen -- and ``running`` is returned."""
    dev = _require_cuda(x, running)
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"unsupported dtype {x.dtype}")
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows, cols = x2.shape
    if running is None:
        out = torch.empty((cols,), dtype=torch.float32, device=dev)
    else:
        if running.dtype != torch.float32 or running.shape != (cols,) or not running.is_contiguous():
            raise RuntimeError("running must be a contiguous fp32 vector with one entry per channel")
        out = running
    args = L.ColAbsmaxArgs(x=_ptr(x2), amax_io=_ptr(out), ldx=(x2.stride(0) if rows > 1 else cols), rows=rows, cols=cols, dtype=_DT[x2.dtype],
                           accumulate=int(running is not None))  # fmt: skip
    with torch.cuda.device(dev):
        rc = _timed("col_absmax", float(rows * cols * x2.element_size() + 4 * cols), dev,
                    lambda: L.load().qlin_col_absmax(C.byref(args), _stream(dev)))  # fmt: skip
        L.check(rc, "qlin_col_absmax")
    return out


# --------------------------------------------------------------------------------------------------
# torch custom ops (namespace qlin_b200), the counterpart of the reference's fms_mo::* registrations
# (fms_mo/custom_ext_kernels/utils.py:674-802).  Fake implementations give shapes and dtypes so the
# ops can be traced.
# --------------------------------------------------------------------------------------------------
@torch.library.custom_op("qlin_b200::imatmul", mutates_args=())
def _imatmul_op(m1: torch.Tensor, m2: torch.Tensor) -> torch.Tensor:
    return imatmul(m1, m2)


@_imatmul_op.register_fake
def _(m1, m2):
    return m1.new_empty((*m1.shape[:-1], m2.shape[1]), dtype=torch.int32)


@torch.library.custom_op("qlin_b200::act_quant_i8", mutates_args=())
def _act_quant_i8_op(x: torch.Tensor, smooth: Optional[torch.Tensor], native_chain: int) -> Tuple[torch.Tensor, torch.Tensor]:
    codes, scale, _ = act_quant(x.reshape(-1, x.shape[-1]), mode=L.Q_I8_DYN, smooth=smooth, native_chain=native_chain)
    return codes.reshape(x.shape), scale


@_act_quant_i8_op.register_fake
def _(x, smooth, native_chain):
    return x.new_empty(x.shape, dtype=torch.int8), x.new_empty((x.numel() // x.shape[-1],), dtype=torch.float32)


@torch.library.custom_op("qlin_b200::iaddmm", mutates_args=())
def _iaddmm_op(bias: torch.Tensor, m1: torch.Tensor, m2: torch.Tensor, scale_i: torch.Tensor, scale_w: torch.Tensor) -> torch.Tensor:
    """fms_mo::iaddmm (fms_mo/custom_ext_kernels/utils.py:729-746): ``scale_i.float() * imatmul(m1, m2) * scale_w + bias``."""
    return gemm(m1, _as_nk(m2), epilogue=L.EPI_SCALE_SEQ, row_scale=scale_i, col_scale=scale_w, bias=bias, out_dtype=torch.float32)


@_iaddmm_op.register_fake
def _(bias, m1, m2, scale_i, scale_w):
    return m1.new_empty((m1.shape[0], m2.shape[1]), dtype=torch.float32)


def tensor_absmax(x: torch.Tensor) -> torch.Tensor:
    """max|x| over the whole tensor as a 1-element fp32 device tensor (``qlin_tensor_fq`` statistics only)."""
    return tensor_fq(x, kind=L.PT_INT_SYM, mode=L.W_MAX, want_out=False)[1]


def fp8_quant_per_tensor(x2: torch.Tensor, *, e5m2: bool = False, eps: float = 1e-5, dl8_flush: bool = False):
    """The per-tensor FP8 scaling of LinearFuncFPxFwdBwd (fms_mo/modules/linear.py:1939-1953 forward, e4m3, scale clamped at
    1e-5; :2003-2017 backward, e5m2, no clamp): ``scale = max(amax / fp8_max, eps)``, ``codes = fp8(x / scale)``.
    Returns ``(codes [rows, cols], scale [1] fp32)``; nothing is read back to the host."""
    amax = tensor_absmax(x2)
    native = 0 if x2.dtype == torch.float32 else 3
    codes, scale, _ = act_quant(x2, mode=L.Q_F8_TENSOR, native_chain=native, scale_in=amax, scale0=(57344.0 if e5m2 else 448.0),
                                dyn_eps=eps, f8_e5m2=e5m2, dl8_flush=dl8_flush)  # fmt: skip
    return codes, scale[:1]


def _scalar(t) -> float:
    return float(t.reshape(-1)[0].item()) if isinstance(t, torch.Tensor) else float(t)


@torch.library.custom_op("qlin_b200::q_iaddmm_dq", mutates_args=())
def _q_iaddmm_dq_op(bias: torch.Tensor, m1: torch.Tensor, m2: torch.Tensor, scale_i: torch.Tensor, zp_i: torch.Tensor,
                    scale_w: torch.Tensor) -> torch.Tensor:  # fmt: skip
    """fms_mo::q_iaddmm_dq (fms_mo/custom_ext_kernels/utils.py:748-782): quantise the float ``m1 [m,k]`` with a
    static per-tensor scale and zero point (uint8 codes shifted by 128), int8 GEMM with ``m2 [k,n]``, then
    ``(scale_i.float() * acc * scale_w + bias).to(m1.dtype)``.  The scale and zero point are read on the host."""
    assert m2.dtype == torch.int8, f"weight tensor is of incorrect dtype {m2.dtype}"
    native = 3 if (m1.dtype != torch.float32 and scale_i.dtype == m1.dtype) else 0
    codes, _, _ = act_quant(m1, mode=L.Q_I8_STATIC, native_chain=native, scale0=_scalar(scale_i), zp0=_scalar(zp_i), shift=128.0)
    return gemm(codes, _as_nk(m2), epilogue=L.EPI_SCALE_SEQ, row_scale=scale_i.reshape(-1)[:1], col_scale=scale_w, bias=bias,
                out_dtype=m1.dtype)  # fmt: skip


@_q_iaddmm_dq_op.register_fake
def _(bias, m1, m2, scale_i, zp_i, scale_w):
    return m1.new_empty((m1.shape[0], m2.shape[1]))


@torch.library.custom_op("qlin_b200::q_per_t_sym", mutates_args=())
def _q_per_t_sym_op(x: torch.Tensor, s: torch.Tensor, zp: torch.Tensor) -> torch.Tensor:
    """fms_mo::q_per_t_sym (fms_mo/custom_ext_kernels/utils.py:792-794):
    ``torch.quantize_per_tensor(x, s, zp, torch.qint8).int_repr()`` for fp32 ``x``."""
    if x.dtype != torch.float32:
        raise RuntimeError("q_per_t_sym takes a float32 tensor, as torch.quantize_per_tensor does")
    codes, _, _ = act_quant(x.reshape(-1, x.shape[-1]), mode=L.Q_I8_AFFINE_RCP, scale0=_scalar(s), zp0=_scalar(zp))
    return codes.reshape(x.shape)


@_q_per_t_sym_op.register_fake
def _(x, s, zp):
    return x.new_empty(x.shape, dtype=torch.int8)
