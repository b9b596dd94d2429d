"""Oracle for the chunk-truncating matmuls (test infrastructure, see ``oracle/__init__.py``).

Restates ``imatmul_kernel`` and ``matmul_kernel`` / ``matmul_kernel_DABC`` with the host-side
normalisation of ``tl_matmul_chunk_truncate``
(fms_mo/custom_ext_kernels/triton_kernels.py:211-302, :96-205, :305-423, :468-621).
"""

from __future__ import annotations

import numpy as np
import torch

MIN_CHUNK_8BIT = 32  # triton_kernels.py:528


def normalise_chunk_size(chunk_size: int) -> int:
    """triton_kernels.py:550-555: a power of two is raised to at least 32, anything else becomes 32
    (8-bit operands).  ``chunk_size == 8`` is handled by the caller through zero-interleaving
    (triton_kernels.py:532-549), which is arithmetically a chunk of 8 real elements."""
    pow2 = chunk_size > 0 and (chunk_size & (chunk_size - 1)) == 0
    return max(chunk_size, MIN_CHUNK_8BIT) if pow2 else MIN_CHUNK_8BIT


def _wrap_i32(x: np.ndarray) -> np.ndarray:
    return ((x + 2**31) % 2**32 - 2**31).astype(np.int64)


def imatmul_chunk_truncate(
    a: torch.Tensor,
    b_kn: torch.Tensor,
    c: torch.Tensor | None = None,
    chunk_trun_bits: int = 0,
    chunk_size: int = 16,
    max_acc_bits: int = 32,
    truncate_then_accumulate: bool = True,
) -> torch.Tensor:
    """int8 ``a [m,k]`` x int8 ``b_kn [k,n]`` -> int32 ``[m,n]`` with the per-chunk clamp and
    round-shift of ``imatmul_kernel`` (triton_kernels.py:262-291):

        p = dot(a_chunk, b_chunk)                      (int32)
        if max_acc_bits < 32: p = clamp(p, -2^(b-1), 2^(b-1)-1)
        if t: p = ((p + (1 << (t-1))) >> t) << t       (arithmetic shift)
        acc += p            (or acc = f(acc + dot) when truncate_then_accumulate is False)

    int32 arithmetic wraps.  The chunk products are computed as float64 matmuls, which are exact
    for |p| < 2^53."""
    assert a.dtype == torch.int8 and b_kn.dtype == torch.int8
    m, k = a.shape
    n = b_kn.shape[1]
    if chunk_size == 8:
        chunk = 8  # zero-interleaved operands: every 32-wide chunk holds 8 real elements
    else:
        chunk = normalise_chunk_size(chunk_size)
    t = int(chunk_trun_bits)
    rb = (1 << (t - 1)) if t > 0 else 0
    lo, hi = -(1 << (max_acc_bits - 1)), (1 << (max_acc_bits - 1)) - 1
    acc = np.zeros((m, n), dtype=np.int64) if c is None else c.to(torch.int64).numpy().copy()
    a64 = a.to(torch.float64)
    b64 = b_kn.to(torch.float64)
    if t == 0 and max_acc_bits >= 32:
        # no per-chunk function: the chunking is not observable, one exact product suffices
        return torch.from_numpy(_wrap_i32(acc + (a64 @ b64).numpy().astype(np.int64)).astype(np.int32))
    for k0 in range(0, k, chunk):
        p = (a64[:, k0 : k0 + chunk] @ b64[k0 : k0 + chunk, :]).numpy().astype(np.int64)
        if not truncate_then_accumulate:
            p = _wrap_i32(acc + p)
        if max_acc_bits < 32:
            p = np.clip(p, lo, hi)
        if t != 0:
            p = _wrap_i32(p + rb)
            p = (p >> t) << t
        acc = _wrap_i32(acc + p) if truncate_then_accumulate else _wrap_i32(p)
    return torch.from_numpy(acc.astype(np.int32))


def round_and_trun_f32(x: torch.Tensor, trun_bits: int, clamp_dl16: bool) -> torch.Tensor:
    """``round_and_trun`` (triton_kernels.py:432-465) on an fp32 tensor: add the round bit to the
    IEEE-754 bit pattern, mask the low bits, then the optional DL16 clamp / flush."""
    if clamp_dl16:
        trun_bits = 14
    bits = x.contiguous().view(torch.int32).numpy().view(np.uint32).astype(np.uint64)
    rb = (1 << (trun_bits - 1)) if trun_bits > 0 else 0
    mask = (~((1 << trun_bits) - 1)) & 0xFFFFFFFF
    bits = ((bits + rb) & 0xFFFFFFFF) & mask
    y = torch.from_numpy(bits.astype(np.uint32).view(np.float32).copy()).reshape(x.shape)
    if clamp_dl16:
        dl16_max, dl16_min = 8581545984.0, 4.665707820095122e-10
        y = torch.where(y >= dl16_max, torch.full_like(y, float("inf")), y)
        y = torch.where(y <= -dl16_max, torch.full_like(y, float("-inf")), y)
        y = torch.where(y.abs() < dl16_min, torch.zeros_like(y), y)
    return y


def fmatmul_chunk_truncate(
    a: torch.Tensor,
    b_kn: torch.Tensor,
    c: torch.Tensor | None = None,
    chunk_trun_bits: int = 0,
    chunk_size: int = 16,
    truncate_then_accumulate: bool = True,
    clamp_acc_to_dl16: bool = False,
) -> torch.Tensor:
    """Float matmul of ``matmul_kernel`` (triton_kernels.py:164-186) for operands that hold
    float8_e4m3 values: per chunk an fp32 dot product, mantissa round / truncate on the chunk
    product (or on the running sum), fp32 accumulation.  ``a`` and ``b_kn`` may be float8 tensors
    or fp32 tensors holding fp8 values; the result is fp32."""
    a32 = a.to(torch.float32)
    b32 = b_kn.to(torch.float32)
    m, k = a32.shape
    n = b32.shape[1]
    chunk = 8 if chunk_size == 8 else normalise_chunk_size(chunk_size)
    acc = torch.zeros((m, n), dtype=torch.float32) if c is None else c.to(torch.float32).clone()
    plain = chunk_trun_bits == 0 and not clamp_acc_to_dl16
    if plain:
        # without a per-chunk function the chunking only fixes the fp32 summation order
        return acc + (a32.double() @ b32.double()).float() if c is not None else (a32.double() @ b32.double()).float()
    for k0 in range(0, k, chunk):
        p = (a32[:, k0 : k0 + chunk].double() @ b32[k0 : k0 + chunk, :].double()).float()
        if truncate_then_accumulate:
            acc = acc + round_and_trun_f32(p, chunk_trun_bits, clamp_acc_to_dl16)
        else:
            acc = round_and_trun_f32(acc + p, chunk_trun_bits, clamp_acc_to_dl16)
    return acc
