"""The file a maintainer of fms-model-optimizer would add as ``fms_mo/custom_ext_kernels/b200.py``.

It is self-contained on purpose: ctypes, torch and the shared library, nothing else of this package, so that it can be
copied into the reference as it stands (INTEGRATION.md shows where it is hooked in).  ``b200_imatmul`` has the contract
of the ``mm_func`` that ``imatmul_ops_reg`` registers as ``fms_mo::imatmul`` (fms_mo/custom_ext_kernels/utils.py:642-720):
int8 ``m1 [m, k]``, int8 ``m2 [k, n]`` given as the ``.t()`` view of the ``[n, k]`` weight, int32 ``[m, n]`` back, with the
chunk-truncation keywords of ``tl_matmul_chunk_truncate`` (fms_mo/custom_ext_kernels/triton_kernels.py:468).
tests/test_gpu_integration_stub.py runs exactly this code against the oracle.
"""

import ctypes as C
import os

import torch

_LIB_PATH = os.environ.get("QLIN_B200_LIB", os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libqlin_b200.so"))
_lib = C.CDLL(_LIB_PATH)


class GemmArgs(C.Structure):  # mirrors qlin_gemm_args in include/qlin_b200.h, field for field
    _fields_ = (
        [(n, C.c_void_p) for n in ("a", "b", "c", "d", "row_scale", "col_scale", "bias", "status")]
        + [(n, C.c_int64) for n in ("lda", "ldb", "ldc", "ldd")]
        + [(n, C.c_int32) for n in ("M", "N", "K", "kind", "chunk_k", "trun_bits", "max_acc_bits", "trunc_then_acc", "clamp_dl16",
                                    "epilogue", "row_scale_stride", "col_scale_stride", "prod_round", "scale_round", "mid_round",
                                    "acc_round", "out_dtype")]  # fmt: skip
        + [("scatter_d", C.c_void_p * 8), ("scatter_rows", C.c_int32), ("scatter_row0", C.c_int32), ("max_ctas", C.c_int32)]
    )


_lib.qlin_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
_lib.qlin_gemm.restype = C.c_int
_lib.qlin_last_error_string.restype = C.c_char_p
QLIN_DT_I8, QLIN_DT_I32 = 1, 3


def b200_imatmul(m1, m2, chunk_trun_bits=0, chunk_size=16, max_acc_bits=32, truncate_then_accumulate=True):
    w = m2.t()  # [n, k] with k contiguous when m2 is the .t() view of the weight: no copy
    if w.stride(1) != 1:
        w = w.contiguous()
    out = torch.empty((m1.shape[0], w.shape[0]), dtype=torch.int32, device=m1.device)
    pow2 = chunk_size > 0 and chunk_size & (chunk_size - 1) == 0
    a = GemmArgs(a=m1.data_ptr(), b=w.data_ptr(), d=out.data_ptr(), lda=m1.stride(0), ldb=w.stride(0), ldd=out.stride(0),
                 M=m1.shape[0], N=w.shape[0], K=m1.shape[1], kind=QLIN_DT_I8, chunk_k=(max(chunk_size, 32) if pow2 else 32),
                 trun_bits=chunk_trun_bits, max_acc_bits=max_acc_bits, trunc_then_acc=int(truncate_then_accumulate),
                 out_dtype=QLIN_DT_I32)  # fmt: skip
    with torch.cuda.device(m1.device):
        rc = _lib.qlin_gemm(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(_lib.qlin_last_error_string().decode())
    return out
