"""The ctypes stub that INTEGRATION.md gives to a maintainer of the reference, run as it stands: its struct mirrors the
header, and its ``b200_imatmul`` honours the ``mm_func`` contract of fms_mo/custom_ext_kernels/utils.py:706-714, bit for
bit against the oracle, including the chunk-truncation keywords and the reference's own way of calling it (a ``.t()`` view)."""

import ctypes as C

import pytest
import torch

from fms_model_optimizer_b200 import _lib as L
from oracle import gemm as OG


def test_stub_struct_is_the_library_struct():
    from fms_model_optimizer_b200 import integration_stub as S

    assert C.sizeof(S.GemmArgs) == C.sizeof(L.GemmArgs)
    assert [(n, getattr(S.GemmArgs, n).offset) for n, _ in S.GemmArgs._fields_] == [(n, getattr(L.GemmArgs, n).offset) for n, _ in L.GemmArgs._fields_]


@pytest.mark.gpu
def test_stub_imatmul_matches_oracle(cuda_dev):
    from fms_model_optimizer_b200 import integration_stub as S

    g = torch.Generator().manual_seed(31)
    x = torch.randint(-127, 128, (70, 320), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (90, 320), generator=g, dtype=torch.int8)
    xd, wd = x.to(cuda_dev), w.to(cuda_dev)
    assert torch.equal(S.b200_imatmul(xd, wd.t()).cpu(), OG.imatmul_chunk_truncate(x, w.t().contiguous()))
    for kw in (dict(chunk_trun_bits=8, chunk_size=64), dict(chunk_trun_bits=4, chunk_size=32, max_acc_bits=20),
               dict(chunk_trun_bits=8, chunk_size=100), dict(chunk_trun_bits=6, chunk_size=64, truncate_then_accumulate=False)):
        assert torch.equal(S.b200_imatmul(xd, wd.t(), **kw).cpu(), OG.imatmul_chunk_truncate(x, w.t().contiguous(), **kw)), kw
    with pytest.raises(RuntimeError, match="aligned|16"):
        S.b200_imatmul(xd[:, 1:], wd.t()[1:, :])
