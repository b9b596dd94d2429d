"""qlin_pact2_bwd_noalloc against qlin_pact2_bwd, through the C ABI.

Some hosts of the library cannot lend it scratch memory (a sealed device pool, a hook that only gets
its input and output buffers, a loop that must not call cudaMalloc).  For them the PACT+ backward has
a twin that keeps its partial sums in an array inside the library image.  This file checks that the
twin returns exactly what the workspace version returns, on two calls in a row (the array is shared
and keeps the previous call's contents), and that it refuses sizes beyond its stated limit.  It is
named to be collected last, so a run that stops at the first failure has already run everything else.
"""

import ctypes as C

import pytest
import torch

from fms_model_optimizer_b200 import _lib as L

pytestmark = pytest.mark.gpu


def _args(x, g, out, cv, cvn, grads, ws, nbits, variant=L.PACT_TWO_SIDED, numel=None):
    dt = {torch.float32: L.DT_F32, torch.float16: L.DT_F16, torch.bfloat16: L.DT_BF16}[x.dtype]
    return L.Pact2Args(x=x.data_ptr(), grad_out=g.data_ptr(), out=out.data_ptr(), clip_val=cv.data_ptr(),
                       clip_valn=(cvn.data_ptr() if cvn is not None else None), grad_clip=grads.data_ptr(),
                       workspace=(ws.data_ptr() if ws is not None else None),
                       numel=(x.numel() if numel is None else numel), dtype=dt, num_bits=nbits, align_zero=1, variant=variant)


def test_noalloc_backward_equals_workspace_backward_twice(cuda_dev):
    lib = L.load()
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    cv = torch.tensor([2.5], device=cuda_dev)
    cvn = torch.tensor([-2.0], device=cuda_dev)
    # two calls in a row with different sizes and dtypes: the second one finds the first one's
    # partial sums in the shared array and must not be affected by them
    for seed, shape, dtype, nbits in ((0, (3000, 1024), torch.float32, 8), (1, (77, 130), torch.bfloat16, 4)):
        gen = torch.Generator(device=cuda_dev).manual_seed(seed)
        x = (torch.randn(shape, generator=gen, device=cuda_dev) * 3).to(dtype)
        g = torch.randn(shape, generator=gen, device=cuda_dev).to(dtype)
        ws = torch.empty(lib.qlin_pact2_bwd_workspace_bytes(x.numel()) // 4, dtype=torch.float32, device=cuda_dev)
        gx_ref, gc_ref = torch.empty_like(x), torch.empty(2, device=cuda_dev)
        gx_new, gc_new = torch.empty_like(x), torch.full((2,), float("nan"), device=cuda_dev)
        a_ref = _args(x, g, gx_ref, cv, cvn, gc_ref, ws, nbits)
        a_new = _args(x, g, gx_new, cv, cvn, gc_new, None, nbits)
        L.check(lib.qlin_pact2_bwd(C.byref(a_ref), stream), "qlin_pact2_bwd")
        L.check(lib.qlin_pact2_bwd_noalloc(C.byref(a_new), stream), "qlin_pact2_bwd_noalloc")
        torch.cuda.synchronize()
        assert torch.equal(gx_new, gx_ref)
        assert torch.equal(gc_new, gc_ref), (gc_new, gc_ref)
        assert torch.isfinite(gc_new).all()


def test_noalloc_rejects_sizes_beyond_its_limit(cuda_dev):
    lib = L.load()
    limit = lib.qlin_pact2_bwd_noalloc_max_numel()
    assert limit == 1 << 31
    t = torch.zeros(16, device=cuda_dev)
    a = _args(t, t, t, t, t, t, None, 8)
    a.numel = limit + 1
    assert lib.qlin_pact2_bwd_noalloc(C.byref(a), None) == L.ERR_TOO_LARGE
    assert b"limit" in lib.qlin_last_error_string()
    a.numel = 16
    a.grad_clip = None
    assert lib.qlin_pact2_bwd_noalloc(C.byref(a), None) == L.ERR_NULL


@pytest.mark.parametrize("variant", [L.PACT_ONE_SIDED, L.PACT_SYMMETRIC])
def test_noalloc_one_sided_and_symmetric_variants(cuda_dev, variant):
    """The members of the family that have no lower clip value (clip_valn is NULL), on a view that starts one element
    into its buffer (no 16-byte alignment: the scalar head and tail paths), and then on an empty tensor, where only the
    finishing kernel runs and must write zeros."""
    lib = L.load()
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    cv = torch.tensor([1.75], device=cuda_dev)
    gen = torch.Generator(device=cuda_dev).manual_seed(5 + variant)
    for numel in (40003, 0):
        # buffers of numel + 2 elements viewed from their second element; the element count goes in explicitly, so
        # the empty case still hands the library valid (non-NULL) pointers
        x = (torch.randn(numel + 2, generator=gen, device=cuda_dev) * 2)[1:]
        g = torch.randn(numel + 2, generator=gen, device=cuda_dev)[1:]
        ws = torch.empty(max(2, lib.qlin_pact2_bwd_workspace_bytes(numel) // 4), dtype=torch.float32, device=cuda_dev)
        gx_ref, gc_ref = torch.zeros(numel + 2, device=cuda_dev)[1:], torch.full((2,), float("nan"), device=cuda_dev)
        gx_new, gc_new = torch.zeros(numel + 2, device=cuda_dev)[1:], torch.full((2,), float("nan"), device=cuda_dev)
        L.check(lib.qlin_pact2_bwd(C.byref(_args(x, g, gx_ref, cv, None, gc_ref, ws, 8, variant, numel)), stream), "qlin_pact2_bwd")
        L.check(lib.qlin_pact2_bwd_noalloc(C.byref(_args(x, g, gx_new, cv, None, gc_new, None, 8, variant, numel)), stream), "noalloc")
        torch.cuda.synchronize()
        assert torch.equal(gx_new[:numel], gx_ref[:numel])
        assert torch.equal(gc_new, gc_ref), (gc_new, gc_ref)
        if numel == 0:
            assert gc_new.tolist() == [0.0, 0.0]


def test_noalloc_rejects_what_the_workspace_version_rejects(cuda_dev):
    lib = L.load()
    t = torch.zeros(16, device=cuda_dev)
    ws = torch.zeros(64, device=cuda_dev)
    for bad_variant in (-1, 3):
        assert lib.qlin_pact2_bwd(C.byref(_args(t, t, t, t, t, t, ws, 8, bad_variant)), None) == L.ERR_UNSUPPORTED
        assert lib.qlin_pact2_bwd_noalloc(C.byref(_args(t, t, t, t, t, t, None, 8, bad_variant)), None) == L.ERR_UNSUPPORTED
    assert lib.qlin_pact2_bwd_noalloc(C.byref(_args(t, t, t, t, None, t, None, 8, L.PACT_TWO_SIDED)), None) == L.ERR_NULL
