"""Out-of-bounds writes, looked for with guard bands and poison.

Every output of a kernel is carved out of a larger buffer filled with a poison byte, with at least 4 KB of poison in
front of it and behind it.  After the kernel has run on a ragged shape (rows and columns that are no multiples of the
tile, K tails, a single row, sub-views with a pitch larger than the row), the guard bands and the pitch padding must
still hold the poison, and the output itself must hold none where the expected result holds none.  This stands in for a
memory checker: it sees stray stores, not stray loads.
"""

import pytest
import torch

from fms_model_optimizer_b200 import _lib as L
from fms_model_optimizer_b200 import ops

pytestmark = pytest.mark.gpu

GUARD = 4096
POISON = 0x5B


class Guarded:
    """A [rows, cols] tensor of `dtype` with row pitch `pitch` elements inside a poisoned byte buffer."""

    def __init__(self, rows, cols, dtype, dev, pitch=None):
        es = torch.empty((), dtype=dtype).element_size()
        self.pitch = pitch or cols
        self.rows, self.cols, self.es = rows, cols, es
        body = rows * self.pitch * es
        self.raw = torch.full((GUARD + body + GUARD,), POISON, dtype=torch.uint8, device=dev)
        self.t = self.raw[GUARD : GUARD + body].view(dtype).view(rows, self.pitch)[:, :cols]

    def check(self, what):
        assert bool((self.raw[:GUARD] == POISON).all()), f"{what}: wrote in front of the buffer"
        assert bool((self.raw[GUARD + self.rows * self.pitch * self.es :] == POISON).all()), f"{what}: wrote behind the buffer"
        if self.pitch > self.cols:
            pad = self.raw[GUARD : GUARD + self.rows * self.pitch * self.es].view(self.rows, self.pitch * self.es)[:, self.cols * self.es :]
            assert bool((pad == POISON).all()), f"{what}: wrote into the pitch padding"


@pytest.mark.parametrize("M,N,K", [(1, 40, 96), (1, 14336 // 8, 512), (100, 300, 1000), (128, 32, 160), (129, 257, 200), (300, 520, 384), (520, 130, 4100)])
@pytest.mark.parametrize("mode", ["raw", "bf16", "chunked"])
def test_gemm_stays_inside_its_output(cuda_dev, M, N, K, mode):
    g = torch.Generator().manual_seed(M * 7 + N)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    acc = (a.double() @ b.double().t()).to(torch.int32)
    ad, bd = a.to(cuda_dev), b.to(cuda_dev)
    pitch = (N + 15) // 8 * 8  # a 16-byte multiple for 2- and 4-byte outputs, wider than the row
    if mode == "raw":
        out = Guarded(M, N, torch.int32, cuda_dev, pitch)
        ops.gemm(ad, bd, out=out.t)
        want = acc
    elif mode == "chunked":
        out = Guarded(M, N, torch.int32, cuda_dev, pitch)
        ops.gemm(ad, bd, out=out.t, chunk_k=64, trun_bits=4)
        want = None
    else:
        out = Guarded(M, N, torch.bfloat16, cuda_dev, pitch)
        rs = torch.full((M,), 2.0**-10, device=cuda_dev)
        ops.gemm(ad, bd, out=out.t, epilogue=L.EPI_SCALE_SEQ, row_scale=rs, out_dtype=torch.bfloat16)
        want = (acc.float() * 2.0**-10).bfloat16()
    torch.cuda.synchronize()
    ops.check_status(cuda_dev)
    out.check(f"gemm {mode} {M}x{N}x{K}")
    if want is not None:
        assert torch.equal(out.t.cpu(), want)


@pytest.mark.parametrize("rows,cols", [(1, 16), (3, 100), (37, 4096), (130, 1000), (5, 40000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_quantiser_stays_inside_its_outputs(cuda_dev, rows, cols, dtype):
    lib = L.load()
    import ctypes as C

    x = torch.randn(rows, cols, device=cuda_dev).to(dtype)
    codes = Guarded(rows, cols, torch.int8, cuda_dev, (cols + 31) // 16 * 16)
    scale = Guarded(1, rows, torch.float32, cuda_dev)
    dq = Guarded(rows, cols, dtype, cuda_dev, (cols + 15) // 8 * 8)
    dt = {torch.float32: L.DT_F32, torch.bfloat16: L.DT_BF16}[dtype]
    args = L.QuantArgs(x=x.data_ptr(), codes=codes.t.data_ptr(), scale_out=scale.t.data_ptr(), dq_out=dq.t.data_ptr(), ldx=cols,
                       ldq=codes.pitch, lddq=dq.pitch, rows=rows, cols=cols, x_dtype=dt, mode=L.Q_I8_DYN, native_chain=(0 if dtype == torch.float32 else 3),
                       qmax_levels=127, dyn_eps=1e-5)  # fmt: skip
    L.check(lib.qlin_act_quant(C.byref(args), C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)), "qlin_act_quant")
    torch.cuda.synchronize()
    for g_, name in ((codes, "codes"), (scale, "scales"), (dq, "dq")):
        g_.check(f"act_quant {name} {rows}x{cols} {dtype}")
    want_codes, want_scale, _ = ops.act_quant(x, mode=L.Q_I8_DYN, native_chain=(0 if dtype == torch.float32 else 3))
    assert torch.equal(codes.t, want_codes) and torch.equal(scale.t.reshape(-1), want_scale)


@pytest.mark.parametrize("numel", [1, 17, 4099, 1 << 20])
def test_pact_kernels_stay_inside_their_outputs(cuda_dev, numel):
    import ctypes as C

    lib = L.load()
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    x = torch.randn(numel, device=cuda_dev) * 3
    gq = torch.randn(numel, device=cuda_dev)
    cv, cvn = torch.tensor([2.0], device=cuda_dev), torch.tensor([-1.5], device=cuda_dev)
    out = Guarded(1, numel, torch.float32, cuda_dev)
    grads = Guarded(1, 2, torch.float32, cuda_dev)
    ws = Guarded(1, max(2, lib.qlin_pact2_bwd_workspace_bytes(numel) // 4), torch.float32, cuda_dev)
    a = L.Pact2Args(x=x.data_ptr(), grad_out=gq.data_ptr(), out=out.t.data_ptr(), clip_val=cv.data_ptr(), clip_valn=cvn.data_ptr(),
                    grad_clip=grads.t.data_ptr(), workspace=ws.t.data_ptr(), numel=numel, dtype=L.DT_F32, num_bits=8, align_zero=1)  # fmt: skip
    L.check(lib.qlin_pact2_fwd(C.byref(a), stream), "fwd")
    torch.cuda.synchronize()
    out.check("pact2_fwd")
    L.check(lib.qlin_pact2_bwd(C.byref(a), stream), "bwd")
    torch.cuda.synchronize()
    for g_, name in ((out, "grad_x"), (grads, "grad_clip"), (ws, "workspace")):
        g_.check(f"pact2_bwd {name} {numel}")
    assert torch.isfinite(grads.t).all()


def test_block_quantiser_stays_inside_its_outputs(cuda_dev):
    rows, cols = 37, 4096
    x = torch.randn(rows, cols, device=cuda_dev).bfloat16()
    r = torch.randn(rows, cols, device=cuda_dev).bfloat16()
    nw = torch.ones(cols, device=cuda_dev, dtype=torch.bfloat16)
    arena = Guarded(1, 3 * rows * cols + 3 * 4 * rows + 1024, torch.uint8, cuda_dev)
    base = arena.t.data_ptr()
    codes_off = [o * rows * cols for o in range(3)]
    scale_off = [(3 * rows * cols + 255) // 256 * 256 + o * 4 * rows for o in range(3)]
    rc = [ops.smooth_reciprocal((torch.rand(cols, device=cuda_dev) + 0.5).bfloat16().float()) for _ in range(3)]
    ops.block_quant(x, prologue=L.BLOCK_NORM, r=r, norm_w=nw, smooth_rcps=rc, store_sum=True, dst=([base], codes_off, scale_off, 0))
    torch.cuda.synchronize()
    arena.check("block_quant replicated outputs")
    want_c, want_s, _, _ = ops.block_quant(x, prologue=L.BLOCK_NORM, r=r, norm_w=nw, smooth_rcps=rc, store_sum=True)
    for o in range(3):
        got = arena.t.reshape(-1)[codes_off[o] : codes_off[o] + rows * cols].view(torch.int8).view(rows, cols)
        assert torch.equal(got, want_c[o])
        gs = arena.t.reshape(-1)[scale_off[o] : scale_off[o] + 4 * rows].view(torch.float32)
        assert torch.equal(gs, want_s[o])
