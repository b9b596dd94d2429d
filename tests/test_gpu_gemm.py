"""GPU parity of the tcgen05 GEMMs against the CPU oracle, through the C ABI.  Integer results are
compared bit for bit; fp8 results within 1e-5 relative (fp32 accumulation order differs)."""

import pytest
import torch

from fms_model_optimizer_b200 import _lib as L
from fms_model_optimizer_b200 import ops
from oracle import gemm as OG

pytestmark = pytest.mark.gpu


def _i8(shape, seed, lo=-127, hi=128):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, shape, dtype=torch.int8, generator=g)


@pytest.mark.parametrize(
    "M,N,K",
    [(1, 16, 32), (128, 256, 128), (100, 200, 96), (129, 257, 144), (300, 700, 4096), (256, 512, 1024), (5, 3, 16),
     (257, 129, 33), (64, 2048, 272), (1024, 1024, 1024)],
)
def test_int8_gemm_bit_exact(cuda_dev, M, N, K):
    a, b = _i8((M, K), 1), _i8((N, K), 2, -128, 128)
    want = OG.imatmul_chunk_truncate(a, b.t().contiguous(), chunk_size=32)
    got = ops.imatmul(a.to(cuda_dev), b.to(cuda_dev).t())
    ops.check_status(cuda_dev)
    assert got.dtype == torch.int32 and torch.equal(got.cpu(), want)


@pytest.mark.parametrize(
    "M,N,K,chunk,t,accb,tta",
    [(128, 128, 128, 64, 8, 32, True), (100, 70, 320, 64, 8, 32, True), (256, 384, 1024, 32, 4, 32, True),
     (256, 256, 1024, 128, 8, 32, True), (256, 256, 1024, 256, 8, 32, True), (256, 256, 1024, 64, 8, 18, True),
     (256, 256, 1024, 64, 8, 32, False), (130, 250, 1000, 64, 8, 24, False), (64, 64, 96, 64, 1, 32, True),
     (64, 64, 512, 16, 8, 32, True), (64, 64, 512, 100, 8, 32, True), (33, 65, 2048, 64, 12, 32, True)],
)
def test_int8_chunk_truncate_bit_exact(cuda_dev, M, N, K, chunk, t, accb, tta):
    a, b = _i8((M, K), 3), _i8((K, N), 4)
    want = OG.imatmul_chunk_truncate(a, b, chunk_trun_bits=t, chunk_size=chunk, max_acc_bits=accb, truncate_then_accumulate=tta)
    got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev), chunk_trun_bits=t, chunk_size=chunk,
                                       max_acc_bits=accb, truncate_then_accumulate=tta)
    ops.check_status(cuda_dev)
    assert torch.equal(got.cpu(), want)


def test_chunk_size_8_and_initial_accumulator(cuda_dev):
    a, b = _i8((96, 256), 5), _i8((256, 80), 6)
    c = torch.randint(-1000, 1000, (96, 80), dtype=torch.int32, generator=torch.Generator().manual_seed(7))
    want = OG.imatmul_chunk_truncate(a, b, c=c, chunk_trun_bits=4, chunk_size=8)
    got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev), c=c.to(cuda_dev), chunk_trun_bits=4, chunk_size=8)
    assert torch.equal(got.cpu(), want)
    want = OG.imatmul_chunk_truncate(a, b, c=c, chunk_size=64)
    got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev), c=c.to(cuda_dev), chunk_size=64)
    assert torch.equal(got.cpu(), want)


def test_b_operand_given_as_kn_contiguous(cuda_dev):
    """tl_matmul accepts any strides for b; a [k,n]-contiguous b is transposed on the way in."""
    a, b = _i8((64, 128), 8), _i8((128, 48), 9)
    want = OG.imatmul_chunk_truncate(a, b, chunk_size=32)
    got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev).contiguous())
    assert torch.equal(got.cpu(), want)


def test_reference_test_properties_int8(cuda_dev):
    """The properties the reference's own GPU test states (tests/triton_kernels/test_triton_mm.py:85-123):
    randint(-128,127) operands, relative error vs the exact product < 1e-5 plain, < 1e-2 with 8-bit
    truncation or an 18-bit accumulator, and the error does not shrink when the chunk grows."""
    for mnk in (64, 256, 1024):
        a, b = _i8((mnk, mnk), 10, -128, 127), _i8((mnk, mnk), 11, -128, 127)
        exact = a.double() @ b.double()
        ad, bd = a.to(cuda_dev), b.to(cuda_dev)

        def rel(t):
            return (torch.norm(t.cpu().double() - exact) / torch.norm(exact)).item()

        assert rel(ops.tl_matmul_chunk_truncate(ad, bd)) < 1e-5
        e32 = rel(ops.tl_matmul_chunk_truncate(ad, bd, chunk_trun_bits=8, chunk_size=32))
        e128 = rel(ops.tl_matmul_chunk_truncate(ad, bd, chunk_trun_bits=8, chunk_size=128))
        assert e32 < 1e-2 and e128 < 1e-2
        assert rel(ops.tl_matmul_chunk_truncate(ad, bd, max_acc_bits=18, chunk_size=32)) < 1e-2


def test_config2_full_size_sampled_and_checksum(cuda_dev):
    """The chunk-truncated int8 GEMM at the full benchmark size (4096 x 8192 x 4096, chunk 64, 8 truncated bits, seed 1):
    (a) a random 48 x 40 sub-block of the output equals the oracle evaluated on those rows / columns
    (the truncation is elementwise per output, so a sub-block is exact parity);
    (b) for the untruncated product the checksum of checksums sum(D) == sum_k colsum(A)_k * colsum(B)_k."""
    torch.manual_seed(1)
    M, K, N = 4096, 8192, 4096
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8)
    b_nk = torch.randint(-127, 128, (N, K), dtype=torch.int8)
    ad, bd = a.to(cuda_dev), b_nk.to(cuda_dev)
    got = ops.tl_matmul_chunk_truncate(ad, bd.t(), chunk_trun_bits=8, chunk_size=64)
    rows = torch.randperm(M)[:48]
    cols = torch.randperm(N)[:40]
    want = OG.imatmul_chunk_truncate(a[rows], b_nk[cols].t().contiguous(), chunk_trun_bits=8, chunk_size=64)
    assert torch.equal(got.cpu()[rows][:, cols], want)
    plain = ops.imatmul(ad, bd.t())
    total = int(plain.to(torch.int64).sum().item())
    expect = int((a.to(torch.int64).sum(0) * b_nk.to(torch.int64).sum(0)).sum().item())
    assert total == expect
    ops.check_status(cuda_dev)


@pytest.mark.parametrize("M,N,K", [(1, 64, 128), (128, 256, 256), (100, 300, 1000), (512, 512, 4096)])
def test_fp8_gemm_matches_oracle(cuda_dev, M, N, K):
    g = torch.Generator().manual_seed(12)
    a = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    want = OG.fmatmul_chunk_truncate(a, b.t())
    got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev).t(), chunk_size=64).cpu()
    assert got.dtype == torch.float32
    assert torch.norm(got - want) / torch.norm(want) < 1e-5  # reference's own bound, test_triton_mm.py:80
    assert (got - want).abs().max() <= 1e-4 * max(1.0, want.abs().max().item())


def test_fp8_chunk_truncation_matches_oracle(cuda_dev):
    g = torch.Generator().manual_seed(13)
    a = torch.randn(96, 512, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(80, 512, generator=g).to(torch.float8_e4m3fn)
    for trun, dl16 in ((8, False), (16, False), (0, True)):
        want = OG.fmatmul_chunk_truncate(a, b.t(), chunk_trun_bits=trun, chunk_size=64, clamp_acc_to_dl16=dl16)
        got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev).t(), chunk_trun_bits=trun, chunk_size=64,
                                           clamp_acc_to_dl16=dl16).cpu()
        # per-chunk products of e4m3 values over 64 terms are exact in fp32, so the truncated chunk
        # terms agree bit for bit; only the final fp32 accumulation order may differ
        tol = 2.0 ** (-(23 - (14 if dl16 else trun)) + 2)
        assert torch.norm(got - want) / torch.norm(want) < tol
        assert torch.norm(got - want) / torch.norm(want) < 1e-3  # reference bound with truncation, test_triton_mm.py:82


def test_fp8_chunk_gemm_against_the_reference_triton_kernel(cuda_dev):
    """The CUDA kernel against outputs of the reference's own Triton matmul_kernel on the same seeded operands (golden
    triton_fp8_mm.pt, made on a B200 by tests/golden/make_triton_golden.py).  The tensor core sums a chunk's products in
    its own order, so a chunk sum can differ in its last fp32 place before the truncation; after truncating 8 or more
    mantissa bits almost every element is identical."""
    from conftest import load_golden

    for c in load_golden("triton_fp8_mm.pt")["cases"]:
        g = torch.Generator().manual_seed(c["seed"])
        a = torch.randn(c["M"], c["K"], generator=g).to(torch.float8_e4m3fn)
        b = torch.randn(c["N"], c["K"], generator=g).to(torch.float8_e4m3fn)
        cc = torch.randint(-1000, 1000, (c["M"], c["N"]), generator=g).to(torch.float32) if c["with_c"] else None
        kw = c["kw"]
        y = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev).t(), c=(cc.to(cuda_dev) if cc is not None else None),
                                         chunk_trun_bits=kw.get("chunk_trun_bits", 0), chunk_size=kw.get("chunk_size", 16),
                                         truncate_then_accumulate=kw.get("truncate_then_accumulate", True),
                                         clamp_acc_to_dl16=kw.get("clamp_acc_to_dl16", False)).cpu()  # fmt: skip
        got, ref = (y[:64, :64], c["block"]) if "block" in c else (y, c["y"])
        rel = (torch.norm(got - ref) / torch.norm(ref)).item()
        trun = 14 if kw.get("clamp_acc_to_dl16", False) else kw.get("chunk_trun_bits", 0)
        assert rel < max(1e-6, 2.0 ** (-(23 - trun))), (c["M"], kw, rel)
        if trun >= 8:
            assert (got == ref).float().mean() > 0.99, (c["M"], kw, (got == ref).float().mean().item())


def test_dequant_epilogue_modes(cuda_dev):
    """Scaled epilogues against the same arithmetic in eager CPU PyTorch."""
    a, b = _i8((70, 192), 14), _i8((90, 192), 15)
    g = torch.Generator().manual_seed(16)
    rs = (torch.rand(70, generator=g) * 0.05 + 1e-3).bfloat16().float()
    cs = torch.rand(90, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(90, generator=g).bfloat16().float() * 0.01
    acc = (a.double() @ b.double().t()).to(torch.int32)
    ad, bd = a.to(cuda_dev), b.to(cuda_dev)
    # deploy chain: (acc.float() * (rs * cs).to(fp16) + bias).to(fp16).to(bf16)
    want = (acc.float() * (rs[:, None] * cs[None, :]).to(torch.float16) + bias).to(torch.float16).to(torch.bfloat16)
    got = ops.gemm(ad, bd, epilogue=L.EPI_SCALE_PROD, row_scale=rs.to(cuda_dev), col_scale=cs.to(cuda_dev),
                   bias=bias.to(cuda_dev), scale_round=torch.float16, acc_round=torch.float16, out_dtype=torch.bfloat16)
    assert torch.equal(got.cpu(), want)
    # iaddmm chain: scale_i.float() * acc * scale_w + bias  (fp32)
    want = rs[:, None] * acc * cs[None, :] + bias
    got = torch.ops.qlin_b200.iaddmm(bias.to(cuda_dev), ad, bd.t(), rs.to(cuda_dev), cs.to(cuda_dev))
    assert torch.equal(got.cpu(), want)
    # fp16 output with scalar scales
    want = ((acc.float() * 0.013) * 0.5).to(torch.float16)
    got = ops.gemm(ad, bd, epilogue=L.EPI_SCALE_SEQ, row_scale=torch.tensor([0.013], device=cuda_dev),
                   col_scale=torch.tensor([0.5], device=cuda_dev), mid_round=torch.float16, out_dtype=torch.float16)
    assert torch.equal(got.cpu(), want)


def test_empty_and_error_cases(cuda_dev):
    a = torch.zeros(0, 64, dtype=torch.int8, device=cuda_dev)
    b = torch.zeros(32, 64, dtype=torch.int8, device=cuda_dev)
    assert ops.gemm(a, b).shape == (0, 32)
    with pytest.raises(RuntimeError):
        ops.gemm(b, torch.zeros(32, 48, dtype=torch.int8, device=cuda_dev))
    with pytest.raises(RuntimeError):
        ops.gemm(b, b.float())
    with pytest.raises(RuntimeError, match="status"):
        ops.gemm(b, b, chunk_k=48, trun_bits=8)


@pytest.mark.parametrize(
    "M,N,K",
    [(1, 14336, 4096), (1, 4096, 14336), (7, 1024, 2048), (16, 4096, 4096), (33, 200, 1000), (64, 128, 512), (96, 520, 4100),
     (100, 2048, 8192), (128, 4096, 4096), (128, 300, 160), (128, 14336, 640)],
)
def test_few_row_gemm_is_exact_and_deterministic(cuda_dev, M, N, K):
    """Problems of at most 128 rows run on the few-row kernel (weight rows as the MMA's M dimension, K split over a cluster
    whose partial sums are added in split order).  The shapes cover one to eight splits, ragged rows, columns and K tails.
    Integer results equal the exact product, raw and through a dequantising epilogue with an initial accumulator; the fp8
    result is the same bits on every run (fixed summation order) and within the fp8 bound of the oracle."""
    a, b = _i8((M, K), 21), _i8((N, K), 22, -128, 128)
    acc = (a.double() @ b.double().t()).to(torch.int32)
    ad, bd = a.to(cuda_dev), b.to(cuda_dev)
    got = ops.gemm(ad, bd)
    ops.check_status(cuda_dev)
    assert torch.equal(got.cpu(), acc)
    g = torch.Generator().manual_seed(23)
    c = torch.randint(-1000, 1000, (M, N), dtype=torch.int32, generator=g)
    got = ops.gemm(ad, bd, c=c.to(cuda_dev))
    assert torch.equal(got.cpu(), acc + c)
    rs = (torch.rand(M, generator=g) * 0.05 + 1e-3).bfloat16().float()
    cs = torch.rand(N, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(N, generator=g).bfloat16().float() * 0.01
    want = (acc.float() * (rs[:, None] * cs[None, :]).to(torch.float16) + bias).to(torch.float16).to(torch.bfloat16)
    got = ops.gemm(ad, bd, epilogue=L.EPI_SCALE_PROD, row_scale=rs.to(cuda_dev), col_scale=cs.to(cuda_dev),
                   bias=bias.to(cuda_dev), scale_round=torch.float16, acc_round=torch.float16, out_dtype=torch.bfloat16)  # fmt: skip
    assert torch.equal(got.cpu(), want)
    want = ((acc.float() * rs[:, None]) * cs[None, :]).bfloat16()
    got = ops.gemm(ad, bd, epilogue=L.EPI_SCALE_SEQ, row_scale=rs.to(cuda_dev), col_scale=cs.to(cuda_dev), out_dtype=torch.bfloat16)
    assert torch.equal(got.cpu(), want)
    want32 = (acc.float() * rs[:, None]) * cs[None, :] + bias
    got = ops.gemm(ad, bd, epilogue=L.EPI_SCALE_SEQ, row_scale=rs.to(cuda_dev), col_scale=cs.to(cuda_dev), bias=bias.to(cuda_dev),
                   out_dtype=torch.float32)  # fmt: skip
    assert torch.equal(got.cpu(), want32)

    fa = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    fb = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    fad, fbd = fa.to(cuda_dev), fb.to(cuda_dev)
    y1 = ops.gemm(fad, fbd)
    y2 = ops.gemm(fad, fbd)
    ops.check_status(cuda_dev)
    assert torch.equal(y1, y2)
    exact = fa.double() @ fb.double().t()
    assert (torch.norm(y1.cpu().double() - exact) / torch.norm(exact)).item() < 1e-5


@pytest.mark.parametrize("M,N,K,chunk", [(300, 260, 512, 64), (128, 128, 256, 32), (1000, 2100, 1024, 128), (64, 4096, 8192, 64)])
def test_low_byte_chunk_mode_is_bit_exact(cuda_dev, M, N, K, chunk):
    """Eight truncated bits with chunks of 32 / 64 / 128 that tile K run with the untruncated total on the tensor core and
    the chunks' low bytes summed on the ALU (sum of round-to-256 = total - sum of sign-extended low bytes).  Several tiles
    per CTA, ragged edges and an initial accumulator; the result is the oracle's, bit for bit."""
    a, b = _i8((M, K), 31), _i8((K, N), 32)
    c = torch.randint(-100000, 100000, (M, N), dtype=torch.int32, generator=torch.Generator().manual_seed(33))
    for cc in (None, c):
        want = OG.imatmul_chunk_truncate(a, b, c=cc, chunk_trun_bits=8, chunk_size=chunk)
        got = ops.tl_matmul_chunk_truncate(a.to(cuda_dev), b.to(cuda_dev), c=(cc.to(cuda_dev) if cc is not None else None),
                                           chunk_trun_bits=8, chunk_size=chunk)  # fmt: skip
        ops.check_status(cuda_dev)
        assert torch.equal(got.cpu(), want)
