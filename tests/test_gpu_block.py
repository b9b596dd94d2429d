"""GPU parity of the fused decoder-block kernels: the quantise step against the oracle on the row the
kernel itself reports (bit-exact), the prologues against PyTorch (to the last bf16 place)."""

import pytest
import torch
import torch.nn.functional as F

from fms_model_optimizer_b200 import _lib as L
from fms_model_optimizer_b200 import ops
from oracle import quantizers as OQ

pytestmark = pytest.mark.gpu


def _smooth(K, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(K, generator=g) * 4 + 0.25).bfloat16()


def _ulp_close(a, b, ulps=1):
    a, b = a.float(), b.float()
    tol = torch.maximum(a.abs(), b.abs()) * (2.0**-8) * ulps + 1e-30
    return bool(((a - b).abs() <= tol).all())


@pytest.mark.parametrize("T,K", [(37, 4096), (19, 512), (9, 7168), (5, 14336), (3, 48)])
def test_plain_prologue_three_outputs_bit_exact(cuda_dev, T, K):
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, K, generator=g)
    x[:, :: max(1, K // 50)] *= 20
    x[1] = 0
    x = x.bfloat16()
    sms = [_smooth(K, 1), None, _smooth(K, 3)]
    rcps = [None if s is None else ops.smooth_reciprocal(s.float().to(cuda_dev)) for s in sms]
    codes, scales, _, _ = ops.block_quant(x.to(cuda_dev), smooth_rcps=rcps)
    for c, s, sm in zip(codes, scales, sms):
        want_c, want_s = OQ.qa_dynamic_max_qfunc(x if sm is None else x / sm)
        assert torch.equal(c.cpu(), want_c)
        assert torch.equal(s.cpu(), want_s.float().reshape(-1))


def test_norm_prologue_with_residual(cuda_dev):
    T, K = 41, 4096
    g = torch.Generator().manual_seed(0)
    x, r = (torch.randn(T, K, generator=g) * 2).bfloat16(), torch.randn(T, K, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(K, generator=g)).bfloat16()
    sms = [_smooth(K, 5), _smooth(K, 6)]
    rcps = [ops.smooth_reciprocal(s.float().to(cuda_dev)) for s in sms]
    codes, scales, xo, h = ops.block_quant(x.to(cuda_dev), prologue=L.BLOCK_NORM, r=r.to(cuda_dev), norm_w=w.to(cuda_dev),
                                           smooth_rcps=rcps, store_sum=True, want_h=True)
    assert torch.equal(xo.cpu(), x + r)
    ref = F.rms_norm((x + r).float(), (K,), w.float(), 1e-5)
    assert _ulp_close(h.cpu(), ref.bfloat16())
    for c, s, sm in zip(codes, scales, sms):
        want_c, want_s = OQ.qa_dynamic_max_qfunc(h.cpu() / sm)
        assert torch.equal(c.cpu(), want_c) and torch.equal(s.cpu(), want_s.float().reshape(-1))
    # without a residual the stream is normalised as it is
    codes2, _, xo2, h2 = ops.block_quant(xo, prologue=L.BLOCK_NORM, norm_w=w.to(cuda_dev), smooth_rcps=rcps, want_h=True)
    assert xo2 is None and torch.equal(h2, h) and all(torch.equal(a, b) for a, b in zip(codes, codes2))


def test_silu_mul_prologue_and_two_pass_given_scale(cuda_dev):
    T, K = 23, 7168
    g = torch.Generator().manual_seed(2)
    gate, up = (torch.randn(T, K, generator=g) * 2).bfloat16(), torch.randn(T, K, generator=g).bfloat16()
    sm = _smooth(K, 7)
    rcp = ops.smooth_reciprocal(sm.float().to(cuda_dev))
    codes, scales, _, h = ops.block_quant(gate.to(cuda_dev), prologue=L.BLOCK_SILU_MUL, r=up.to(cuda_dev), smooth_rcps=[rcp], want_h=True)
    ref = (F.silu(gate.float()).bfloat16() * up)
    assert _ulp_close(h.cpu(), ref)
    want_c, want_s = OQ.qa_dynamic_max_qfunc(h.cpu() / sm)
    assert torch.equal(codes[0].cpu(), want_c) and torch.equal(scales[0].cpu(), want_s.float().reshape(-1))
    # first pass of a row-parallel shard: scales only; second pass with the (larger) reduced scale
    _, s_only, _, _ = ops.block_quant(gate.to(cuda_dev), prologue=L.BLOCK_SILU_MUL, r=up.to(cuda_dev), smooth_rcps=[rcp], mode=L.BLOCK_SCALE_ONLY)
    assert torch.equal(s_only[0], scales[0])
    bigger = (scales[0] * 1.5).bfloat16().float()
    c2, s2, _, _ = ops.block_quant(gate.to(cuda_dev), prologue=L.BLOCK_SILU_MUL, r=up.to(cuda_dev), smooth_rcps=[rcp],
                                   mode=L.BLOCK_GIVEN_SCALE, scale_in=bigger)
    want = torch.round((h.cpu() / sm) / bigger.cpu().bfloat16()[:, None]).to(torch.int8)
    assert torch.equal(c2[0].cpu(), want) and s2[0] is bigger


def test_rope_matches_fp32_formula(cuda_dev):
    B, S, H, D = 2, 96, 3, 128
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B * S, H, D, generator=g).bfloat16()
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(torch.arange(S).float(), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    got = ops.rope_(x.clone().to(cuda_dev), cos.to(cuda_dev), sin.to(cuda_dev), S).cpu()
    xf = x.float().view(B, S, H, D)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    x1, x2 = xf[..., : D // 2], xf[..., D // 2 :]
    want = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).view(B * S, H, D)
    # one bf16 rounding of a sum whose terms may cancel: bound the error by the size of the terms
    mag = torch.cat([(x1 * c).abs() + (x2 * s).abs(), (x2 * c).abs() + (x1 * s).abs()], -1).view(B * S, H, D)
    assert ((got.float() - want).abs() <= mag * 2.0**-8 + 1e-30).all()


def test_gemm_row_block_scatter_to_local_buffers(cuda_dev):
    """The scatter epilogue with all destinations on this GPU: row block i of the output lands in buffer i at the
    requested row offset, bit-identical to the plain launch."""
    g = torch.Generator().manual_seed(11)
    M, K, N, rows = 512, 256, 384, 128
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(cuda_dev)
    b = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(cuda_dev)
    rs = (torch.rand(M, generator=g) * 0.01).to(cuda_dev)
    cs = (torch.rand(N, generator=g) * 0.01).to(cuda_dev)
    kw = dict(epilogue=L.EPI_SCALE_PROD, row_scale=rs, col_scale=cs, scale_round=torch.float16, acc_round=torch.float16,
              out_dtype=torch.bfloat16)
    want = ops.gemm(a, b, **kw)
    bufs = [torch.zeros(3 * rows, N, dtype=torch.bfloat16, device=cuda_dev) for _ in range(M // rows)]
    ops.gemm(a, b, scatter=([t.data_ptr() for t in bufs], rows, rows), **kw)
    for i, t in enumerate(bufs):
        assert torch.equal(t[rows : 2 * rows], want[i * rows : (i + 1) * rows])
        assert not t[:rows].any() and not t[2 * rows :].any()
    raw = ops.gemm(a, b)
    bufs = [torch.zeros(rows, N, dtype=torch.int32, device=cuda_dev) for _ in range(M // rows)]
    ops.gemm(a, b, scatter=([t.data_ptr() for t in bufs], rows, 0))
    assert torch.equal(torch.cat(bufs), raw)
    assert torch.equal(raw.cpu(), (a.cpu().double() @ b.cpu().double().t()).to(torch.int32))


def test_block_quant_partial_sums_and_replicated_outputs(cuda_dev):
    T, K, parts, ndst = 24, 1024, 4, 3
    g = torch.Generator().manual_seed(12)
    x = torch.randn(T, K, generator=g).bfloat16()
    part = torch.randn(parts, T, K, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(K, generator=g)).bfloat16()
    sms = [_smooth(K, 8), _smooth(K, 9)]
    rcps = [ops.smooth_reciprocal(s.float().to(cuda_dev)) for s in sms]
    part_d = part.to(cuda_dev)
    # destinations: byte buffers holding [codes0 | codes1 | scales0 | scales1] for 2 * T rows; these rows go to row T..2T
    R = 2 * T
    offs_c = [0, R * K]
    offs_s = [2 * R * K, 2 * R * K + 4 * R]
    dsts = [torch.zeros(2 * R * K + 8 * R, dtype=torch.uint8, device=cuda_dev) for _ in range(ndst)]
    xin = x.to(cuda_dev).clone()
    _, _, xo, h = ops.block_quant(xin, prologue=L.BLOCK_NORM, r=part_d[0], r_parts=parts, r_part_stride=T * K, norm_w=w.to(cuda_dev),
                                  smooth_rcps=rcps, sum_into=xin, want_h=True, dst=([d.data_ptr() for d in dsts], offs_c, offs_s, T))
    red = part.float().sum(0)  # four addends: the fp32 sum is exact enough to be order independent here? no -- emulate the order
    acc = part[0].float()
    for s in range(1, parts):
        acc = acc + part[s].float()
    want_x = x + acc.bfloat16()
    assert xo is xin and torch.equal(xin.cpu(), want_x)
    assert _ulp_close(h.cpu(), F.rms_norm(want_x.float(), (K,), w.float(), 1e-5).bfloat16())
    del red
    for d in dsts:
        for o, sm in enumerate(sms):
            want_c, want_s = OQ.qa_dynamic_max_qfunc(h.cpu() / sm)
            codes = d[offs_c[o] : offs_c[o] + R * K].view(torch.int8).view(R, K)
            scales = d[offs_s[o] : offs_s[o] + 4 * R].view(torch.float32)
            assert torch.equal(codes[T:].cpu(), want_c) and not codes[:T].any()
            assert torch.equal(scales[T:].cpu(), want_s.float().reshape(-1)) and not scales[:T].any()


@pytest.mark.parametrize("T,K", [(700, 512), (300, 1024), (260, 1792), (130, 2064), (90, 7168), (40, 9000 // 16 * 16)])
def test_block_size_follows_the_row_length(cuda_dev, T, K):
    """Rows of a few hundred to a few thousand elements (the shards of a row-parallel Linear's input) run with blocks of
    32 to 1024 threads; every size class against the oracle, with enough rows for the persistent loop and the shared
    reciprocal vectors."""
    g = torch.Generator().manual_seed(T + K)
    x = (torch.randn(T, K, generator=g) * 2).bfloat16()
    r = torch.randn(T, K, generator=g).bfloat16()
    sm = _smooth(K, 11)
    rcp = ops.smooth_reciprocal(sm.float().to(cuda_dev))
    codes, scales, _, h = ops.block_quant(x.to(cuda_dev), prologue=L.BLOCK_SILU_MUL, r=r.to(cuda_dev), smooth_rcps=[rcp], want_h=True)
    ref = (F.silu(x.float()).bfloat16() * r)
    assert _ulp_close(h.cpu(), ref, ulps=2)
    want_c, want_s = OQ.qa_dynamic_max_qfunc(h.cpu() / sm)
    assert torch.equal(codes[0].cpu(), want_c) and torch.equal(scales[0].cpu(), want_s.float().reshape(-1))
    codes, scales, _, _ = ops.block_quant(x.to(cuda_dev), smooth_rcps=[rcp, None])
    for c, s, m in zip(codes, scales, (sm, None)):
        want_c, want_s = OQ.qa_dynamic_max_qfunc(x if m is None else x / m)
        assert torch.equal(c.cpu(), want_c) and torch.equal(s.cpu(), want_s.float().reshape(-1))
    ops.check_status(cuda_dev)
