"""GPU parity of the row quantise, weight fake-quant and PACT+ kernels against the oracle and the
golden outputs of the reference, through the C ABI."""

import pytest
import torch

from conftest import load_golden
from fms_model_optimizer_b200 import _lib as L
from fms_model_optimizer_b200 import ops
from fms_model_optimizer_b200.quant.quantizers import PACT, PACT2, SAWB, PACTplusSym, QMaxDynamic, Qmax, to_fp8
from oracle import quantizers as OQ

pytestmark = pytest.mark.gpu


def _x(M, K, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[: max(1, K // 100)]] *= 20
    if M > 3:
        x[1] = 0
        x[2] *= 1e-7
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(33, 80), (40, 4096), (7, 14336), (5, 33), (64, 768), (3, 40000), (1, 16)])
def test_per_token_int8_codes_bit_exact(cuda_dev, dtype, M, K):
    x = _x(M, K, dtype)
    g = torch.Generator().manual_seed(1)
    sm = (torch.rand(K, generator=g) * 4 + 0.25).to(dtype)
    for smooth in (None, sm):
        xs = x if smooth is None else x / smooth
        want_codes, want_scale = OQ.qa_dynamic_max_qfunc(xs)
        native = 0 if dtype == torch.float32 else 3
        codes, scale, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_I8_DYN, smooth=None if smooth is None else smooth.to(cuda_dev),
                                        native_chain=native)
        assert torch.equal(codes.cpu(), want_codes)
        assert torch.equal(scale.cpu(), want_scale.float().reshape(-1))


def test_fp32_chain_on_bf16_input(cuda_dev):
    """native_chain = 0: the canonical evaluation, formulas in fp32 on the widened input."""
    x = _x(48, 512, torch.bfloat16, 2)
    want_codes, want_scale = OQ.qa_dynamic_max_qfunc(x.float())
    codes, scale, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_I8_DYN, native_chain=0)
    assert torch.equal(codes.cpu(), want_codes) and torch.equal(scale.cpu(), want_scale.reshape(-1))
    assert codes.cpu().abs().max() <= 127


def test_qmax_dynamic_matches_reference_golden(cuda_dev):
    for c in load_golden("quantizers.pt")["qmax_dynamic"]:
        q = QMaxDynamic(8, dim=-1)
        y = q(c["x"].to(cuda_dev))
        assert torch.equal(y.cpu(), c["y"]), c["dtype"]


def test_static_activation_quantisers(cuda_dev):
    x = _x(37, 96, torch.float32, 3) * 0.3
    cv, cvn = torch.tensor(2.44), torch.tensor(-1.75)
    a_levels = 255
    in_scale = torch.tensor([(cv - cvn) / a_levels])
    zp = torch.round(-cvn / in_scale).to(torch.int)
    want = OQ.qa_raw_qfunc(x, in_scale, zp, False)
    codes, _, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_I8_STATIC, scale0=float(in_scale), zp0=float(zp), shift=128.0, add2=0.0)
    assert torch.equal(codes.cpu(), want)
    quant_scale = a_levels / torch.tensor([cv - cvn])
    step = 1.0 / quant_scale
    qzp = torch.round(cvn * quant_scale)
    want = OQ.qa_fmo_mo_qfunc(x, cv, cvn, step, qzp, False)
    codes, _, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_I8_STATIC_CLAMP_FIRST, scale0=float(step), zp0=float(qzp),
                                lo=float(cvn), hi=float(cv), shift=128.0)
    assert torch.equal(codes.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_fp8_dynamic_quant_bit_exact(cuda_dev, dtype):
    for M, K in ((24, 192), (9, 4096), (5, 40)):
        x = _x(M, K, dtype, 4)
        want_q, want_s = OQ.fp8_dyn_quant(x)
        native = 0 if dtype == torch.float32 else 3
        q, s, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_F8_DYN, native_chain=native)
        assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))
        assert torch.equal(s.cpu(), want_s.float().reshape(-1))
        want_q, _ = OQ.fp8_dyn_quant(x, dl8_flush=True)
        q, _, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_F8_DYN, native_chain=native, dl8_flush=True)
        assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))


def test_pact2_forward_backward_vs_reference_golden(cuda_dev):
    for c in load_golden("quantizers.pt")["pact2"]:
        q = PACT2(c["nbits"], init_clip_valn=c["cvn"], init_clip_val=c["cv"], dequantize=True, pact_plus=True, align_zero=True).to(cuda_dev)
        x = c["x"].to(cuda_dev).requires_grad_(True)
        y = q(x)
        assert torch.equal(y.detach().cpu(), c["y"]), (c["dtype"], c["nbits"], c["cv"])
        y.backward(c["g"].to(cuda_dev))
        assert torch.equal(x.grad.cpu(), c["gx"])
        # the two clip gradients are full-tensor sums; the kernel adds in a fixed tree order, the
        # reference in ATen's order: compare within the rounding of a 3552-term sum in that dtype
        eps = {torch.float32: 2e-5, torch.bfloat16: 2e-2, torch.float16: 4e-3}[c["dtype"]]
        for got, want in ((q.clip_val.grad, c["gcv"]), (q.clip_valn.grad, c["gcvn"])):
            scale = max(1.0, c["g"].float().abs().sum().item() * 0.05)
            assert abs(got.item() - want.float().item()) <= eps * scale, (c["dtype"], got.item(), want.item())


def test_pact_one_sided_and_symmetric_vs_reference_golden(cuda_dev):
    g = load_golden("extra.pt")
    eps = {torch.float32: 2e-5, torch.bfloat16: 2e-2, torch.float16: 4e-3}
    for kind in ("pact1", "pactsym"):
        for c in g[kind]:
            if kind == "pact1":
                q = PACT(c["nbits"], init_clip_val=c["cv"], dequantize=True, pact_plus=True).to(cuda_dev)
            else:
                q = PACTplusSym(c["nbits"], init_clip_val=c["cv"], dequantize=True, intg_zp=c["intg"]).to(cuda_dev)
            x = c["x"].to(cuda_dev).requires_grad_(True)
            y = q(x)
            assert torch.equal(y.detach().cpu(), c["y"]), (kind, c["dtype"], c["nbits"])
            y.backward(c["g"].to(cuda_dev))
            assert torch.equal(x.grad.cpu(), c["gx"])
            scale = max(1.0, c["g"].float().abs().sum().item() * 0.05)
            got, want = q.clip_val.grad.item(), c["gcv"].float().item()
            assert abs(got - want) <= eps[c["dtype"]] * scale, (kind, c["dtype"], got, want)


def test_pact2_backward_is_deterministic_and_matches_oracle_fp32(cuda_dev):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(300, 1000, generator=g) * 3)
    go = torch.randn(300, 1000, generator=g)
    cv, cvn = torch.tensor([2.5]), torch.tensor([-2.0])
    gx_o, ga_o, gan_o = OQ.pact2plus_bwd(x.double(), go.double(), cv.double(), cvn.double(), 8, True)
    gx, gc = ops.pact2_bwd(x.to(cuda_dev), go.to(cuda_dev), cv.to(cuda_dev), cvn.to(cuda_dev), 8, True)
    gx2, gc2 = ops.pact2_bwd(x.to(cuda_dev), go.to(cuda_dev), cv.to(cuda_dev), cvn.to(cuda_dev), 8, True)
    assert torch.equal(gc, gc2) and torch.equal(gx, gx2)
    gx_f, _, _ = OQ.pact2plus_bwd(x, go, cv, cvn, 8, True)
    assert torch.equal(gx.cpu(), gx_f)
    assert abs(gc[0].item() - ga_o.item()) < 1e-3 * max(1.0, abs(ga_o.item()))
    assert abs(gc[1].item() - gan_o.item()) < 1e-3 * max(1.0, abs(gan_o.item()))


def test_sawb_perch_vs_reference_golden(cuda_dev):
    for c in load_golden("quantizers.pt")["sawb_perch"]:
        q = SAWB(c["nbits"], dequantize=True, align_zero=True, perCh=48).to(cuda_dev)
        q.train()
        y = q(c["w"].to(cuda_dev))
        clip = q.clip_val.cpu()
        # the channel statistics are sums over 80 values: last-ulp differences in the clip value are
        # possible, elements then differ by at most one quantisation step
        # clip = c1 * mean|w| + c0 * rms(w) cancels about one decimal digit
        assert torch.allclose(clip.float(), c["clip"].float(), rtol=3e-5 if c["dtype"] == torch.float32 else 2e-2)
        step = (c["clip"].float() * 2 / (2 ** c["nbits"] - 2))[:, None]
        diff = (y.cpu().float() - c["y"].float()).abs()
        assert (diff <= step * 1.01 + 1e-7).all()
        lv = torch.round(y.cpu().float() / step) - torch.round(c["y"].float() / step)
        assert lv.abs().max() <= 1 and (lv != 0).float().mean() < (0.01 if c["dtype"] == torch.float32 else 0.1)
        # with the reference's clip values the quantise step is bit exact
        dq, codes, _ = ops.weight_fq_perch(c["w"].to(cuda_dev), num_bits=c["nbits"], mode=L.W_GIVEN, clip=c["clip"].float().to(cuda_dev),
                                           want_dq=True, want_codes=True)
        assert torch.equal(dq.cpu(), c["y"])
        _, codes, _ = ops.weight_fq_perch(c["w"].float().to(cuda_dev), num_bits=c["nbits"], mode=L.W_GIVEN,
                                          clip=c["clip_f32"].to(cuda_dev), want_dq=False, want_codes=True)
        assert torch.equal(codes.cpu(), c["codes"])
        # eval mode reuses the stored (fp32) clip buffer: the scale is then formed in fp32
        q.eval()
        q.clip_val.copy_(c["clip"].to(cuda_dev))
        want_eval = OQ.perch_fake_quant(c["w"], c["clip"], c["nbits"]).to(c["w"].dtype)
        assert torch.equal(q(c["w"].to(cuda_dev)).cpu(), want_eval)


def test_qmax_perch_vs_reference_golden(cuda_dev):
    for c in load_golden("quantizers.pt")["qmax_perch"]:
        q = Qmax(8, align_zero=True, perCh=48).to(cuda_dev)
        q.train()
        y = q(c["w"].to(cuda_dev))
        assert torch.equal(y.cpu(), c["y_train"])
        assert torch.equal(q.clip_val.cpu(), c["clip_after_train"])
        q.eval()
        assert torch.equal(q(c["w"].to(cuda_dev)).cpu(), c["y_eval"])


def test_ragged_and_unaligned_rows_take_the_scalar_path(cuda_dev):
    x = _x(9, 50, torch.float32, 6)
    base = torch.zeros(9 * 50 + 1, device=cuda_dev)
    xv = base[1:].view(9, 50)
    xv.copy_(x)
    want_codes, want_scale = OQ.qa_dynamic_max_qfunc(x)
    codes, scale, _ = ops.act_quant(xv, mode=L.Q_I8_DYN)
    assert torch.equal(codes.cpu(), want_codes) and torch.equal(scale.cpu(), want_scale.reshape(-1))


def _bits(t):
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32)


def test_per_tensor_sawb_vs_reference_golden(cuda_dev):
    for c in load_golden("extra.pt")["sawb_tensor"]:
        q = SAWB(c["nbits"], dequantize=True, align_zero=True, perCh=False).to(c["dtype"]).to(cuda_dev)
        q.train()
        w = c["w"].to(cuda_dev)
        y = q(w)
        # the clip value is c1 * mean|w| + c0 * rms(w) over 7200 values summed in a different order:
        # last-place differences are possible and cancel about one decimal digit
        rtol = {torch.float32: 3e-5, torch.bfloat16: 2e-2, torch.float16: 4e-3}[c["dtype"]]
        assert torch.allclose(q.clip_val.float().cpu(), c["clip"].float(), rtol=rtol), (c["dtype"], c["nbits"])
        step = c["clip"].float() * 2 / (2 ** c["nbits"] - 2)
        assert ((y.cpu().float() - c["y"].float()).abs() <= step * 1.01 + c["clip"].float().abs() * rtol).all()
        # with the reference's clip value every elementwise step is bit exact
        for x, key, deq in ((c["w"], "y", True), (c["w"] * 1.5, "y_eval", True), (c["w"], "codes", False)):
            out, _ = ops.tensor_fq(x.to(cuda_dev), kind=L.PT_INT_SYM, mode=L.W_GIVEN, num_bits=c["nbits"], clip=c["clip"].to(cuda_dev),
                                   align_zero=True, dequantize=deq)
            assert torch.equal(_bits(out.cpu()), _bits(c[key])), (c["dtype"], c["nbits"], key)
        q.eval()
        q.clip_val.copy_(c["clip"].to(cuda_dev))
        assert torch.equal(q(w * 1.5).cpu(), c["y_eval"])


def test_per_tensor_qmax_vs_reference_golden(cuda_dev):
    for c in load_golden("extra.pt")["qmax_tensor"]:
        q = Qmax(8, align_zero=c["align"], minmax=False).to(c["dtype"]).to(cuda_dev)
        q.train()
        w = c["w"].to(cuda_dev)
        assert torch.equal(q(w).cpu(), c["y1"]), (c["dtype"], c["align"])
        assert torch.equal(q(w * 0.5).cpu(), c["y2"])
        assert torch.equal(q.clip_val.cpu(), c["clip"])
        q.eval()
        assert torch.equal(q(w).cpu(), c["y_eval"])


def test_fp8_fake_quantisers_vs_reference_golden(cuda_dev):
    for c in load_golden("extra.pt")["fp8_fake"]:
        x = c["x"].to(cuda_dev)
        for mode, kw, scale in (("fp8_e4m3_scale_perToken", dict(perToken=True), 1), ("fp8_e4m3_scale_perCh", dict(perCh=37), 1),
                                ("fp8_e4m3_scale", {}, 1), ("fp8_e4m3_sat", {}, 300)):  # fmt: skip
            got = to_fp8(8, q_mode=mode, **kw).to(cuda_dev)(x * scale)
            assert got.dtype == c[mode].dtype and torch.equal(_bits(got.cpu()), _bits(c[mode])), (mode, c["dtype"])


def test_per_tensor_sawb_large_tensor_statistics(cuda_dev):
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(3072, 768, generator=g) * 0.03)
    want_clip = OQ.sawb_clip_pertensor(w.double(), 8).float()
    out, clip = ops.tensor_fq(w.to(cuda_dev), kind=L.PT_INT_SYM, mode=L.W_SAWB, num_bits=8, c0=31.76, c1=-35.04)
    assert torch.allclose(clip.cpu(), want_clip, rtol=2e-5)
    assert torch.equal(out.cpu(), OQ.pertensor_sym_fake_quant(w, clip.cpu(), 8))
    out2, clip2 = ops.tensor_fq(w.to(cuda_dev), kind=L.PT_INT_SYM, mode=L.W_SAWB, num_bits=8, c0=31.76, c1=-35.04)
    assert torch.equal(clip, clip2) and torch.equal(out, out2)
