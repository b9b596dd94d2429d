"""GPU parity of the drop-in modules against the reference's own outputs (golden files) and the
oracle, on the seeded inputs the golden files hold."""

import pytest
import torch

from conftest import load_golden
from fms_model_optimizer_b200 import ops
from fms_model_optimizer_b200.modules import LinearFPxAcc, QLinear, QLinearINT8Deploy, QLinearINT8Train
from fms_model_optimizer_b200.modules.linear import lower_qmodel_b200
from oracle import qlinear as OL
from test_host_logic import _RefLikeQLinear

pytestmark = pytest.mark.gpu


def test_deploy_int8_matches_reference_outputs(cuda_dev):
    for c in load_golden("deploy_int8.pt")["cases"]:
        q = QLinearINT8Deploy.from_fms_mo(
            _RefLikeQLinear(c), use_dynamic_max_act_Qfunc=-1, truncate_lsb=c["trun"], chunk_size=c["chunk"],
            max_acc_bits=c["accb"], target_device="cpu",
        ).to(cuda_dev)  # built with CPU arithmetic (as the golden run was), then moved
        y = q(c["x"].reshape(5, 8, -1).to(cuda_dev))
        assert y.dtype == c["x"].dtype and y.shape == c["y_kernel"].shape
        assert torch.equal(y.cpu(), c["y_kernel"]), (c["dtype"], c["trun"], c["chunk"], c["accb"])
        sd = q.state_dict()
        assert sd["weight"].dtype == torch.int8


def test_config1_shape_int8_linear_vs_oracle(cuda_dev):
    """The single W8A8 INT8 Linear workload (M=2048, K=4096, N=4096, bf16, 1% outlier channels x20, SmoothQuant 0.5,
    seed 0) through QLinear -> lowering -> QLinearINT8Deploy, against the oracle: int8 codes,
    int32 accumulators and the bf16 output bit for bit; and within 0.25 abs / 2e-2 rel-Frobenius
    of the reference's bf16 fake-quant forward (the figures the two reference paths differ by)."""
    torch.manual_seed(0)
    M, K, N = 2048, 4096, 4096
    x = torch.randn(M, K)
    x[:, torch.randperm(K)[:41]] *= 20
    x = x.bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    bias = (torch.randn(N) * 0.01).bfloat16()
    act_scale = x.float().abs().amax(0)
    sq = OL.smoothq_scale(act_scale.bfloat16(), w, 0.5, torch.bfloat16)
    w_clip = OL.qmax_clip_after_first_train_forward(w * sq)
    c = dict(weight=w, bias=bias, w_cv=w_clip, act_scale=act_scale.bfloat16())
    st = OL.deploy_from_fms_mo(w, bias, w_clip, act_scale.bfloat16(), 0.5)
    want, codes, in_scale, acc = OL.deploy_forward(st, x, return_parts=True)
    q = QLinearINT8Deploy.from_fms_mo(_RefLikeQLinear(c), use_dynamic_max_act_Qfunc=-1, target_device="cpu").to(cuda_dev)
    assert torch.equal(q.weight.cpu(), st.weight)
    y = q(x.to(cuda_dev))
    from fms_model_optimizer_b200 import _lib as L, ops

    g_codes, g_scale, _ = ops.act_quant(x.to(cuda_dev), mode=L.Q_I8_DYN, smooth=st.smoothq_scale.float().reshape(-1).to(cuda_dev), native_chain=3)
    assert torch.equal(g_codes.cpu(), codes)
    assert torch.equal(ops.imatmul(g_codes, q.weight.t()).cpu(), acc)
    assert torch.equal(y.cpu(), want)
    # Secondary: the reference's own bf16 fake-quant forward.  In bf16 the reference's deploy path
    # casts a rounded quotient of +128 straight to int8, which wraps to -128 (linear.py:1100); rows
    # holding such a code are off by design, the others agree to bf16 fake-quant accuracy.
    fake = OL.qlinear_fakequant_forward(x, w, bias, sq, w_clip)
    clean = ~(codes == -128).any(dim=1)
    assert clean.float().mean() > 0.5
    d = (y.cpu().float() - fake.float())[clean]
    assert d.abs().max() < 0.5 and torch.norm(d) / torch.norm(fake.float()[clean]) < 3e-2


def test_linear_fp8_matches_reference_outputs(cuda_dev):
    for c in load_golden("linear_fp8.pt")["cases"]:
        lin = torch.nn.Linear(c["weight"].shape[1], c["weight"].shape[0], bias=c["bias"] is not None).to(c["dtype"])
        with torch.no_grad():
            lin.weight.copy_(c["weight"])
            if c["bias"] is not None:
                lin.bias.copy_(c["bias"])
        q = LinearFPxAcc.from_nn(lin.to(cuda_dev), trun_bits=c["trun"], chunk_size=c["chunk"], dynamic_fp8="per_token",
                                 clamp_acc_to_dl16=c["dl16"])
        with torch.no_grad():
            y = q(c["x"].reshape(2, 12, -1).to(cuda_dev)).cpu()
        want = c["y"]
        assert y.dtype == want.dtype and y.shape == want.shape
        # e4m3 codes and scales are bit exact (test_gpu_quant); the fp32 accumulation order is the
        # kernel's own, so outputs agree to the rounding of the output dtype
        ulp = {torch.bfloat16: 2**-7, torch.float16: 2**-10, torch.float32: 2**-18}[c["dtype"]]
        tol = (ulp * 2 if c["trun"] == 0 and not c["dl16"] else 2.0 ** (-(23 - max(c["trun"], 14 if c["dl16"] else 0)) + 3))
        err = (y.float() - want.float()).abs()
        assert (err <= tol * want.float().abs().clamp(min=1.0)).all(), (c["dtype"], c["trun"], c["dl16"], err.max())
        if c["trun"] == 0 and not c["dl16"]:
            # sums of e4m3 products are often exact in fp32; where they are not, the order of the
            # fp32 additions shows in the last bit of an fp32 output and almost never after rounding
            # to a 16-bit output
            assert (y != want).float().mean() < (0.10 if c["dtype"] == torch.float32 else 0.002), c["dtype"]


def test_config3_shapes_fp8_linear_vs_oracle(cuda_dev):
    """The FP8 Linear sweep shapes (seed 2; the two large ones cut to 512 rows here, at full size in the next test), bf16 in / out, against the oracle: relative Frobenius error
    below 1e-3 (bf16 output rounding) and fewer than 1% of elements off by more than one bf16 ulp."""
    torch.manual_seed(2)
    for M, K, N in ((1, 4096, 14336), (128, 4096, 4096), (512, 4096, 14336), (512, 14336, 4096)):
        x = torch.randn(M, K).bfloat16()
        w = torch.randn(N, K).bfloat16()
        want = OL.linear_fpx_forward(x, w, None, chunk_size=64)
        lin = torch.nn.Linear(K, N, bias=False).bfloat16()
        with torch.no_grad():
            lin.weight.copy_(w)
        q = LinearFPxAcc.from_nn(lin.to(cuda_dev), trun_bits=0, chunk_size=64, dynamic_fp8="per_token")
        with torch.no_grad():
            y = q(x.to(cuda_dev)).cpu()
        rel = torch.norm(y.float() - want.float()) / torch.norm(want.float())
        assert rel < 1e-3, (M, K, N, rel)
        assert ((y.float() - want.float()).abs() > 2**-6 * want.float().abs().clamp(min=1.0)).float().mean() < 0.01


def test_fp8_linear_large_shapes_full_size_sampled(cuda_dev):
    """The two large shapes of the FP8 sweep at their stated size, M = 8192 (8192 x 4096 x 14336 and 8192 x 14336 x 4096,
    seed 2, bf16 in / out).  Per-token and per-channel scales make every output element a function of one row of x and one
    row of W only, so the oracle evaluated on a random 64 x 48 choice of rows and columns is exact parity for those
    elements: e4m3 codes and scales are bit exact, outputs within the bf16 rounding of an fp32 sum taken in another
    order (at most one bf16 place, fewer than 1 % of elements differing at all)."""
    from fms_model_optimizer_b200 import _lib as L

    torch.manual_seed(2)
    for M, K, N in ((8192, 4096, 14336), (8192, 14336, 4096)):
        x = torch.randn(M, K).bfloat16()
        w = torch.randn(N, K).bfloat16()
        lin = torch.nn.Linear(K, N, bias=False).bfloat16()
        with torch.no_grad():
            lin.weight.copy_(w)
        q = LinearFPxAcc.from_nn(lin.to(cuda_dev), trun_bits=0, chunk_size=64, dynamic_fp8="per_token")
        with torch.no_grad():
            y = q(x.to(cuda_dev)).cpu()
        rows, cols = torch.randperm(M)[:64], torch.randperm(N)[:48]
        want, xq, x_scale, wq, w_scale, _ = OL.linear_fpx_forward(x[rows], w[cols], None, chunk_size=64, return_parts=True)
        got = y[rows][:, cols]
        diff = (got.float() - want.float()).abs()
        assert (diff <= 2.0**-7 * want.float().abs().clamp(min=1e-2)).all(), (M, K, N, diff.max())
        assert (got != want).float().mean() < 0.01, (M, K, N)
        # the codes and scales of the sampled rows, bit for bit
        cq, cs, _ = ops.act_quant(x[rows].to(cuda_dev), mode=L.Q_F8_DYN, native_chain=3)
        assert torch.equal(cq.cpu().view(torch.uint8), xq.to(torch.float8_e4m3fn).view(torch.uint8))
        assert torch.equal(cs.cpu(), x_scale.reshape(-1).float())
        del q, lin, y
        torch.cuda.empty_cache()


def test_qat_qlinear_forward_backward_vs_oracle(cuda_dev):
    """One QLinear with PACT+ activations (clip +-6) and SAWB+ per-channel weights, forward and
    backward in fp32, against the oracle built from the reference's formulas (BERT-base shapes)."""
    from oracle import quantizers as OQ

    torch.manual_seed(3)
    M, K, N = 256, 768, 3072
    x = torch.randn(M, K) * 2.5
    lin = QLinear(K, N, num_bits_feature=8, qa_mode="pact+", num_bits_weight=8, qw_mode="sawb+perCh",
                  qcfg={"smoothq": False}, device=cuda_dev, act_clip_init_val=6.0, act_clip_init_valn=-6.0)
    w = lin.weight.detach().cpu().clone()
    b = lin.bias.detach().cpu().clone()
    G = torch.randn(M, N)
    lin.train()
    xd = x.to(cuda_dev).requires_grad_(True)
    y = lin(xd)
    (y * G.to(cuda_dev)).sum().backward()
    # oracle
    xo = x.clone().requires_grad_(True)
    wo = w.clone().requires_grad_(True)
    cv, cvn = torch.tensor([6.0]), torch.tensor([-6.0])
    qx = OQ.pact2plus_fwd(xo.detach(), cv, cvn, 8, True)
    qw, clip = OQ.sawb_perch(wo.detach(), 8)
    yo = torch.nn.functional.linear(qx, qw, b)
    assert torch.allclose(lin.quantize_weight.clip_val.cpu(), clip, rtol=3e-5)
    assert torch.norm(y.detach().cpu() - yo) / torch.norm(yo) < 1e-3  # TF32-free fp32 GEMM vs CPU GEMM
    g_qx = G @ qw
    gx_o, ga_o, gan_o = OQ.pact2plus_bwd(x, g_qx, cv, cvn, 8, True)
    assert torch.norm(xd.grad.cpu() - gx_o) / torch.norm(gx_o) < 1e-3
    assert abs(lin.quantize_feature.clip_val.grad.item() - ga_o.item()) < 2e-2 * max(1.0, abs(ga_o.item()))
    assert abs(lin.quantize_feature.clip_valn.grad.item() - gan_o.item()) < 2e-2 * max(1.0, abs(gan_o.item()))
    gw_o = G.t() @ qx
    assert torch.norm(lin.weight.grad.cpu() - gw_o) / torch.norm(gw_o) < 1e-3


def test_lowering_swaps_modules(cuda_dev):
    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q = QLinear(64, 48, num_bits_feature=8, qa_mode="pertokenmax", num_bits_weight=8, qw_mode="maxperCh",
                             qcfg={"smoothq": True, "smoothq_alpha": 0.5}, device=cuda_dev)
            self.f = torch.nn.Linear(48, 32, device=cuda_dev)

        def forward(self, x):
            return self.f(self.q(x))

    m = Toy()
    x = torch.randn(10, 64, device=cuda_dev)
    m.q.set_act_scale(x.abs().amax(0))
    m.train()
    with torch.no_grad():
        y_fake = m.q(x)
    m.eval()
    lower_qmodel_b200(m, use_dyn_max_act=-1)
    assert type(m.q).__name__ == "QLinearINT8Deploy" and type(m.f).__name__ == "LinearFPxAcc"
    with torch.no_grad():
        y = m.q(x)
    assert torch.norm(y - y_fake) / torch.norm(y_fake) < 2e-2
    with torch.no_grad():
        assert m(x).shape == (10, 32)


def test_int8_train_linear_matches_reference_outputs(cuda_dev):
    """QLinearINT8Train.forward against outputs of the reference class (bit-exact), and its
    floating-point backward against autograd of a plain linear."""
    for c in load_golden("extra.pt")["int8train"]:
        K, N = c["x"].shape[1], c["weight"].shape[0]
        lin = torch.nn.Linear(K, N, bias=c["bias"] is not None).to(c["dtype"])
        with torch.no_grad():
            lin.weight.copy_(c["weight"])
            if c["bias"] is not None:
                lin.bias.copy_(c["bias"])
        q = QLinearINT8Train.from_fms_mo(lin.to(cuda_dev), lsb_trun_bits=c["trun"], chunk_size=c["chunk"], max_acc_bits=c["accb"])
        x = c["x"].reshape(4, 5, K).to(cuda_dev).requires_grad_(True)
        y = q(x)
        assert y.dtype == c["dtype"] and torch.equal(y.detach().cpu(), c["y"]), (c["dtype"], c["trun"], c["chunk"], c["accb"])
        g = torch.randn_like(y)
        y.backward(g)
        xr = c["x"].reshape(4, 5, K).to(cuda_dev).requires_grad_(True)
        wr = c["weight"].to(cuda_dev).requires_grad_(True)
        torch.nn.functional.linear(xr, wr).backward(g)
        tol = 1e-4 if c["dtype"] == torch.float32 else 5e-2
        assert torch.allclose(x.grad.float(), xr.grad.float(), rtol=tol, atol=tol)
        assert torch.allclose(q.weight.grad.float(), wr.grad.float(), rtol=tol, atol=tol)
        if c["bias"] is not None:
            assert torch.allclose(q.bias.grad.float(), g.reshape(-1, N).sum(0).float(), rtol=tol, atol=tol)


def test_int8_train_linear_larger_shape_vs_oracle(cuda_dev):
    torch.manual_seed(3)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        x = torch.randn(300, 1024).to(dtype)
        lin = torch.nn.Linear(1024, 520, bias=True).to(dtype)
        want = OL.linear_int8_train_forward(x, lin.weight.detach(), lin.bias.detach(), 8, 64, 32)
        q = QLinearINT8Train.from_fms_mo(lin.to(cuda_dev), lsb_trun_bits=8, chunk_size=64, max_acc_bits=32)
        with torch.no_grad():
            got = q(x.to(cuda_dev))
        assert torch.equal(got.cpu(), want), dtype


class _QStub(torch.nn.Module):
    """Carries what QLinearCublasI8I32NT.from_fms_mo reads from a QLinear's quantizers."""

    def __init__(self, num_bits, clip_val, clip_valn=None, codes=None):
        super().__init__()
        self.num_bits = num_bits
        self.clip_val = clip_val
        self.clip_valn = clip_valn
        self.dequantize = True
        self._codes = codes

    def forward(self, w):
        assert not self.dequantize
        return self._codes.to(w.device, torch.float32)


def test_static_int8_linear_matches_reference_outputs(cuda_dev):
    from fms_model_optimizer_b200.modules import QLinearCublasI8I32NT, QLinearCutlassI8I32NT
    from fms_model_optimizer_b200.quant.quantizers import SAWB

    for c in load_golden("extra.pt")["static_int8"]:
        dt = c["dtype"]
        K, N = c["x"].shape[1], c["weight"].shape[0]
        src = torch.nn.Linear(K, N).to(dt)
        with torch.no_grad():
            src.weight.copy_(c["weight"])
            src.bias.copy_(c["bias"])
        src = src.to(cuda_dev)
        src.num_bits_feature = src.num_bits_weight = 8
        src.quantize_feature = _QStub(8, torch.tensor([c["a_cv"]]).to(dt).to(cuda_dev), torch.tensor([c["a_cvn"]]).to(dt).to(cuda_dev))
        qw = SAWB(8, dequantize=True, align_zero=True, perCh=N).to(dt).to(cuda_dev)  # this package's GPU quantizer, eval mode
        qw.clip_val.copy_(c["w_cv"].to(cuda_dev))
        qw.eval()
        src.quantize_weight = qw
        for cls in (QLinearCublasI8I32NT, QLinearCutlassI8I32NT):
            dep = cls.from_fms_mo(src)
            assert torch.equal(dep.weight.cpu(), c["w_int8"]) and torch.equal(dep.bias.cpu(), c["new_bias"])
            assert torch.equal(dep.input_scale.cpu(), c["input_scale"]) and torch.equal(dep.input_zp.cpu(), c["input_zp"])
            y = dep(c["x"].reshape(4, 6, K).to(cuda_dev))
            assert y.dtype == dt and torch.equal(y.cpu(), c["y"]), (dt, cls.__name__)


def test_fused_quantise_gemm_ops_match_reference_outputs(cuda_dev):
    g = load_golden("extra.pt")
    for c in g["q_iaddmm_dq"]:
        y = torch.ops.qlin_b200.q_iaddmm_dq(c["bias"].to(cuda_dev), c["x"].to(cuda_dev), c["w_i8"].to(cuda_dev).t(),
                                            c["scale_i"].to(cuda_dev), c["zp_i"].to(cuda_dev), c["scale_w"].to(cuda_dev))
        assert y.dtype == c["y"].dtype and torch.equal(y.cpu(), c["y"]), c["dtype"]
    for c in g["q_per_t_sym"]:
        y = torch.ops.qlin_b200.q_per_t_sym(c["x"].to(cuda_dev), c["s"], c["zp"])
        assert torch.equal(y.cpu(), c["y"])
    torch.manual_seed(2)
    x = torch.randn(257, 1000) * 3
    y = torch.ops.qlin_b200.q_per_t_sym(x.to(cuda_dev), torch.tensor(0.0213), torch.tensor(3))
    assert torch.equal(y.cpu(), OL.q_per_t_sym(x, 0.0213, 3))
    assert torch.equal(y.cpu(), torch.quantize_per_tensor(x, 0.0213, 3, torch.qint8).int_repr())


def test_linear_fp8_per_tensor_forward_backward_matches_reference_outputs(cuda_dev):
    """dynamic_fp8="per_tensor": e4m3 forward and e5m2 backward against outputs and gradients of the reference's autograd
    function.  Codes and scales are bit exact; the fp32 accumulation order is the kernel's own, so results agree to the
    rounding of the output dtype (or of the truncated accumulator where truncation is on)."""
    for c in load_golden("extra.pt")["fp8_train"]:
        K, N = c["weight"].shape[1], c["weight"].shape[0]
        lin = torch.nn.Linear(K, N, bias=c["bias"] is not None).to(c["dtype"])
        with torch.no_grad():
            lin.weight.copy_(c["weight"])
            if c["bias"] is not None:
                lin.bias.copy_(c["bias"])
        q = LinearFPxAcc.from_nn(lin.to(cuda_dev), trun_bits=c["trun"], chunk_size=c["chunk"], dynamic_fp8="per_tensor",
                                 clamp_acc_to_dl16=c["dl16"])
        x = c["x"].reshape(2, 12, K).to(cuda_dev).requires_grad_(True)
        y = q(x)
        y.backward(c["g"].to(cuda_dev))
        ulp = {torch.bfloat16: 2**-7, torch.float16: 2**-10, torch.float32: 2**-18}[c["dtype"]]
        tol = (ulp * 2 if c["trun"] == 0 and not c["dl16"] else 2.0 ** (-(23 - max(c["trun"], 14 if c["dl16"] else 0)) + 3))
        for name, got, want in (("y", y.detach(), c["y"]), ("gx", x.grad, c["gx"].reshape(2, 12, K)), ("gw", q.weight.grad, c["gw"])):
            got = got.cpu()
            assert got.dtype == want.dtype and got.shape == want.shape, name
            err = (got.float() - want.float()).abs()
            scale = want.float().abs().clamp(min=want.float().abs().mean().item())
            assert (err <= tol * scale).all(), (name, c["dtype"], c["trun"], c["dl16"], err.max().item())
        if c["bias"] is not None:
            gb, want = q.bias.grad.cpu(), c["gb"]
            assert gb.dtype == want.dtype
            assert torch.allclose(gb.float(), want.float(), rtol=4 * ulp, atol=4 * ulp * want.float().abs().max().item())


def test_e5m2_codes_bit_exact_and_gemm_exact_on_small_sums(cuda_dev):
    g = torch.Generator().manual_seed(21)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        x = (torch.randn(40, 96, generator=g) * 3).to(dtype)
        want_scale = x.abs().amax(dim=None) / torch.finfo(torch.float8_e5m2).max
        want = (x / want_scale).to(torch.float8_e5m2)
        codes, scale = ops.fp8_quant_per_tensor(x.to(cuda_dev), e5m2=True, eps=0.0)
        assert torch.equal(codes.cpu().view(torch.uint8), want.view(torch.uint8)), dtype
        assert scale.cpu().item() == want_scale.float().item()
    # e5m2 x e5m2 products of small integers sum exactly in fp32: the GEMM must be exact
    a = torch.randint(-4, 5, (256, 128), generator=g).float().to(torch.float8_e5m2)
    b = torch.randint(-4, 5, (384, 128), generator=g).float().to(torch.float8_e5m2)
    out = ops.gemm(a.to(cuda_dev), b.to(cuda_dev))
    assert torch.equal(out.cpu(), a.float() @ b.float().t())


def test_deploy_static_and_zero_shift_match_reference_outputs(cuda_dev):
    """QLinearINT8Deploy with static per-tensor activation quantisation (both formulas) and SmoothQuant in fp32, bf16 and
    fp16, with the fake zero-shift dynamic quantiser, and built by from_torch_iW: outputs equal the reference's own bit for
    bit (golden deploy_more.pt, produced by the reference on CPU)."""
    from test_host_logic import _ref_like_static

    g = load_golden("deploy_more.pt")
    for c in g["static"]:
        q = QLinearINT8Deploy.from_fms_mo(_ref_like_static(c), use_dynamic_max_act_Qfunc=False, use_PT_native_Qfunc=c["native"],
                                          target_device="cpu").to(cuda_dev)
        # the int8 codes first (the reference's qa_raw_qfunc / qa_fmo_mo_qfunc on x / smoothq_scale), then the output
        from fms_model_optimizer_b200 import _lib as L

        prep = q._prepared(cuda_dev)
        nat = 3 if c["dtype"] != torch.float32 else 0  # 16-bit models: smoothing and the quantiser chain both in the model dtype
        xd = c["x"].to(cuda_dev)
        if c["native"]:
            codes, _, _ = ops.act_quant(xd, mode=L.Q_I8_STATIC, smooth=prep["smooth"], smooth_rcp=prep["smooth_rcp"], native_chain=nat,
                                        scale0=float(q.input_scale), zp0=float(q.input_zp), shift=128.0, add2=0.0)
        else:
            codes, _, _ = ops.act_quant(xd, mode=L.Q_I8_STATIC_CLAMP_FIRST, smooth=prep["smooth"], smooth_rcp=prep["smooth_rcp"],
                                        native_chain=nat, scale0=float(q.quant_stepsize), zp0=float(q.quant_zero_point),
                                        lo=float(q.cvs[1]), hi=float(q.cvs[0]), shift=128.0)
        bad = (codes.cpu() != c["codes"]).sum().item()
        assert bad == 0, (c["dtype"], c["native"], "codes differ", bad, codes.numel())
        y = q(c["x"].reshape(6, 6, -1).to(cuda_dev))
        assert y.dtype == c["y"].dtype
        assert torch.equal(y.cpu(), c["y"]), (c["dtype"], c["native"], (y.cpu().float() - c["y"].float()).abs().max().item())
    for c in g["zero_shift"]:
        q = QLinearINT8Deploy.from_fms_mo(_RefLikeQLinear(c), use_dynamic_max_act_Qfunc=c["zero_shift"], target_device="cpu").to(cuda_dev)
        y = q(c["x"].reshape(6, 6, -1).to(cuda_dev))
        assert torch.equal(y.cpu(), c["y"]), (c["dtype"], c["zero_shift"], (y.cpu().float() - c["y"].float()).abs().max())
    for c in g["torch_iW"]:
        nnlin = torch.nn.Linear(c["weight"].shape[1], c["weight"].shape[0])
        with torch.no_grad():
            nnlin.weight.copy_(c["weight"])
            nnlin.bias.copy_(c["bias"])
        q = QLinearINT8Deploy.from_torch_iW(nnlin, "int8", c["a_cv"], c["a_cvn"], c["w_cv"], c["zero_shift"],
                                            use_PT_native_Qfunc=c["native"], target_device="cpu").to(cuda_dev)
        y = q(c["x"].to(cuda_dev))
        assert torch.equal(y.cpu(), c["y"]), (c["dtype"], c["native"])


def test_cublas_from_reference_matches_reference_outputs(cuda_dev):
    import torch.ao.nn.quantized.reference as nnqr

    from fms_model_optimizer_b200.modules import QLinearCublasI8I32NT

    for c in load_golden("deploy_more.pt")["from_reference"]:
        N, K = c["weight"].shape
        fl = torch.nn.Linear(K, N)
        with torch.no_grad():
            fl.weight.copy_(c["weight"])
            fl.bias.copy_(c["bias"])
        qparams = {"qscheme": torch.per_channel_affine, "dtype": torch.qint8, "scale": c["w_scales"], "zero_point": torch.zeros(N, dtype=torch.int64), "axis": 0}
        q = QLinearCublasI8I32NT.from_reference(nnqr.Linear.from_float(fl, qparams), c["in_scale"].clone(), c["in_zp"].clone(), torch.quint8,
                                                forceSymA=c["force_sym"]).to(cuda_dev)
        y = q(c["x"].to(cuda_dev))
        assert torch.equal(y.cpu(), c["y"]), c["force_sym"]


def test_deploy_module_sees_in_place_buffer_updates(cuda_dev):
    """A forward, then load_state_dict with other scales and bias (same storage, new values), then a forward again: the
    second result equals a fresh module's."""
    c = load_golden("deploy_int8.pt")["cases"][0]
    a = QLinearINT8Deploy.from_fms_mo(_RefLikeQLinear(c), use_dynamic_max_act_Qfunc=-1, target_device="cpu").to(cuda_dev)
    x = c["x"].to(cuda_dev)
    y0 = a(x)
    sd = {k: v.clone() for k, v in a.state_dict().items()}
    sd["w_scale"] = sd["w_scale"] * 2
    sd["bias"] = sd["bias"] + 1
    a.load_state_dict(sd)
    b = QLinearINT8Deploy.from_fms_mo(_RefLikeQLinear(c), use_dynamic_max_act_Qfunc=-1, target_device="cpu").to(cuda_dev)
    b.load_state_dict(sd)
    y1 = a(x)
    assert torch.equal(y1, b(x)) and not torch.equal(y1, y0)
