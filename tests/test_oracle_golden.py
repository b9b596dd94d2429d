"""The oracle against outputs of fms-model-optimizer itself (tests/golden/*.pt, produced by
tests/golden/make_golden.py) and against the reference test-suite's own W8A8 golden vectors."""

import pytest
import torch
import torch.nn.functional as F

from conftest import load_golden
from oracle import gemm as OG
from oracle import qlinear as OL
from oracle import quantizers as OQ


def test_pact2_fwd_bwd_matches_reference():
    for c in load_golden("quantizers.pt")["pact2"]:
        cv, cvn = torch.tensor([c["cv"]]), torch.tensor([c["cvn"]])
        y = OQ.pact2plus_fwd(c["x"], cv, cvn, c["nbits"], True)
        assert torch.equal(y, c["y"]), (c["dtype"], c["nbits"], c["cv"])
        gx, gcv, gcvn = OQ.pact2plus_bwd(c["x"], c["g"], cv, cvn, c["nbits"], True)
        assert torch.equal(gx, c["gx"])
        assert torch.equal(gcv.reshape(1).float(), c["gcv"].float())
        assert torch.equal(gcvn.reshape(1).float(), c["gcvn"].float())


def test_sawb_perch_matches_reference():
    for c in load_golden("quantizers.pt")["sawb_perch"]:
        y, clip = OQ.sawb_perch(c["w"], c["nbits"], dequantize=True)
        assert torch.equal(clip, c["clip"])
        assert torch.equal(y, c["y"])
        codes, clip32 = OQ.sawb_perch(c["w"].float(), c["nbits"], dequantize=False)
        assert torch.equal(clip32, c["clip_f32"])
        assert torch.equal(codes, c["codes"])


def test_qmax_perch_matches_reference():
    for c in load_golden("quantizers.pt")["qmax_perch"]:
        y, clip = OQ.qmax_perch(c["w"], 8)
        assert torch.equal(y, c["y_train"])
        latched = OL.qmax_clip_after_first_train_forward(c["w"], torch.float32)
        assert torch.equal(latched, c["clip_after_train"])
        y_eval = OQ.perch_fake_quant(c["w"], latched, 8).to(c["w"].dtype)
        assert torch.equal(y_eval, c["y_eval"])


def test_qmax_dynamic_matches_reference():
    for c in load_golden("quantizers.pt")["qmax_dynamic"]:
        assert torch.equal(OQ.qmax_dynamic(c["x"], 8), c["y"])


def test_qlinear_fakequant_matches_reference():
    for c in load_golden("qlinear_fakequant.pt")["cases"]:
        sq = OL.smoothq_scale(c["act_scale"], c["weight"], c["alpha"], c["x"].dtype)
        assert torch.equal(sq, c["sq"])
        w_clip = OL.qmax_clip_after_first_train_forward(c["weight"] * sq)
        assert torch.equal(w_clip, c["w_clip"])
        y = OL.qlinear_fakequant_forward(c["x"], c["weight"], c["bias"], sq, w_clip)
        assert torch.equal(y, c["y_eval"])


def test_deploy_matches_reference():
    for c in load_golden("deploy_int8.pt")["cases"]:
        st = OL.deploy_from_fms_mo(c["weight"], c["bias"], c["w_cv"], c["act_scale"], 0.5)
        assert torch.equal(st.weight, c["w_int8"])
        assert torch.equal(st.w_scale, c["w_scale"])
        assert torch.equal(st.smoothq_scale, c["smoothq_scale"])
        assert torch.equal(st.bias, c["dep_bias"])
        x3 = c["x"].reshape(5, 8, -1)
        y, codes, in_scale, acc = OL.deploy_forward(
            st, x3, truncate_lsb=c["trun"], chunk_size=c["chunk"], max_acc_bits=c["accb"], return_parts=True
        )
        assert torch.equal(y, c["y_kernel"])
        # The reference's own PyTorch chunk loop (iaddmm_int, linear.py:1142-1175) keeps the
        # accumulator shifted right by t bits and rescales by 2^t at the end; when chunking is
        # active its output must follow from the oracle's truncated accumulator.
        K = c["x"].shape[-1]
        if K > c["chunk"]:
            chunk = c["chunk"]
            acc_loop = torch.zeros_like(acc)
            rb = (1 << (c["trun"] - 1)) if c["trun"] > 0 else 0
            lo, hi = -(1 << (c["accb"] - 1)), (1 << (c["accb"] - 1)) - 1
            for k0 in range(0, K, chunk):
                p = (codes[:, k0 : k0 + chunk].double() @ st.weight.t()[k0 : k0 + chunk].double()).to(torch.int32)
                if c["accb"] < 32:
                    p = p.clamp(lo, hi)
                if c["trun"] > 0:
                    p = torch.bitwise_right_shift(p + rb, c["trun"])
                acc_loop += p
            assert torch.equal(acc_loop << c["trun"], acc), "oracle chunk GEMM differs from the torch-loop arithmetic"
            y_loop = (acc_loop * ((1 << c["trun"]) * in_scale * st.w_scale) + st.bias).to(torch.float16)
            y_loop = y_loop.reshape(5, 8, -1).to(c["x"].dtype)
            assert torch.equal(y_loop, c["y_loop"])


def test_linear_fp8_matches_reference():
    for c in load_golden("linear_fp8.pt")["cases"]:
        y = OL.linear_fpx_forward(
            c["x"].reshape(2, 12, -1), c["weight"], c["bias"], trun_bits=c["trun"], chunk_size=c["chunk"],
            clamp_acc_to_dl16=c["dl16"],
        )
        assert torch.equal(y, c["y"]), (c["dtype"], c["trun"], c["chunk"], c["dl16"])


def _aiu_i8i8(x, weight, bias, qdata, wtype, atype):
    """fms_mo::i8i8_aiu (fms_mo/aiu_addons/i8i8/i8i8_aiu_op.py:180-231) with smoothquant off, restated
    through the oracle's pieces: activations quantised symmetric per tensor / per token with codes
    clamped to +-127, int8 weights dequantised with w_cv / 127, fp16 linear."""
    out_feat, in_feat = weight.shape
    n_w = 1 if wtype == "per_tensor" else out_feat
    w_cv = qdata[:n_w]
    a_cv, a_cvn = qdata[2 * n_w : 2 * n_w + 1], qdata[2 * n_w + 1 : 2 * n_w + 2]
    sq = qdata[-1:]
    if atype == "per_tensor_symm":
        scale_x = 127 / a_cv
        x_dq = torch.round(x / sq * scale_x).clamp(-127, 127).to(torch.int8).div(scale_x).mul(sq)
    elif atype == "per_tensor_asymm":
        scale_x = 255 / (a_cv - a_cvn)
        zp_x = a_cvn * scale_x
        x_dq = torch.round(x / sq * scale_x - zp_x).clamp(0, 255).add(zp_x).div(scale_x).mul(sq)
    else:
        x_sq = x / sq
        scale_x = 127 / x_sq.abs().max(dim=-1, keepdim=True)[0]
        x_dq = torch.round(x_sq * scale_x).clamp(-127, 127).div(scale_x).mul(sq)
    w = weight * (w_cv if wtype == "per_tensor" else w_cv.unsqueeze(1)) / 127 / sq
    return F.linear(x_dq.to(x.dtype), w.to(x.dtype), bias.to(x.dtype))


def test_reference_w8a8_golden_vectors():
    vecs = load_golden("aiu_i8i8_vectors.pt")
    assert len(vecs) == 6
    for name, d in vecs.items():
        wtype = "per_tensor" if "w-per_tensor" in name else "per_channel"
        atype = name.split("_a-")[1].split("_sq")[0]
        x = d["x"].to(torch.float16)
        out = _aiu_i8i8(x, d["w_int"], d["bias"], d["qdata"].to(torch.float16), wtype, atype)
        assert torch.all((out - d["reference_out"]).abs() < 1e-4), name
        if atype == "per_token":
            # the per-token codes of this sibling definition equal the deploy quantiser's codes
            # wherever multiply-by-reciprocal and divide round alike (checked, not assumed)
            codes, _ = OQ.qa_dynamic_max_qfunc(x.reshape(-1, x.shape[-1]).float())
            x2 = x.reshape(-1, x.shape[-1]).float()
            alt = torch.round(x2 * (127 / x2.abs().max(dim=-1, keepdim=True)[0])).clamp(-127, 127).to(torch.int8)
            assert (codes != alt).float().mean() < 0.05


def test_chunk_gemm_properties():
    """Properties the reference's own GPU tests state for the truncating matmul
    (tests/triton_kernels/test_triton_mm.py:85-123), on the oracle."""
    torch.manual_seed(0)
    a = torch.randint(-128, 127, (64, 256), dtype=torch.int8)
    b = torch.randint(-128, 127, (256, 64), dtype=torch.int8)
    exact = (a.double() @ b.double())
    plain = OG.imatmul_chunk_truncate(a, b, chunk_size=32).double()
    assert torch.equal(plain, exact)

    def rel(t):
        return (torch.norm(t.double() - exact) / torch.norm(exact)).item()

    e32 = rel(OG.imatmul_chunk_truncate(a, b, chunk_trun_bits=8, chunk_size=32))
    e128 = rel(OG.imatmul_chunk_truncate(a, b, chunk_trun_bits=8, chunk_size=128))
    assert e32 < 1e-2 and e128 < 1e-2
    assert rel(OG.imatmul_chunk_truncate(a, b, max_acc_bits=18, chunk_size=32)) < 1e-2


def test_pact_one_sided_and_symmetric_match_reference():
    g = load_golden("extra.pt")
    for c in g["pact1"]:
        cv = torch.tensor([c["cv"]])
        assert torch.equal(OQ.pact_one_sided_fwd(c["x"], cv, c["nbits"]), c["y"]), (c["dtype"], c["nbits"])
        gx, gcv = OQ.pact_one_sided_bwd(c["x"], c["g"], cv, c["nbits"])
        assert torch.equal(gx, c["gx"])
        assert torch.equal(gcv.reshape(1).float(), c["gcv"].float())
    for c in g["pactsym"]:
        cv = torch.tensor([c["cv"]])
        assert torch.equal(OQ.pact_sym_fwd(c["x"], cv, c["nbits"], c["intg"]), c["y"]), (c["dtype"], c["nbits"], c["intg"])
        gx, gcv = OQ.pact_sym_bwd(c["x"], c["g"], cv, c["nbits"], c["intg"])
        assert torch.equal(gx, c["gx"])
        assert torch.equal(gcv.reshape(1).float(), c["gcv"].float())


def test_linear_int8_train_forward_matches_reference():
    for c in load_golden("extra.pt")["int8train"]:
        K = c["x"].shape[1]
        y = OL.linear_int8_train_forward(c["x"].reshape(4, 5, K), c["weight"], c["bias"], c["trun"], c["chunk"], c["accb"])
        assert y.dtype == c["y"].dtype and torch.equal(y, c["y"]), (c["dtype"], c["trun"], c["chunk"], c["accb"])


def test_per_tensor_sawb_and_qmax_match_reference():
    g = load_golden("extra.pt")
    for c in g["sawb_tensor"]:
        clip = OQ.sawb_clip_pertensor(c["w"], c["nbits"])
        assert torch.equal(clip, c["clip"]), (c["dtype"], c["nbits"])
        assert torch.equal(OQ.pertensor_sym_fake_quant(c["w"], clip, c["nbits"]), c["y"])
        assert torch.equal(OQ.pertensor_sym_fake_quant(c["w"] * 1.5, clip, c["nbits"]), c["y_eval"])
        assert torch.equal(OQ.pertensor_sym_fake_quant(c["w"], clip, c["nbits"], dequantize=False), c["codes"])
    for c in g["qmax_tensor"]:
        w = c["w"]
        m1, m2 = w.abs().max().unsqueeze(0), (w * 0.5).abs().max().unsqueeze(0)
        assert torch.equal(OQ.pertensor_sym_fake_quant(w, m1, 8, c["align"]), c["y1"])
        assert torch.equal(OQ.pertensor_sym_fake_quant(w * 0.5, m2, 8, c["align"]), c["y2"])
        clip = m1 * (1.0 - 0.1) + m1 * 0.1  # first call latches the fresh value, then the moving average
        clip = clip * (1.0 - 0.1) + m2 * 0.1
        assert torch.equal(clip, c["clip"])
        assert torch.equal(OQ.pertensor_sym_fake_quant(w, clip, 8, c["align"]), c["y_eval"])


def test_fp8_fake_quantisers_match_reference():
    for c in load_golden("extra.pt")["fp8_fake"]:
        x = c["x"]
        for key, fn in (("fp8_e4m3_scale_perToken", OQ.to_fp8_scaled_rows), ("fp8_e4m3_scale_perCh", OQ.to_fp8_scaled_rows),
                        ("fp8_e4m3_scale", OQ.to_fp8_scaled_tensor)):  # fmt: skip
            got = fn(x)[0]
            assert got.dtype == c[key].dtype and torch.equal(got.view(torch.int16 if x.element_size() == 2 else torch.int32),
                                                             c[key].view(torch.int16 if x.element_size() == 2 else torch.int32)), (key, c["dtype"])
        got = OQ.to_fp8_saturated(x * 300)
        assert torch.equal(got, c["fp8_e4m3_sat"])


def test_static_int8_linear_and_fused_ops_match_reference():
    g = load_golden("extra.pt")
    for c in g["static_int8"]:
        dt = c["dtype"]
        a_cv, a_cvn = torch.tensor([c["a_cv"]]).to(dt), torch.tensor([c["a_cvn"]]).to(dt)
        st = OL.static_int8_from_fms_mo(c["weight"], c["bias"], a_cv, a_cvn, c["w_cv"])
        assert torch.equal(st["input_scale"], c["input_scale"]) and torch.equal(st["input_zp"], c["input_zp"])
        assert torch.equal(st["w_scale"], c["w_scale"]) and torch.equal(st["weight"], c["w_int8"])
        assert torch.equal(st["bias"], c["new_bias"])
        K = c["x"].shape[1]
        y = OL.static_int8_forward(c["x"].reshape(4, 6, K), st)
        assert y.dtype == c["y"].dtype and torch.equal(y, c["y"]), dt
    for c in g["q_iaddmm_dq"]:
        y = OL.q_iaddmm_dq(c["bias"], c["x"], c["w_i8"].t(), c["scale_i"], c["zp_i"], c["scale_w"])
        assert y.dtype == c["y"].dtype and torch.equal(y, c["y"]), c["dtype"]
    for c in g["q_per_t_sym"]:
        assert torch.equal(OL.q_per_t_sym(c["x"], c["s"], c["zp"]), c["y"])


def test_fp8_linear_per_tensor_forward_backward_matches_reference():
    for c in load_golden("extra.pt")["fp8_train"]:
        K = c["x"].shape[1]
        x3 = c["x"].reshape(2, 12, K)
        y = OL.linear_fpx_forward(x3, c["weight"], c["bias"], c["trun"], c["chunk"], "per_tensor", c["dl16"])
        assert torch.equal(y, c["y"]), (c["dtype"], c["trun"], c["dl16"])
        gx, gw, gb = OL.linear_fpx_backward(x3, c["weight"], c["g"], None if c["bias"] is None else c["bias"].dtype, c["trun"],
                                            c["chunk"], c["dl16"])
        assert torch.equal(gx, c["gx"].reshape(gx.shape)) and torch.equal(gw, c["gw"])
        assert (gb is None and c["gb"] is None) or torch.equal(gb, c["gb"])


def test_deploy_static_zero_shift_and_torch_iW_equal_reference_outputs():
    """QLinearINT8Deploy with static per-tensor activations (both quantiser formulas, SmoothQuant on), with the fake
    zero-shift dynamic quantiser, and built by from_torch_iW: buffers, codes and outputs equal the reference's."""
    g = load_golden("deploy_more.pt")
    for c in g["static"]:
        st = OL.deploy_static_from_fms_mo(c["weight"], c["bias"], c["w_cv"], c["a_cv"], c["a_cvn"], c["act_scale"], 0.5, c["native"])
        for k, ref in (("weight", "w_int8"), ("bias", "dep_bias"), ("input_scale", "input_scale"), ("w_scale", "w_scale"), ("input_zp", "input_zp")):
            assert torch.equal(st[k], c[ref]), (c["dtype"], c["native"], k)
        assert torch.equal(OL.deploy_static_codes(st, c["x"]), c["codes"])
        assert torch.equal(OL.deploy_static_forward(st, c["x"].reshape(6, 6, -1)), c["y"])
    for c in g["zero_shift"]:
        st = OL.deploy_zero_shift_from_fms_mo(c["weight"], c["bias"], c["w_cv"], c["act_scale"], c["zero_shift"])
        assert torch.equal(st["bias"], c["dep_bias"]) and torch.equal(st["corr_term"], c["corr_term"])
        assert torch.equal(OL.deploy_zero_shift_forward(st, c["x"].reshape(6, 6, -1)), c["y"])
    for c in g["torch_iW"]:
        st = OL.deploy_from_torch_iW(c["weight"], c["bias"], c["a_cv"], c["a_cvn"], c["w_cv"], c["zero_shift"], c["native"])
        assert torch.equal(st["bias"], c["dep_bias"]) and torch.equal(st["w_scale"], c["w_scale"])
        assert torch.equal(OL.deploy_static_forward(st, c["x"], acc_dtype=torch.float), c["y"])


def _triton_case_inputs(c):
    g = torch.Generator().manual_seed(c["seed"])
    a = torch.randn(c["M"], c["K"], generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(c["N"], c["K"], generator=g).to(torch.float8_e4m3fn)
    cc = torch.randint(-1000, 1000, (c["M"], c["N"]), generator=g).to(torch.float32) if c["with_c"] else None
    return a, b, cc


def test_float_chunk_gemm_equals_the_reference_triton_kernel():
    """The float chunk-truncating matmul of the oracle against outputs of the reference's own Triton kernel
    (matmul_kernel / matmul_kernel_DABC through tl_matmul_chunk_truncate, run on a B200 by
    tests/golden/make_triton_golden.py): bit for bit wherever a chunk function is applied (mantissa truncation, DL16
    clamp, truncate-after-accumulate, initial accumulator); for the plain product, where the chunking only fixes an fp32
    summation order, to 1e-7 relative."""
    g = load_golden("triton_fp8_mm.pt")
    assert len(g["cases"]) == 6
    for c in g["cases"]:
        a, b, cc = _triton_case_inputs(c)
        kw = c["kw"]
        y = OG.fmatmul_chunk_truncate(a, b.t(), c=cc, chunk_trun_bits=kw.get("chunk_trun_bits", 0), chunk_size=kw.get("chunk_size", 16),
                                      truncate_then_accumulate=kw.get("truncate_then_accumulate", True),
                                      clamp_acc_to_dl16=kw.get("clamp_acc_to_dl16", False))  # fmt: skip
        got, ref = (y[:64, :64], c["block"]) if "block" in c else (y, c["y"])
        if kw.get("chunk_trun_bits", 0) > 0 or kw.get("clamp_acc_to_dl16", False):
            assert torch.equal(got, ref), (c["M"], kw)
        else:
            assert torch.norm(got - ref) / torch.norm(ref) < 1e-7, (c["M"], kw)
        if "sum" in c:
            assert abs(y.double().sum().item() - c["sum"]) <= 1e-6 * c["abs_sum"]


def test_bmm_oracle_matches_reference_fixture():
    """oracle/bmm.py against QBmm / QBmmINT8Deploy run by the reference itself (bmm.pt): the fake-quantized product and
    the deploy buffers bit for bit, the deploy output bit for bit including the infinities of its fp16 stage."""
    from oracle import bmm as OB

    for c in load_golden("bmm.pt")["cases"]:
        kw, (nb1, nb2) = c["kw"], c["num_bits"]
        dt = c["dtype"]
        cv1 = torch.tensor([kw["m1_clip_init_val"]]).to(dt)
        cvn1 = torch.tensor([kw["m1_clip_init_valn"]]).to(dt)
        cv2 = torch.tensor([kw["m2_clip_init_val"]]).to(dt)
        uni = kw["m1_unidirectional"]
        q1 = dict(mode=kw["qm1_mode"], num_bits=nb1, clip_val=cv1, clip_valn=cvn1, one_sided=uni)
        q2 = dict(mode=kw["qm2_mode"], num_bits=nb2, clip_val=cv2, clip_valn=None, one_sided=False)
        y = OB.qbmm_fake(c["m1"], c["m2"], q1, q2, kw["replaceBmm"])
        assert y.dtype == c["y"].dtype and torch.equal(y, c["y"]), c["name"]
        buf = OB.deploy_buffers(cv1, cvn1, nb1, kw["qm1_mode"], cv2, nb2)
        for k, v in c["deploy_buffers"].items():
            assert buf[k].dtype == v.dtype and torch.equal(buf[k], v), (c["name"], k)
        yd = OB.qbmm_int8_deploy(c["m1"], c["m2"], buf)
        want = c["y_deploy"]
        assert yd.dtype == want.dtype and torch.equal(torch.nan_to_num(yd.float(), nan=12345.0), torch.nan_to_num(want.float(), nan=12345.0)), c["name"]
