"""CPU tests of the host-side logic: module construction mirrors the reference's buffers, the chunk
normalisation matches, and modules refuse to run without a CUDA device."""

import pytest
import torch

from conftest import load_golden
from fms_model_optimizer_b200.modules import QLinear, QLinearINT8Deploy
from fms_model_optimizer_b200.modules.linear import _normalised_chunk
from oracle import gemm as OG


class _RefLikeQmax(torch.nn.Module):
    def __init__(self, clip):
        super().__init__()
        self.register_buffer("clip_val", clip)

    def forward(self, w):
        return w


class _RefLikeQLinear(torch.nn.Linear):
    """Carries the attributes from_fms_mo reads from the reference's QLinear."""

    def __init__(self, c):
        N, K = c["weight"].shape
        super().__init__(K, N, bias=True)
        with torch.no_grad():
            self.weight = torch.nn.Parameter(c["weight"].clone())
            self.bias = torch.nn.Parameter(c["bias"].clone())
        self.num_bits_feature = 8
        self.num_bits_weight = 8
        self.qa_mode = "pertokenmax"
        self.qw_mode = "maxperCh"
        self.quantize_feature = torch.nn.Identity()
        self.quantize_weight = _RefLikeQmax(c["w_cv"].clone())
        self.smoothq = True
        self.register_buffer("smoothq_act_scale", c["act_scale"].clone())
        self.register_buffer("smoothq_alpha", torch.tensor([0.5], dtype=torch.float32).to(c["act_scale"].dtype))


def test_from_fms_mo_reproduces_reference_buffers():
    for c in load_golden("deploy_int8.pt")["cases"]:
        q = QLinearINT8Deploy.from_fms_mo(
            _RefLikeQLinear(c), use_dynamic_max_act_Qfunc=-1, truncate_lsb=c["trun"], chunk_size=c["chunk"],
            max_acc_bits=c["accb"], target_device="cpu",
        )
        assert q.weight.dtype == torch.int8 and torch.equal(q.weight, c["w_int8"])
        assert torch.equal(q.w_scale, c["w_scale"])
        assert torch.equal(q.smoothq_scale, c["smoothq_scale"])
        assert torch.equal(q.bias, c["dep_bias"])
        assert set(dict(q.named_buffers())) >= {"input_scale", "input_zp", "w_scale", "w_zp", "smoothq_scale", "corr_term", "bias"}
        with pytest.raises(RuntimeError, match="CUDA"):
            q(c["x"])


def test_chunk_normalisation_matches_oracle_statement():
    for cs in (1, 8, 16, 31, 32, 33, 48, 64, 100, 128, 1000, 4096, 100000):
        if cs == 8:
            continue
        assert _normalised_chunk(cs) == OG.normalise_chunk_size(cs)


def test_qlinear_constructs_on_cpu_and_refuses_to_run():
    lin = QLinear(64, 32, num_bits_feature=8, qa_mode="pact+", num_bits_weight=8, qw_mode="sawb+perCh",
                  qcfg={"smoothq": False}, device="cpu", act_clip_init_val=6.0, act_clip_init_valn=-6.0)
    assert type(lin.quantize_feature).__name__ == "PACT2"
    assert type(lin.quantize_weight).__name__ == "SAWB"
    assert float(lin.quantize_feature.clip_val) == 6.0 and float(lin.quantize_feature.clip_valn) == -6.0
    with pytest.raises(RuntimeError):
        lin(torch.randn(4, 64))


def test_quantizer_factories_map_mode_strings_like_the_reference():
    """get_activation_quantizer / get_weight_quantizer (fms_mo/quant/quantizers.py:46-374): which class and which
    arguments every mode string on the quantized-Linear path resolves to.  Construction needs no GPU."""
    from fms_model_optimizer_b200.quant import quantizers as Q

    a = Q.get_activation_quantizer("pact+", nbits=8, clip_val=6.0, clip_valn=-6.0)
    assert isinstance(a, Q.PACT2) and a.clip_val.item() == 6.0 and a.clip_valn.item() == -6.0
    a = Q.get_activation_quantizer("pact+", nbits=4, clip_val=5.0, clip_valn=0.0, non_neg=True)
    assert isinstance(a, Q.PACT) and a.num_bits == 4 and a.clip_val.item() == 5.0
    a = Q.get_activation_quantizer("pactsym+", nbits=8, clip_val=3.0, align_zero=True)
    assert isinstance(a, Q.PACTplusSym) and a.intg_zp is True
    assert isinstance(Q.get_activation_quantizer("pertokenmax", nbits=8), Q.QMaxDynamic)
    a = Q.get_activation_quantizer("max", nbits=8, align_zero=False)
    assert isinstance(a, Q.Qmax) and not a.perCh and a.align_zero is False
    assert Q.get_activation_quantizer("maxsym", nbits=8, align_zero=False).align_zero is True
    a = Q.get_activation_quantizer("fp8_e4m3_scale_perToken", nbits=8)
    assert isinstance(a, Q.to_fp8) and a.perToken and not a.perCh
    w = Q.get_weight_quantizer("sawb+", nbits=8, w_shape=(48, 80))
    assert isinstance(w, Q.SAWB) and not w.perCh and w.clip_val.shape == (1,)
    w = Q.get_weight_quantizer("sawb+perCh", nbits=4, w_shape=(48, 80))
    assert isinstance(w, Q.SAWB) and w.perCh == 48 and w.clip_val.shape == (48,)
    w = Q.get_weight_quantizer("maxperCh", nbits=8, w_shape=(48, 80))
    assert isinstance(w, Q.Qmax) and w.perCh == 48
    assert not Q.get_weight_quantizer("max", nbits=8, w_shape=(48, 80)).perCh
    w = Q.get_weight_quantizer("pact+", nbits=8, w_shape=(48, 80), clip_val=2.5)
    assert isinstance(w, Q.PACTplusSym) and w.clip_val.item() == 2.5
    w = Q.get_weight_quantizer("fp8_e4m3_scale_perCh", nbits=8, w_shape=(48, 80))
    assert isinstance(w, Q.to_fp8) and w.perCh == 48
    for bad in ("lsq+", "dorefa"):
        with pytest.raises(NotImplementedError):
            Q.get_activation_quantizer(bad, nbits=8)
    with pytest.raises(ValueError):
        Q.to_fp8(8, q_mode="fp8_e5m2_sat")


class _RefLikePact(torch.nn.Module):
    """Stands in for the reference's PACT2 quantizer: only the clip values are read by from_fms_mo."""

    def __init__(self, cv, cvn):
        super().__init__()
        self.clip_val = torch.nn.Parameter(cv.clone())
        self.clip_valn = torch.nn.Parameter(cvn.clone())


def _ref_like_static(c):
    m = _RefLikeQLinear(c)
    m.qa_mode = "pact+"
    m.quantize_feature = _RefLikePact(c["a_cv"], c["a_cvn"])
    return m


def test_static_and_zero_shift_constructors_reproduce_reference_buffers():
    g = load_golden("deploy_more.pt")
    for c in g["static"]:
        q = QLinearINT8Deploy.from_fms_mo(_ref_like_static(c), use_dynamic_max_act_Qfunc=False, use_PT_native_Qfunc=c["native"],
                                          target_device="cpu")
        assert torch.equal(q.weight, c["w_int8"]) and torch.equal(q.bias, c["dep_bias"]), (c["dtype"], c["native"])
        assert torch.equal(q.input_scale, c["input_scale"]) and torch.equal(q.input_zp, c["input_zp"])
        assert torch.equal(q.w_scale, c["w_scale"]) and torch.equal(q.smoothq_scale, c["smoothq_scale"])
    for c in g["zero_shift"]:
        q = QLinearINT8Deploy.from_fms_mo(_RefLikeQLinear(c), use_dynamic_max_act_Qfunc=c["zero_shift"], target_device="cpu")
        assert q.use_fake_zero_shift and int(q.input_zp) == c["zero_shift"]
        assert torch.equal(q.weight, c["w_int8"]) and torch.equal(q.bias, c["dep_bias"]) and torch.equal(q.corr_term, c["corr_term"])
    for c in g["torch_iW"]:
        nnlin = torch.nn.Linear(c["weight"].shape[1], c["weight"].shape[0])
        with torch.no_grad():
            nnlin.weight.copy_(c["weight"])
            nnlin.bias.copy_(c["bias"])
        q = QLinearINT8Deploy.from_torch_iW(nnlin, "int8", c["a_cv"], c["a_cvn"], c["w_cv"], c["zero_shift"],
                                            use_PT_native_Qfunc=c["native"], target_device="cpu")
        assert torch.equal(q.bias.detach(), c["dep_bias"]) and torch.equal(q.w_scale, c["w_scale"])
        assert torch.equal(q.input_scale, c["input_scale"]) and torch.equal(q.input_zp, c["input_zp"])


def test_from_reference_reproduces_reference_buffers():
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
                                                forceSymA=c["force_sym"])
        assert torch.equal(q.weight, c["w_int8"]) and torch.equal(q.w_scale, c["w_scale"])
        assert torch.equal(q.input_scale, c["dep_input_scale"]) and torch.equal(q.input_zp, c["dep_input_zp"])
        assert torch.equal(q.bias.detach(), c["dep_bias"])
        assert q.input_dtype == (torch.qint8 if c["force_sym"] else torch.quint8)


def test_lowering_default_arguments_leave_plain_linears_alone():
    """With the default ``use_dyn_max_act=False`` no FP8 scaling mode follows from the arguments, so plain Linears stay;
    with -1 they become FP8 Linears with per-token scales."""
    from fms_model_optimizer_b200.modules import LinearFPxAcc
    from fms_model_optimizer_b200.modules.linear import lower_qmodel_b200

    c = load_golden("deploy_int8.pt")["cases"][0]

    def toy():
        m = torch.nn.Module()
        m.q = _RefLikeQLinear(c)
        type(m.q).__name__  # the lowering matches QLinear by class name
        m.head = torch.nn.Linear(8, 4)
        return m

    class QLinear(_RefLikeQLinear):
        pass

    for dyn, head_type in ((False, torch.nn.Linear), (-1, LinearFPxAcc)):
        m = toy()
        m.q = QLinear(c)
        lower_qmodel_b200(m, use_dyn_max_act=dyn)
        assert type(m.q) is QLinearINT8Deploy
        assert type(m.head) is head_type


def test_qbmm_deploy_buffers_equal_the_reference_fixture():
    """QBmm's constructor surface and QBmmINT8Deploy.from_fms_mo are host logic: built on the CPU they must carry the
    reference's parameter names, bit widths and buffers (bmm.pt, made by the reference's own classes)."""
    from conftest import load_golden
    from fms_model_optimizer_b200.modules import QBmm, QBmmINT8Deploy

    for c in load_golden("bmm.pt")["cases"]:
        q = QBmm(qcfg=dict(c["qcfg"]), **c["kw"]).to(c["dtype"])
        assert (q.num_bits_m1, q.num_bits_m2) == tuple(c["num_bits"])
        assert sorted(n for n, _ in q.named_parameters()) == sorted(c["clip_grads"])
        d = QBmmINT8Deploy.from_fms_mo(q, target_device="cpu")
        assert sorted(n for n, _ in d.named_buffers()) == sorted(c["deploy_buffers"])
        for k, v in c["deploy_buffers"].items():
            got = getattr(d, k)
            assert got.dtype == v.dtype and torch.equal(got, v), (c["name"], k)
    with pytest.raises(NotImplementedError):
        QBmm(num_bits_m1=8, qm1_mode="pactsym+", num_bits_m2=8, qm2_mode="pactsym+", qcfg={"qmodel_calibration_new": 3})
    with pytest.raises(RuntimeError, match="CUDA"):
        QBmmINT8Deploy.from_fms_mo(q, target_device="cpu")(c["m1"], c["m2"])
