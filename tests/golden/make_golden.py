"""Generates the golden fixtures under tests/golden/ by running fms-model-optimizer itself.

Run once, in a container that has the reference source tree, as

    python tests/golden/make_golden.py /path/to/fms-model-optimizer

It imports ``fms_mo`` from that tree, drives the reference's own classes on CPU with small seeded
inputs and stores inputs and outputs as ``.pt`` files next to this script.  The tests never import
the reference; they only read these files.

Where the reference needs a CUDA device (its Triton matmuls), the reference's Python code is run
unchanged and only the matmul callable is replaced by ``oracle.gemm`` (stated per case below), so
those files pin the reference's quantise / dequantise chains, not the matmul.
"""

from __future__ import annotations

import importlib.metadata
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
if len(sys.argv) < 2:
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/fms-model-optimizer")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF))
sys.path.insert(0, str(ROOT))

_orig_version = importlib.metadata.version


def _version(name):  # the reference asks for its own installed version; it runs from source here
    return "0.0.0" if name == "fms-model-optimizer" else _orig_version(name)


importlib.metadata.version = _version

from fms_mo.custom_ext_kernels.utils import imatmul_ops_reg  # noqa: E402
from fms_mo.modules import linear as ref_linear  # noqa: E402
from fms_mo.quant import quantizers as ref_q  # noqa: E402

from oracle import gemm as OG  # noqa: E402


def save(name, obj):
    torch.save(obj, HERE / name)
    print(f"wrote {name}")


def gen_quantizers():
    torch.manual_seed(23)
    out = {}
    # PACT+ two-sided, forward and backward
    cases = []
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for nbits in (8, 4):
            for cv, cvn in ((2.5, -2.5), (3.55, -1.75), (6.0, -6.0)):
                x = (torch.randn(37, 96) * 3).to(dtype).requires_grad_(True)
                q = ref_q.PACT2(nbits, init_clip_valn=cvn, init_clip_val=cv, dequantize=True, pact_plus=True, align_zero=True)
                y = q(x)
                g = torch.randn(37, 96).to(dtype)
                y.backward(g)
                cases.append(
                    dict(dtype=dtype, nbits=nbits, cv=cv, cvn=cvn, x=x.detach().clone(), y=y.detach().clone(), g=g,
                         gx=x.grad.clone(), gcv=q.clip_val.grad.clone(), gcvn=q.clip_valn.grad.clone())
                )  # fmt: skip
    out["pact2"] = cases
    # SAWB+ per channel (training mode) and Qmax per channel
    cases = []
    for dtype in (torch.float32, torch.bfloat16):
        for nbits in (8, 4):
            w = (torch.randn(48, 80) * 0.05).to(dtype)
            q = ref_q.SAWB(nbits, dequantize=True, align_zero=True, perCh=48)
            q.train()
            y = q(w)
            q2 = ref_q.SAWB(nbits, dequantize=False, align_zero=True, perCh=48)
            q2.train()
            codes = q2(w.float())
            cases.append(dict(dtype=dtype, nbits=nbits, w=w, y=y.clone(), clip=q.clip_val.clone(), codes=codes.clone(),
                              clip_f32=q2.clip_val.clone()))  # fmt: skip
    out["sawb_perch"] = cases
    cases = []
    for dtype in (torch.float32, torch.bfloat16):
        w = (torch.randn(48, 80) * 0.05).to(dtype)
        q = ref_q.Qmax(8, align_zero=True, perCh=48)
        q.train()
        y = q(w)
        clip_after_train = q.clip_val.clone()
        q.eval()
        y_eval = q(w)
        cases.append(dict(dtype=dtype, w=w, y_train=y.clone(), clip_after_train=clip_after_train, y_eval=y_eval.clone()))
    out["qmax_perch"] = cases
    # per-token dynamic max (fake quant)
    cases = []
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        x = torch.randn(33, 80).to(dtype)
        x[5] = 0
        x[7] *= 1e-7
        x[:, 11] *= 20
        q = ref_q.QMaxDynamic(8, dim=-1)
        cases.append(dict(dtype=dtype, x=x, y=q(x).clone()))
    out["qmax_dynamic"] = cases
    save("quantizers.pt", out)


def build_ref_qlinear(K, N, dtype, x_cal, alpha=0.5, bias=True):
    qcfg = {"smoothq": True, "smoothq_alpha": alpha}
    lin = ref_linear.QLinear(K, N, bias=bias, num_bits_feature=8, qa_mode="pertokenmax", num_bits_weight=8,
                             qw_mode="maxperCh", qcfg=qcfg, device="cpu")  # fmt: skip
    with torch.no_grad():
        lin.weight.copy_(torch.randn(N, K) * 0.02)
        if bias:
            lin.bias.copy_(torch.randn(N) * 0.01)
    lin = lin.to(dtype)
    lin.set_act_scale(x_cal.float().abs().amax(0))
    return lin


def make_x(M, K, dtype):
    x = torch.randn(M, K)
    cols = torch.randperm(K)[: max(1, K // 100)]
    x[:, cols] *= 20
    return x.to(dtype)


def gen_qlinear():
    torch.manual_seed(0)
    cases = []
    for dtype in (torch.float32, torch.bfloat16):
        M, K, N = 40, 128, 96
        x = make_x(M, K, dtype)
        lin = build_ref_qlinear(K, N, dtype, x)
        lin.train()
        with torch.no_grad():
            y_train = lin(x)
        lin.eval()
        with torch.no_grad():
            y_eval = lin(x)
            sq = lin.get_smoothq_scale(x)
        cases.append(dict(dtype=dtype, x=x, weight=lin.weight.detach().clone(), bias=lin.bias.detach().clone(),
                          act_scale=lin.smoothq_act_scale.clone(), alpha=0.5, sq=sq.clone(),
                          w_clip=lin.quantize_weight.clip_val.clone(), y_train=y_train.clone(), y_eval=y_eval.clone()))  # fmt: skip
    save("qlinear_fakequant.pt", dict(cases=cases))


_mm = {"fn": None}


def _dispatch_mm(m1, m2):
    return _mm["fn"](m1, m2)


def gen_deploy():
    """QLinearINT8Deploy.from_fms_mo + forward.  fms_mo::imatmul is registered with a dispatcher:
    (a) ``kernel``: the reference runs its use_int_kernel="triton" code path and the matmul callable
        is oracle.gemm.imatmul_chunk_truncate (the Triton kernel cannot run without a GPU);
    (b) ``torch_loop``: the reference's own PyTorch chunk loop (iaddmm_int) with a plain integer
        matmul as callable -- entirely reference arithmetic."""
    torch.manual_seed(1)
    imatmul_ops_reg("triton", mm_func=_dispatch_mm)
    cases = []
    for dtype in (torch.float32, torch.bfloat16):
        M, K, N = 40, 256, 96
        x = make_x(M, K, dtype)
        lin = build_ref_qlinear(K, N, dtype, x)
        lin.train()
        with torch.no_grad():
            lin(x)
        lin.eval()
        for trun, chunk, accb in ((0, 100000, 32), (8, 64, 32), (4, 32, 32), (8, 64, 20)):
            dep = ref_linear.QLinearINT8Deploy.from_fms_mo(
                lin, use_int_kernel="triton", use_dynamic_max_act_Qfunc=-1, truncate_lsb=trun, chunk_size=chunk,
                max_acc_bits=accb, target_device="cpu",
            )  # fmt: skip
            # (a) kernel path
            dep.use_int_kernel = "triton"
            dep.iaddmm = dep.iaddmm_int
            _mm["fn"] = lambda m1, m2: OG.imatmul_chunk_truncate(m1, m2, chunk_trun_bits=trun, chunk_size=chunk, max_acc_bits=accb)
            y_kernel = dep(x.reshape(5, 8, K))
            # (b) reference torch loop
            dep.use_int_kernel = "cutlass"
            _mm["fn"] = lambda m1, m2: (m1.double() @ m2.double()).to(torch.int32)
            y_loop = dep(x.reshape(5, 8, K))
            cases.append(dict(dtype=dtype, x=x, weight=lin.weight.detach().clone(), bias=lin.bias.detach().clone(),
                              act_scale=lin.smoothq_act_scale.clone(), w_cv=lin.quantize_weight.clip_val.clone(),
                              trun=trun, chunk=chunk, accb=accb, w_int8=dep.weight.detach().clone(),
                              w_scale=dep.w_scale.clone(), smoothq_scale=dep.smoothq_scale.clone(),
                              dep_bias=dep.bias.clone(), y_kernel=y_kernel.clone(), y_loop=y_loop.clone()))  # fmt: skip
    save("deploy_int8.pt", dict(cases=cases))


def gen_fp8():
    """LinearFPxAcc forward: the reference's autograd function runs unchanged; its ``tl_matmul``
    callable is replaced by oracle.gemm.fmatmul_chunk_truncate."""
    torch.manual_seed(2)

    def tl_matmul(a, b, chunk_trun_bits=0, chunk_size=16, clamp_acc_to_dl16=False, **kw):
        return OG.fmatmul_chunk_truncate(a, b, chunk_trun_bits=chunk_trun_bits, chunk_size=chunk_size,
                                         clamp_acc_to_dl16=clamp_acc_to_dl16)  # fmt: skip

    ref_linear.tl_matmul = tl_matmul
    cases = []
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for trun, chunk, dl16, bias in ((0, 16, False, False), (0, 64, False, True), (8, 64, False, True), (0, 64, True, False)):
            M, K, N = 24, 192, 80
            x = torch.randn(M, K).to(dtype)
            x[3] = 0
            nn_lin = torch.nn.Linear(K, N, bias=bias).to(dtype)
            with torch.no_grad():
                nn_lin.weight.copy_(torch.randn(N, K).to(dtype))
            lin = ref_linear.LinearFPxAcc.from_nn(nn_lin, trun_bits=trun, chunk_size=chunk, dynamic_fp8="per_token",
                                                  clamp_acc_to_dl16=dl16, target_device="cpu")  # fmt: skip
            with torch.no_grad():
                y = lin(x.reshape(2, 12, K))
            cases.append(dict(dtype=dtype, trun=trun, chunk=chunk, dl16=dl16, x=x, weight=nn_lin.weight.detach().clone(),
                              bias=None if not bias else nn_lin.bias.detach().clone(), y=y.clone()))  # fmt: skip
    save("linear_fp8.pt", dict(cases=cases))


def gen_aiu_vectors():
    """The six W8A8 golden vectors of the reference's test-suite (tests/artifacts/aiu_addons),
    re-saved as one file: inputs and expected output of fms_mo::i8i8_aiu with smoothquant off."""
    out = {}
    art = REF / "tests" / "artifacts" / "aiu_addons"
    for f in sorted(art.glob("ref_w-*_a-*_sq-N.pt")):
        out[f.stem] = torch.load(f, weights_only=True)
    save("aiu_i8i8_vectors.pt", out)


def gen_static_int8():
    """QLinearCublasI8I32NT.from_fms_mo + forward (its library GEMM op replaced by an exact integer matmul),
    fms_mo::q_iaddmm_dq and fms_mo::q_per_t_sym as registered by the reference's imatmul_ops_reg."""
    torch.manual_seed(11)
    lib = torch.library.Library("mygemm", "DEF")
    lib.define("gemm_nt_i8i32(Tensor x, Tensor w) -> Tensor")
    lib.impl("gemm_nt_i8i32", lambda x, w: (x.double() @ w.double().t()).to(torch.int32), "CompositeExplicitAutograd")
    _keep.append(lib)
    imatmul_ops_reg("triton", mm_func=_dispatch_mm)
    _mm["fn"] = lambda m1, m2: (m1.double() @ m2.double()).to(torch.int32)
    out = {"static_int8": [], "q_iaddmm_dq": [], "q_per_t_sym": []}
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        M, K, N = 24, 160, 88
        x = (torch.randn(M, K) * 1.5).to(dtype)
        lin = ref_linear.QLinear(K, N, bias=True, num_bits_feature=8, qa_mode="pact+", num_bits_weight=8, qw_mode="sawb+perCh",
                                 qcfg={}, device="cpu")  # fmt: skip
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K) * 0.05)
            lin.bias.copy_(torch.randn(N) * 0.1)
            lin.quantize_feature.clip_val.fill_(3.7)
            lin.quantize_feature.clip_valn.fill_(-2.9)
        lin = lin.to(dtype)
        lin.train()
        with torch.no_grad():
            lin(x)
        lin.eval()
        dep = ref_linear.QLinearCublasI8I32NT.from_fms_mo(lin, target_device="cpu")
        y = dep(x.reshape(4, 6, K))
        out["static_int8"].append(dict(dtype=dtype, x=x, weight=lin.weight.detach().clone(), bias=lin.bias.detach().clone(),
                                       a_cv=3.7, a_cvn=-2.9, w_cv=lin.quantize_weight.clip_val.clone(),
                                       input_scale=dep.input_scale.clone(), input_zp=dep.input_zp.clone(),
                                       w_scale=dep.w_scale.clone(), w_int8=dep.weight.detach().clone(),
                                       new_bias=dep.bias.detach().clone(), y=y.clone()))  # fmt: skip
        if dtype != torch.bfloat16:
            w_i8 = torch.randint(-127, 128, (N, K), dtype=torch.int8)
            s_i, zp_i = torch.tensor([0.031]).to(dtype), torch.tensor([117])
            s_w = (torch.rand(N) * 0.01 + 0.001)
            bias = (torch.randn(N) * 0.1).to(dtype)
            y = torch.ops.fms_mo.q_iaddmm_dq(bias, x, w_i8.t(), s_i, zp_i, s_w)
            out["q_iaddmm_dq"].append(dict(dtype=dtype, x=x, w_i8=w_i8, scale_i=s_i, zp_i=zp_i, scale_w=s_w, bias=bias, y=y.clone()))
    xf = torch.randn(31, 77) * 2
    for s_, zp_ in ((0.0173, 0), (0.0291, -5)):
        st, zt = torch.tensor(s_), torch.tensor(zp_)
        out["q_per_t_sym"].append(dict(x=xf, s=st, zp=zt, y=torch.ops.fms_mo.q_per_t_sym(xf, st, zt).clone()))
    return out


def gen_fp8_per_tensor():
    """LinearFPxAcc with dynamic_fp8="per_tensor": forward and backward of the reference's autograd function, its
    ``tl_matmul`` callable replaced by oracle.gemm.fmatmul_chunk_truncate."""
    torch.manual_seed(13)

    def tl_matmul(a, b, chunk_trun_bits=0, chunk_size=16, clamp_acc_to_dl16=False, **kw):
        return OG.fmatmul_chunk_truncate(a, b, chunk_trun_bits=chunk_trun_bits, chunk_size=chunk_size,
                                         clamp_acc_to_dl16=clamp_acc_to_dl16)  # fmt: skip

    ref_linear.tl_matmul = tl_matmul
    cases = []
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for trun, chunk, dl16, bias in ((0, 64, False, True), (8, 32, False, False), (0, 64, True, True)):
            M, K, N = 24, 192, 80
            x = torch.randn(M, K).to(dtype).requires_grad_(True)
            nn_lin = torch.nn.Linear(K, N, bias=bias).to(dtype)
            with torch.no_grad():
                nn_lin.weight.copy_(torch.randn(N, K).to(dtype) * 0.3)
            lin = ref_linear.LinearFPxAcc.from_nn(nn_lin, trun_bits=trun, chunk_size=chunk, dynamic_fp8="per_tensor",
                                                  clamp_acc_to_dl16=dl16, target_device="cpu")  # fmt: skip
            y = lin(x.reshape(2, 12, K))
            g = torch.randn(2, 12, N).to(dtype)
            y.backward(g)
            cases.append(dict(dtype=dtype, trun=trun, chunk=chunk, dl16=dl16, x=x.detach().clone(), g=g,
                              weight=nn_lin.weight.detach().clone(), bias=None if not bias else nn_lin.bias.detach().clone(),
                              y=y.detach().clone(), gx=x.grad.clone(), gw=lin.weight.grad.clone(),
                              gb=None if not bias else lin.bias.grad.clone()))  # fmt: skip
    return cases


_keep = []


def gen_extra():
    """One-sided and symmetric PACT+ (forward and backward) and QLinearINT8Train.forward (its tl_matmul
    replaced by oracle.gemm.imatmul_chunk_truncate, everything else the reference's code)."""
    torch.manual_seed(5)
    out = {"pact1": [], "pactsym": [], "int8train": []}
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for nbits in (8, 4):
            x = (torch.randn(29, 96) * 3).to(dtype).requires_grad_(True)
            g = torch.randn(29, 96).to(dtype)
            q = ref_q.PACT(nbits, init_clip_val=3.3, dequantize=True, pact_plus=True)
            y = q(x)
            y.backward(g)
            out["pact1"].append(dict(dtype=dtype, nbits=nbits, cv=3.3, x=x.detach().clone(), g=g, y=y.detach().clone(),
                                     gx=x.grad.clone(), gcv=q.clip_val.grad.clone()))  # fmt: skip
            for intg in (True, False):
                x = (torch.randn(29, 96) * 3).to(dtype).requires_grad_(True)
                q = ref_q.PACTplusSym(nbits, init_clip_val=2.7, dequantize=True, intg_zp=intg)
                y = q(x)
                y.backward(g)
                out["pactsym"].append(dict(dtype=dtype, nbits=nbits, cv=2.7, intg=intg, x=x.detach().clone(), g=g,
                                           y=y.detach().clone(), gx=x.grad.clone(), gcv=q.clip_val.grad.clone()))  # fmt: skip

    def tl_matmul(a, b, chunk_trun_bits=0, chunk_size=16, max_acc_bits=32, **kw):
        return OG.imatmul_chunk_truncate(a, b, chunk_trun_bits=chunk_trun_bits, chunk_size=chunk_size, max_acc_bits=max_acc_bits)

    ref_linear.tl_matmul = tl_matmul
    for dtype in (torch.float32, torch.bfloat16):
        for trun, chunk, accb, bias in ((0, 64, 32, True), (8, 64, 32, False), (4, 32, 24, True)):
            M, K, N = 20, 192, 72
            x = torch.randn(M, K).to(dtype)
            lin = torch.nn.Linear(K, N, bias=bias).to(dtype)
            q = ref_linear.QLinearINT8Train.from_fms_mo(lin, lsb_trun_bits=trun, chunk_size=chunk, max_acc_bits=accb,
                                                        target_device="cpu")  # fmt: skip
            with torch.no_grad():
                y = q(x.reshape(4, 5, K))
            out["int8train"].append(dict(dtype=dtype, trun=trun, chunk=chunk, accb=accb, x=x, weight=lin.weight.detach().clone(),
                                         bias=None if not bias else lin.bias.detach().clone(), y=y.clone()))  # fmt: skip
    # per-tensor SAWB+ (training and eval), per-tensor Qmax, FP8 e4m3 quantise-dequantise
    out["sawb_tensor"], out["qmax_tensor"], out["fp8_fake"] = [], [], []
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for nbits in (8, 4, 2):
            w = (torch.randn(72, 100) * 0.05).to(dtype)
            q = ref_q.SAWB(nbits, dequantize=True, align_zero=True, perCh=False).to(dtype)
            q.train()
            y = q(w)
            clip = q.clip_val.clone()
            q.eval()
            y_eval = q(w * 1.5)
            q2 = ref_q.SAWB(nbits, dequantize=False, align_zero=True, perCh=False).to(dtype)
            q2.train()
            out["sawb_tensor"].append(dict(dtype=dtype, nbits=nbits, w=w, y=y.clone(), clip=clip, y_eval=y_eval.clone(),
                                           codes=q2(w).clone()))  # fmt: skip
        for align in (True, False):
            w = (torch.randn(72, 100) * 0.05).to(dtype)
            q = ref_q.Qmax(8, align_zero=align, minmax=False).to(dtype)
            q.train()
            y1 = q(w)
            y2 = q(w * 0.5)
            clip = q.clip_val.clone()
            q.eval()
            out["qmax_tensor"].append(dict(dtype=dtype, align=align, w=w, y1=y1.clone(), y2=y2.clone(), clip=clip,
                                           y_eval=q(w).clone()))  # fmt: skip
        x = torch.randn(37, 96).to(dtype)
        x[:, 5] *= 30
        x[3] *= 1e-3
        case = dict(dtype=dtype, x=x)
        for mode, kw in (("fp8_e4m3_scale_perToken", dict(perToken=True)), ("fp8_e4m3_scale_perCh", dict(perCh=37)),
                         ("fp8_e4m3_scale", {}), ("fp8_e4m3_sat", {})):  # fmt: skip
            case[mode] = ref_q.to_fp8(8, q_mode=mode, **kw)(x * (300 if mode.endswith("sat") else 1)).clone()
        out["fp8_fake"].append(case)
    out.update(gen_static_int8())
    out["fp8_train"] = gen_fp8_per_tensor()
    save("extra.pt", out)


def gen_deploy_more():
    """QLinearINT8Deploy beyond the per-token dynamic case: the two static per-tensor quantisers (use_PT_native_Qfunc on and
    off) with SmoothQuant, the fake zero-shift dynamic quantiser, from_torch_iW, and QLinearCublasI8I32NT.from_reference.
    The reference's own iaddmm_int runs with an exact integer matmul as its matmul callable."""
    torch.manual_seed(21)
    imatmul_ops_reg("triton", mm_func=_dispatch_mm)
    _mm["fn"] = lambda m1, m2: (m1.double() @ m2.double()).to(torch.int32)
    out = {"static": [], "zero_shift": [], "torch_iW": [], "from_reference": []}
    M, K, N = 36, 192, 80
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        x = make_x(M, K, dtype)
        lin = ref_linear.QLinear(K, N, bias=True, num_bits_feature=8, qa_mode="pact+", num_bits_weight=8, qw_mode="maxperCh",
                                 qcfg={"smoothq": True, "smoothq_alpha": 0.5}, device="cpu")  # fmt: skip
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K) * 0.02)
            lin.bias.copy_(torch.randn(N) * 0.01)
            lin.quantize_feature.clip_val.fill_(2.37)
            lin.quantize_feature.clip_valn.fill_(-1.93)
        lin = lin.to(dtype)
        lin.set_act_scale(x.float().abs().amax(0))
        lin.train()
        with torch.no_grad():
            lin(x)
        lin.eval()
        base = dict(dtype=dtype, x=x, weight=lin.weight.detach().clone(), bias=lin.bias.detach().clone(),
                    act_scale=lin.smoothq_act_scale.clone(), w_cv=lin.quantize_weight.clip_val.clone(),
                    a_cv=lin.quantize_feature.clip_val.detach().clone(), a_cvn=lin.quantize_feature.clip_valn.detach().clone())  # fmt: skip
        for native in (True, False):
            dep = ref_linear.QLinearINT8Deploy.from_fms_mo(lin, use_int_kernel="cutlass", use_dynamic_max_act_Qfunc=False,
                                                          use_PT_native_Qfunc=native, target_device="cpu")  # fmt: skip
            dep.iaddmm = dep.iaddmm_int
            y = dep(x.reshape(6, 6, K))
            xs = x / dep.smoothq_scale if torch.all(dep.smoothq_scale != 1).item() else x
            codes = (dep.qa_raw_qfunc(xs) if native else dep.qa_fmo_mo_qfunc(xs)).clone()
            out["static"].append(dict(base, native=native, input_scale=dep.input_scale.clone(), input_zp=dep.input_zp.clone(),
                                      w_scale=dep.w_scale.clone(), w_int8=dep.weight.detach().clone(), dep_bias=dep.bias.clone(),
                                      smoothq_scale=dep.smoothq_scale.clone(), codes=codes, y=y.clone()))  # fmt: skip
        # fake zero shift is meant for symmetric dynamic activations: a QLinear with per-token max activations
        lin_sym = build_ref_qlinear(K, N, dtype, x)
        lin_sym.train()
        with torch.no_grad():
            lin_sym(x)
        lin_sym.eval()
        base_sym = dict(dtype=dtype, x=x, weight=lin_sym.weight.detach().clone(), bias=lin_sym.bias.detach().clone(),
                        act_scale=lin_sym.smoothq_act_scale.clone(), w_cv=lin_sym.quantize_weight.clip_val.clone())
        for zs in (8, 40):
            dep = ref_linear.QLinearINT8Deploy.from_fms_mo(lin_sym, use_int_kernel="cutlass", use_dynamic_max_act_Qfunc=zs, target_device="cpu")
            dep.iaddmm = dep.iaddmm_int
            y = dep(x.reshape(6, 6, K))
            out["zero_shift"].append(dict(base_sym, zero_shift=zs, w_scale=dep.w_scale.clone(), w_int8=dep.weight.detach().clone(),
                                          dep_bias=dep.bias.clone(), corr_term=dep.corr_term.clone(),
                                          smoothq_scale=dep.smoothq_scale.clone(), y=y.clone()))  # fmt: skip
    # from_torch_iW: an nn.Linear that already holds integer weights
    for native in (True, False):
        for dtype in (torch.float32, torch.float16):
            nnlin = torch.nn.Linear(K, N, bias=True)
            with torch.no_grad():
                nnlin.weight.copy_(torch.randint(-127, 128, (N, K)).float())
                nnlin.bias.copy_(torch.randn(N) * 0.05)
            x = (torch.randn(M, K) * 1.2).to(dtype)
            dep = ref_linear.QLinearINT8Deploy.from_torch_iW(nnlin, "int8", 3.1, -2.4, 0.21, 17.0, use_int_kernel="cutlass",
                                                            use_PT_native_Qfunc=native, target_device="cpu")  # fmt: skip
            # the reference's constructor leaves out four attributes its own forward reads; they are set here to the
            # values that from_fms_mo gives an asymmetric static module without SmoothQuant
            dep.useSymAct = False
            dep.useDynMaxQfunc = False
            dep.use_fake_zero_shift = False
            dep.register_buffer("smoothq_scale", torch.tensor([1.0]))
            dep.iaddmm = dep.iaddmm_int
            y = dep(x)
            out["torch_iW"].append(dict(dtype=dtype, native=native, x=x, weight=nnlin.weight.detach().clone(), bias=nnlin.bias.detach().clone(),
                                        a_cv=3.1, a_cvn=-2.4, w_cv=0.21, zero_shift=17.0, dep_bias=dep.bias.detach().clone(),
                                        input_scale=dep.input_scale.clone(), input_zp=dep.input_zp.clone(), w_scale=dep.w_scale.clone(),
                                        y=y.clone()))  # fmt: skip
    # QLinearCublasI8I32NT.from_reference: a torch.ao reference-quantized Linear as input
    import torch.ao.nn.quantized.reference as nnqr

    for force_sym in (False, True):
        fl = torch.nn.Linear(K, N, bias=True)
        with torch.no_grad():
            fl.weight.copy_(torch.randn(N, K) * 0.05)
        w_scales = fl.weight.detach().abs().amax(1) / 127
        qparams = {"qscheme": torch.per_channel_affine, "dtype": torch.qint8, "scale": w_scales, "zero_point": torch.zeros(N, dtype=torch.int64), "axis": 0}
        refq = nnqr.Linear.from_float(fl, qparams)
        x = torch.randn(M, K) * 1.5
        in_s, in_zp = torch.tensor(0.0237), torch.tensor(121)
        dep = ref_linear.QLinearCublasI8I32NT.from_reference(refq, in_s.clone(), in_zp.clone(), torch.quint8, forceSymA=force_sym)
        y = dep(x)
        out["from_reference"].append(dict(x=x, weight=fl.weight.detach().clone(), bias=fl.bias.detach().clone(), w_scales=w_scales.clone(),
                                          in_scale=in_s, in_zp=in_zp, force_sym=force_sym, dep_input_scale=dep.input_scale.clone(),
                                          dep_input_zp=dep.input_zp.clone(), dep_bias=dep.bias.detach().clone(),
                                          w_int8=dep.weight.detach().clone(), w_scale=dep.w_scale.clone(), y=y.clone()))  # fmt: skip
    save("deploy_more.pt", out)


C4_CFG = dict(num_hidden_layers=2, hidden_size=768, num_attention_heads=12, intermediate_size=3072, vocab_size=30522,
              max_position_embeddings=128, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)  # no dropout: the step is deterministic
C4_BATCH, C4_SEQ = 4, 32


def gen_c4():
    """The QAT workload as the reference prepares it: a random-init BERT encoder (BERT-base widths, two layers) through
    ``qmodel_prep`` with the ``qat_int8`` recipe (PACT+ activations with clip values +-6, SAWB+ per-channel weights, no
    calibration), one training-mode forward and backward in fp32 on CPU with the loss ``(out * G).sum()``.  The fixture
    keeps the inputs' seeds, the output, every clip-value gradient, every bias gradient and, of every weight gradient,
    its sum, its absolute sum and its leading 48 x 48 block (the full gradients would be 57 MB).  The test rebuilds the
    same model from the same seed (transformers' BertModel initialiser on the CPU generator)."""
    from transformers import BertConfig, BertModel

    from fms_mo import qconfig_init, qmodel_prep

    torch.manual_seed(3)
    model = BertModel(BertConfig(**C4_CFG))
    init_sd = {k: v.clone() for k, v in model.state_dict().items()}
    ids = torch.randint(0, C4_CFG["vocab_size"], (C4_BATCH, C4_SEQ))
    G = torch.randn(C4_BATCH, C4_SEQ, C4_CFG["hidden_size"])
    qcfg = qconfig_init(recipe="qat_int8")
    qcfg.update(qmodel_calibration=0, qw_mode="sawb+perCh", act_clip_init_val=6.0, act_clip_init_valn=-6.0)
    qmodel_prep(model, (ids,), qcfg, use_dynamo=True)
    qnames = [n for n, m in model.named_modules() if type(m).__name__ == "QLinear"]
    model.train()
    out = model(ids).last_hidden_state
    (out * G).sum().backward()
    grads = {}
    for n, p in model.named_parameters():
        if p.grad is None:
            continue
        g = p.grad.detach()
        if "clip_val" in n or n.endswith(".bias") or g.numel() <= 4096:
            grads[n] = g.clone()
        else:
            grads[n] = dict(sum=g.double().sum().item(), abs_sum=g.double().abs().sum().item(), norm=g.double().norm().item(),
                            block=g.reshape(g.shape[0], -1)[:48, :48].clone())
    w_clips = {n: model.get_submodule(n).quantize_weight.clip_val.detach().clone() for n in qnames}
    # a checksum of the initial weights pins the test's rebuilt model to this one
    init_sum = {k: v.double().sum().item() for k, v in init_sd.items() if v.dtype.is_floating_point}
    save("c4_bert2.pt", dict(cfg=C4_CFG, batch=C4_BATCH, seq=C4_SEQ, ids=ids, G=G.bfloat16(), G_is="randn after ids, seed 3 (bf16 copy stored for a check)",
                             qlinear_names=qnames, out=out.detach().clone(), grads=grads, w_clips=w_clips, init_sum=init_sum,
                             qcfg={k: qcfg[k] for k in ("qa_mode", "qw_mode", "nbits_a", "nbits_w", "act_clip_init_val", "act_clip_init_valn")},
                             align_zero=qcfg.get("align_zero", True)))


def gen_bmm():
    """QBmm (fake-quantized matmul) and QBmmINT8Deploy (fms_mo/modules/bmm.py:26-228, 607-758) on CPU.

    The deploy forward subtracts a correction term whose sum runs over dimension 0 of m2's codes
    (bmm.py:741-746), so it only evaluates where that term broadcasts against the product: the cases below use
    m == k.  With a symmetric m1 the zero point is 128 and the term is zero; with an asymmetric m1 it is whatever
    the reference computes, stored here as it came out."""
    from fms_mo.modules.bmm import QBmm, QBmmINT8Deploy

    cases = []
    spec = [  # name, bits m1, mode m1, one-sided m1, mode m2, sym_7bits, dtype, (m, k, n)
        ("sym8_fp32", 8, "pactsym+", False, "pactsym+", False, torch.float32, (32, 32, 48)),
        ("sym8_bf16", 8, "pactsym+", False, "pactsym+", False, torch.bfloat16, (32, 32, 48)),
        ("sym8_fp16", 8, "pactsym+", False, "pactsym+", False, torch.float16, (32, 32, 48)),
        ("asym8_fp32", 8, "pact+", False, "pactsym+", False, torch.float32, (32, 32, 48)),
        ("onesided7_fp32", 8, "pact+", True, "pactsym+", True, torch.float32, (48, 48, 16)),
        ("sym8_fp32_bmm3d", 8, "pactsym+", False, "pactsym+", False, torch.float32, (64, 64, 64)),
    ]
    for i, (name, nb1, mode1, uni, mode2, sym7, dtype, (m, k, n)) in enumerate(spec):
        g = torch.Generator().manual_seed(700 + i)
        qcfg = {"use_PT_native_Qfunc": False, "sym_7bits_bmm": sym7}
        cv1, cvn1, cv2 = (1.0, 0.0, 2.5) if uni else (3.0, -2.0, 2.5)
        q = QBmm(num_bits_m1=nb1, qm1_mode=mode1, num_bits_m2=8, qm2_mode=mode2, m1_unidirectional=uni, replaceBmm=("bmm3d" not in name),
                 qcfg=qcfg, m1_clip_init_val=cv1, m1_clip_init_valn=cvn1, m2_clip_init_val=cv2, m2_clip_init_valn=-cv2)  # fmt: skip
        lead = (2, 2) if "bmm3d" in name else (2, 3)
        m1 = torch.randn(*lead, m, k, generator=g)
        m2 = torch.randn(*lead, k, n, generator=g)
        if uni:
            m1 = torch.softmax(m1 * 3, dim=-1)
        q = q.to(dtype)
        m1, m2 = m1.to(dtype), m2.to(dtype)
        a = m1.clone().requires_grad_(True)
        b = m2.clone().requires_grad_(True)
        y = q(a, b)
        go = torch.randn(y.shape, generator=g).to(dtype)
        y.backward(go)
        d = QBmmINT8Deploy.from_fms_mo(q, target_device="cpu")
        yd = d(m1, m2)
        cases.append(dict(name=name, kw=dict(num_bits_m1=nb1, qm1_mode=mode1, num_bits_m2=8, qm2_mode=mode2, m1_unidirectional=uni,
                                             replaceBmm=("bmm3d" not in name), m1_clip_init_val=cv1, m1_clip_init_valn=cvn1,
                                             m2_clip_init_val=cv2, m2_clip_init_valn=-cv2),
                          qcfg=qcfg, dtype=dtype, m1=m1, m2=m2, grad_out=go, y=y.detach().clone(), grad_m1=a.grad.clone(), grad_m2=b.grad.clone(),
                          clip_grads={n_: p_.grad.clone() for n_, p_ in q.named_parameters()},
                          deploy_buffers={n_: b_.clone() for n_, b_ in d.named_buffers()}, y_deploy=yd.clone(),
                          num_bits=(q.num_bits_m1, q.num_bits_m2)))  # fmt: skip
        print(name, "fake vs deploy max diff", (yd.float() - y.float()).abs().max().item())
    save("bmm.pt", dict(cases=cases))


if __name__ == "__main__":
    gen_quantizers()
    gen_qlinear()
    gen_deploy()
    gen_fp8()
    gen_aiu_vectors()
    gen_extra()
    gen_deploy_more()
    gen_c4()
    gen_bmm()
