"""Oracle for the quantized Linear modules (test infrastructure, see ``oracle/__init__.py``).

Restates, on CPU tensors, the forward passes of ``QLinear`` (fake-quant path),
``QLinearINT8Deploy`` (integer path) and ``LinearFPxAcc`` (FP8 path) of
``fms_mo/modules/linear.py``.  The matmuls go through ``oracle.gemm``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import gemm as G
from . import quantizers as Q


def smoothq_scale(act_scale: torch.Tensor, weight: torch.Tensor, alpha: float, dtype: torch.dtype) -> torch.Tensor:
    """QLinear.get_smoothq_scale (fms_mo/modules/linear.py:345-368); the deploy copy is
    linear.py:799-817.  All-zero activation scales mean "no smoothing" (scale 1)."""
    if act_scale.sum().item() == 0.0:
        return torch.tensor([1.0]).to(dtype)
    weight_scale = weight.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
    return (act_scale.pow(alpha) / weight_scale.pow(1.0 - alpha)).clamp(min=1e-5).to(dtype)


def qmax_clip_after_first_train_forward(w_smoothed: torch.Tensor, buffer_dtype: torch.dtype | None = None) -> torch.Tensor:
    """The clip_val buffer of Qmax(perCh) after one training-mode forward
    (fms_mo/quant/quantizers.py:3098-3128): the fresh per-row absmax is copied into the buffer and
    then passed through the moving average ``buf * (1 - 0.1) + cv_new * 0.1``.  The buffer is fp32
    unless the owning module was cast (``QLinear.to(dtype)`` casts it along)."""
    buffer_dtype = buffer_dtype if buffer_dtype is not None else w_smoothed.dtype
    cv_new = torch.max(w_smoothed.abs().reshape([w_smoothed.shape[0], -1]), dim=1).values
    buf = cv_new.to(buffer_dtype)
    return (buf * (1.0 - 0.1) + cv_new * 0.1).to(buffer_dtype)


def qlinear_fakequant_forward(
    x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], sq_scale: torch.Tensor, w_clip: torch.Tensor,
    num_bits: int = 8,
) -> torch.Tensor:  # fmt: skip
    """QLinear.forward (fms_mo/modules/linear.py:248-305) in eval mode with
    ``qa_mode="pertokenmax"`` (QMaxDynamic) and ``qw_mode="maxperCh"`` (Qmax per channel with the
    stored clip values): ``F.linear(Qa(x / s), Qw(W * s), bias)``."""
    qinput = Q.qmax_dynamic(x / sq_scale, num_bits).to(x.dtype)
    qweight = Q.perch_fake_quant(weight * sq_scale, w_clip, num_bits).to((weight * sq_scale).dtype).to(weight.dtype)
    return F.linear(qinput, qweight, bias)


@dataclass
class DeployState:
    """Buffers of a QLinearINT8Deploy built by from_fms_mo with per-token dynamic activations."""

    weight: torch.Tensor  # int8 [N, K]
    w_scale: torch.Tensor  # [N]
    smoothq_scale: torch.Tensor  # [1, K] or [1]
    bias: torch.Tensor  # [N], weight dtype
    input_zp: torch.Tensor
    corr_term: torch.Tensor


def deploy_from_fms_mo(
    weight: torch.Tensor, bias: Optional[torch.Tensor], w_cv: torch.Tensor, act_scale: Optional[torch.Tensor],
    alpha: float = 0.5, nbits_w: int = 8,
) -> DeployState:  # fmt: skip
    """QLinearINT8Deploy.from_fms_mo (fms_mo/modules/linear.py:780-911) for a symmetric dynamic
    activation quantiser (``use_dynamic_max_act_Qfunc=-1``) and a non-SAWB weight quantiser:
    SmoothQuant scale, ``w_scale = w_cv * 2 / 254``, int8 weights
    ``round((W * sq).t() / w_scale).clamp(-127, 127).t()``, zero correction term."""
    w_levels = 2**nbits_w - 2
    sq = torch.tensor([1.0], dtype=weight.dtype)
    if act_scale is not None:
        w_sq = weight.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
        # the module keeps alpha as a one-element buffer, so both powers are tensor-tensor pows
        # (not the sqrt fast path a Python scalar 0.5 would take)
        alpha_t = torch.tensor([alpha], dtype=torch.float32).to(act_scale.dtype)
        if torch.all(act_scale != 0).item():
            sq = (act_scale**alpha_t / w_sq ** (1.0 - alpha_t)).clamp(min=1e-5).to(act_scale.dtype)
    w_scale = w_cv * 2 / w_levels
    w_int8 = torch.round((weight * sq).t() / w_scale).clamp(-w_levels / 2, w_levels / 2).t().to(torch.int).to(torch.int8)
    corr_term = 0 * w_scale.float() * torch.tensor(1.0).float()
    new_bias = bias.float() - corr_term if bias is not None else -corr_term
    return DeployState(w_int8, w_scale, sq, new_bias.to(weight.dtype), torch.tensor(127, dtype=torch.int), corr_term)


def deploy_forward(
    st: DeployState, x: torch.Tensor, truncate_lsb: int = 0, chunk_size: int = 100000, max_acc_bits: int = 32,
    acc_dtype: torch.dtype = torch.float16, return_parts: bool = False,
):  # fmt: skip
    """QLinearINT8Deploy.forward with a kernel that chunks internally, i.e. the
    ``use_int_kernel="triton"`` branch (fms_mo/modules/linear.py:1309-1338, :1115-1188):
    ``x / smoothq_scale`` -> per-token int8 codes -> chunk-truncating int matmul ->
    ``(acc.float() * (input_scale * w_scale).to(fp16) + bias).to(acc_dtype)`` -> input dtype."""
    org_dtype = x.dtype
    tar_shape = tuple(x.shape[:-1]) + (st.weight.shape[0],)
    x2 = x.view(-1, x.shape[-1])
    if torch.all(st.smoothq_scale != 1).item():
        x2 = x2 / st.smoothq_scale
    codes, input_scale = Q.qa_dynamic_max_qfunc(x2)
    acc = G.imatmul_chunk_truncate(
        codes, st.weight.t(), chunk_trun_bits=truncate_lsb, chunk_size=chunk_size, max_acc_bits=max_acc_bits
    )
    out = (acc.float() * (input_scale * st.w_scale).to(torch.float16) + st.bias).to(acc_dtype)
    out = out.reshape(tar_shape).to(org_dtype)
    if return_parts:
        return out, codes, input_scale, acc
    return out


def linear_fpx_forward(
    x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], trun_bits: int = 0, chunk_size: int = 16,
    fp8_dyn="per_token", clamp_acc_to_dl16: bool = False, return_parts: bool = False,
):  # fmt: skip
    """LinearFuncFPxFwdBwd.forward (fms_mo/modules/linear.py:1902-1975) with dynamic FP8 scaling:
    e4m3 quantisation of x (per token) and W (per output channel), fp32-accumulated matmul with
    optional chunk truncation, ``* x_scale * w_scale.t()``, cast to the input dtype, ``+ bias``."""
    org_dtype = x.dtype
    target_shape = x.shape[:-1] + (weight.shape[0],)
    x2 = x.reshape(-1, x.shape[-1])
    per_tensor = fp8_dyn == "per_tensor"
    xq, x_scale = Q.fp8_dyn_quant(x2, per_tensor, clamp_acc_to_dl16)
    wq, w_scale = Q.fp8_dyn_quant(weight, per_tensor, clamp_acc_to_dl16)
    acc = G.fmatmul_chunk_truncate(
        xq.to(torch.float32), wq.to(torch.float32).t(), chunk_trun_bits=trun_bits, chunk_size=chunk_size,
        clamp_acc_to_dl16=clamp_acc_to_dl16,
    )  # fmt: skip
    out = (acc * x_scale * w_scale.t()).to(org_dtype).reshape(target_shape)
    if bias is not None:
        out = out + bias.to(org_dtype)
    if return_parts:
        return out, xq, x_scale, wq, w_scale, acc
    return out


def linear_int8_train_forward(x, weight, bias, lsb_trun_bits=0, chunk_size=64, max_acc_bits=32):
    """LinearFuncINT8FwdFP32Bwd.forward (fms_mo/modules/linear.py:2142-2191): per-token and per-channel
    ``amax / 127`` scales without a lower clamp, codes cast to int8 without clamp, chunk-truncating
    int matmul, ``acc.float() * x_scale * w_scale.t()`` cast to the input dtype, ``+ bias``."""
    org_dtype = x.dtype
    tar_shape = x.shape[:-1] + (weight.shape[0],)
    x2 = x.reshape(-1, x.shape[-1])
    x_scale = x2.abs().amax(dim=-1, keepdim=True) / 127
    w_scale = weight.abs().amax(dim=-1, keepdim=True) / 127
    x_i8 = torch.round(x2 / x_scale).to(torch.int8)
    w_i8 = torch.round(weight / w_scale).to(torch.int8)
    acc = G.imatmul_chunk_truncate(x_i8, w_i8.t(), chunk_trun_bits=lsb_trun_bits, chunk_size=chunk_size, max_acc_bits=max_acc_bits)
    out = (acc.to(torch.float) * x_scale * w_scale.t()).reshape(tar_shape).to(org_dtype)
    if bias is not None:
        out = out + bias.to(org_dtype)
    return out


def static_int8_from_fms_mo(weight, bias, a_cv, a_cvn, w_cv, nbits_a=8, nbits_w=8):
    """QLinearCublasI8I32NT.from_fms_mo (fms_mo/modules/linear.py:1427-1490) for a QLinear whose weight
    quantizer is SAWB per channel in eval mode: returns ``dict(input_scale, input_zp, w_scale, weight, bias)``."""
    input_scale = (a_cv - a_cvn) / (2**nbits_a - 1)
    input_zp = torch.round(-a_cvn / input_scale).to(torch.int)
    w_scale = (w_cv * 2 / (2**nbits_w - 2)).float()
    w_int8 = Q.perch_fake_quant(weight.float(), w_cv, nbits_w, dequantize=False).to(torch.int8)
    corr_term = (w_scale * input_scale * (input_zp - 128) * w_int8.sum(dim=1)).to(bias.dtype)
    return dict(input_scale=input_scale, input_zp=input_zp, w_scale=w_scale, weight=w_int8, bias=bias - corr_term)


def static_int8_forward(x, st, input_is_uint8=True):
    """QLinearCublasI8I32NT.forward (fms_mo/modules/linear.py:1499-1537) with an exact integer matmul."""
    in_dtype = x.dtype
    if input_is_uint8:
        q = torch.clamp((x / st["input_scale"] + st["input_zp"]).round(), 0, 255)
        q = (q.to(torch.int16) - 128).to(torch.int8)
    else:
        q = torch.clamp((x / st["input_scale"] + st["input_zp"]).round(), -127, 127).to(torch.int8)
    tar_shape = q.shape[:-1] + (st["weight"].shape[0],)
    acc = G.imatmul_chunk_truncate(q.reshape(-1, q.shape[-1]), st["weight"].t()).reshape(tar_shape)
    return (st["input_scale"] * st["w_scale"] * acc + st["bias"]).to(in_dtype)


def q_iaddmm_dq(bias, m1, m2, scale_i, zp_i, scale_w):
    """fms_mo::q_iaddmm_dq (fms_mo/custom_ext_kernels/utils.py:748-782)."""
    q = torch.clamp((m1 / scale_i + zp_i - 128).round(), -128, 127).to(torch.int8)
    acc = G.imatmul_chunk_truncate(q, m2)
    return (scale_i.float() * acc * scale_w + bias).to(m1.dtype)


def q_per_t_sym(x, s, zp):
    """fms_mo::q_per_t_sym (fms_mo/custom_ext_kernels/utils.py:792-794): the arithmetic of
    torch.quantize_per_tensor, ``clamp(nearbyint(x * (1 / s)) + zp, -128, 127)`` in fp32."""
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.as_tensor(s, dtype=torch.float32)
    return torch.clamp(torch.round(x.float() * inv) + int(zp), -128, 127).to(torch.int8)


def linear_fpx_backward(x, weight, grad_output, bias_dtype=None, trun_bits=0, chunk_size=16, clamp_acc_to_dl16=False):
    """LinearFuncFPxFwdBwd.backward with ``fp8_dyn="per_tensor"`` (fms_mo/modules/linear.py:1977-2058): e5m2 codes of
    x, W and grad_output with one unclamped ``amax / 57344`` scale each, two fp32-accumulated matmuls with optional chunk
    truncation, ``* grad_out_scale * scale`` and a cast; the bias gradient is the column sum of the (scaled) e5m2 gradient
    codes.  Returns ``(grad_input, grad_weight, grad_bias)``."""
    e5m2_max = torch.finfo(torch.float8_e5m2).max
    dl8_min = 0.0087890625
    out_dim, in_dim = weight.shape
    x2 = x.reshape(-1, x.shape[-1])
    dtype_input = x2.dtype
    g2 = grad_output.reshape(-1, out_dim).to(dtype_input)
    x_scale = x2.abs().amax(dim=None) / e5m2_max
    w_scale = weight.abs().amax(dim=None) / e5m2_max
    g_scale = g2.abs().amax(dim=None) / e5m2_max
    xq = (x2 / x_scale).to(torch.float8_e5m2).to(torch.float)
    wq = (weight / w_scale).to(torch.float8_e5m2).to(torch.float)
    gq = (g2 / g_scale).to(torch.float8_e5m2).to(torch.float)
    if clamp_acc_to_dl16:
        xq.masked_fill_(xq.abs() < dl8_min, 0)
        wq.masked_fill_(wq.abs() < dl8_min, 0)
        gq.masked_fill_(gq.abs() < dl8_min, 0)
    kw = dict(chunk_trun_bits=trun_bits, chunk_size=chunk_size, clamp_acc_to_dl16=clamp_acc_to_dl16)
    grad_weight = (G.fmatmul_chunk_truncate(gq.transpose(0, 1).contiguous(), xq, **kw) * g_scale.t() * x_scale).to(weight.dtype)
    grad_input = (G.fmatmul_chunk_truncate(gq, wq, **kw) * g_scale * w_scale).to(dtype_input)
    grad_input = grad_input.reshape(grad_output.shape[:-1] + (in_dim,))
    grad_bias = gq.sum(0).to(bias_dtype) if bias_dtype is not None else None
    return grad_input, grad_weight, grad_bias


# --------------------------------------------------------------------------------------------------
# QLinearINT8Deploy beyond the per-token dynamic case
# --------------------------------------------------------------------------------------------------
def deploy_static_from_fms_mo(weight, bias, w_cv, a_cv, a_cvn, act_scale, alpha=0.5, native=True, sym_act=False, nbits=8):
    """QLinearINT8Deploy.from_fms_mo (fms_mo/modules/linear.py:780-911) with ``use_dynamic_max_act_Qfunc=False``: static
    per-tensor activation quantisation from the PACT clip values, in the "PT native" form (``use_PT_native_Qfunc=True``,
    :832-834) or the older fms_mo form (:835-846).  Returns a dict of the module's buffers."""
    w_levels = 2**nbits - 2
    a_levels = 2**nbits - 1 - int(sym_act)
    sq = torch.tensor([1.0], dtype=weight.dtype)
    if act_scale is not None and torch.all(act_scale != 0).item():
        w_sq = weight.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
        alpha_t = torch.tensor([alpha], dtype=torch.float32).to(act_scale.dtype)
        sq = (act_scale**alpha_t / w_sq ** (1.0 - alpha_t)).clamp(min=1e-5).to(act_scale.dtype)
    st = dict(native=native, sym_act=sym_act, cvs=(a_cv, a_cvn), smoothq_scale=sq)
    w_scale = w_cv * 2 / w_levels
    if native:
        input_scale = torch.tensor([(a_cv - a_cvn) / a_levels])
        input_zp = torch.round(-a_cvn / input_scale)
    else:
        quant_scale = a_levels / torch.tensor([a_cv - a_cvn])
        st["quant_stepsize"] = 1.0 / quant_scale
        st["quant_zero_point"] = torch.round(a_cvn * quant_scale)
        input_scale = st["quant_stepsize"]
        input_zp = -st["quant_zero_point"]
        w_scale = 1.0 / (w_levels / (w_cv * 2))
    input_zp = input_zp.to(torch.int)
    w_int8 = torch.round((weight * sq).t() / w_scale).clamp(-w_levels / 2, w_levels / 2).t().to(torch.int)
    corr_int = 0 if sym_act else (input_zp - 128) * w_int8.sum(dim=1)
    corr_term = corr_int * w_scale.float() * input_scale.float()
    new_bias = (bias.float() - corr_term) if bias is not None else -corr_term
    st.update(input_scale=input_scale, input_zp=input_zp, w_scale=w_scale, weight=w_int8.to(torch.int8), bias=new_bias.to(weight.dtype))
    return st


def deploy_static_codes(st, x2):
    """qa_raw_qfunc / qa_fmo_mo_qfunc (fms_mo/modules/linear.py:1061-1083) after the SmoothQuant division of forward (:1330)."""
    if torch.all(st["smoothq_scale"] != 1).item():
        x2 = x2 / st["smoothq_scale"]
    sym = int(st["sym_act"])
    if st["native"]:
        return torch.clamp((x2 / st["input_scale"] + st["input_zp"] - 128 + sym).round(), -128, 127).to(torch.int8)
    return (torch.round(x2.clamp(st["cvs"][1], st["cvs"][0]) / st["quant_stepsize"] - st["quant_zero_point"]) - (128 - sym)).to(torch.int8)


def deploy_static_forward(st, x, acc_dtype=torch.float16):
    """QLinearINT8Deploy.forward + iaddmm_int (fms_mo/modules/linear.py:1309-1338, :1115-1188) for the static quantisers."""
    org_dtype = x.dtype
    tar_shape = tuple(x.shape[:-1]) + (st["weight"].shape[0],)
    codes = deploy_static_codes(st, x.reshape(-1, x.shape[-1]))
    acc = G.imatmul_chunk_truncate(codes, st["weight"].t())
    out = (acc.float() * (st["input_scale"] * st["w_scale"]).to(torch.float16) + st["bias"]).to(acc_dtype)
    return out.reshape(tar_shape).to(org_dtype)


def deploy_zero_shift_from_fms_mo(weight, bias, w_cv, act_scale, zero_shift, alpha=0.5, nbits=8):
    """from_fms_mo with ``0 < use_dynamic_max_act_Qfunc < 65``: dynamic per-tensor symmetric activations with a fake zero
    shift (fms_mo/modules/linear.py:828-831, :886-906).  The partial correction ``zp * sum_k W`` is kept apart from the
    bias because the input scale is only known at run time."""
    w_levels = 2**nbits - 2
    sq = torch.tensor([1.0], dtype=weight.dtype)
    if act_scale is not None and torch.all(act_scale != 0).item():
        w_sq = weight.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
        alpha_t = torch.tensor([alpha], dtype=torch.float32).to(act_scale.dtype)
        sq = (act_scale**alpha_t / w_sq ** (1.0 - alpha_t)).clamp(min=1e-5).to(act_scale.dtype)
    w_scale = w_cv * 2 / w_levels
    w_int8 = torch.round((weight * sq).t() / w_scale).clamp(-w_levels / 2, w_levels / 2).t().to(torch.int)
    input_zp = torch.tensor(zero_shift)
    corr_term = (input_zp * w_int8.sum(dim=1)) * w_scale.float() * torch.tensor(1.0).float()
    new_bias = (bias.float() - corr_term) if bias is not None else -corr_term
    new_bias = new_bias + corr_term
    return dict(smoothq_scale=sq, w_scale=w_scale, weight=w_int8.to(torch.int8), input_zp=input_zp, corr_term=corr_term,
                bias=new_bias.to(weight.dtype), nbits_a=nbits)


def deploy_zero_shift_forward(st, x, acc_dtype=torch.float16):
    """forward with qa_dyn_max_fake_zero_shift (fms_mo/modules/linear.py:1102-1113) and the bias update of iaddmm_int
    (:1179-1182)."""
    org_dtype = x.dtype
    tar_shape = tuple(x.shape[:-1]) + (st["weight"].shape[0],)
    x2 = x.reshape(-1, x.shape[-1])
    if torch.all(st["smoothq_scale"] != 1).item():
        x2 = x2 / st["smoothq_scale"]
    amax = x2.abs().max()
    levels = 2 ** (st["nbits_a"] - 1) - 1 - st["input_zp"]
    input_scale = amax.clamp(min=1e-5) / levels
    codes = (torch.round(x2 / input_scale) + st["input_zp"]).to(torch.int8)
    acc = G.imatmul_chunk_truncate(codes, st["weight"].t())
    updated_bias = st["bias"] - input_scale * st["corr_term"]
    out = (acc.float() * (input_scale * st["w_scale"]).to(torch.float16) + updated_bias).to(acc_dtype)
    return out.reshape(tar_shape).to(org_dtype)


def deploy_from_torch_iW(weight_int, bias, a_cv, a_cvn, w_cv, zero_shift, native=True, acc_dtype=torch.float):
    """QLinearINT8Deploy.from_torch_iW (fms_mo/modules/linear.py:922-1038): integer weights given, static activations."""
    if native:
        input_scale = torch.Tensor([(a_cv - a_cvn) / 255])
        input_zp = torch.round(-a_cvn / input_scale).to(torch.int)
        w_scale = torch.Tensor([w_cv * 2 / 254])
        st = {}
    else:
        quant_scale = 255 / torch.Tensor([a_cv - a_cvn])
        st = dict(quant_stepsize=1.0 / quant_scale, quant_zero_point=torch.round(a_cvn * quant_scale))
        input_scale = st["quant_stepsize"]
        input_zp = -st["quant_zero_point"]
        w_scale = 1.0 / (254 / torch.Tensor([w_cv * 2]))
    corr_term = (input_zp - 128) * torch.Tensor([zero_shift]) * w_scale * input_scale
    st.update(native=native, sym_act=False, cvs=(a_cv, a_cvn), smoothq_scale=torch.tensor([1.0]), input_scale=input_scale,
              input_zp=input_zp, w_scale=w_scale, weight=weight_int.to(torch.int8), bias=(bias - corr_term).to(acc_dtype))
    return st
