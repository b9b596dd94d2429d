"""Oracle for the quantizers on the hot path (test infrastructure, see ``oracle/__init__.py``).

Each function restates one quantizer of ``fms_mo/quant/quantizers.py`` or one activation quantiser
of ``QLinearINT8Deploy`` (``fms_mo/modules/linear.py``) with the same ATen CPU operators in the
same order, so intermediate rounding in bf16 / fp16 matches the reference.
"""

from __future__ import annotations

import torch

# ---------------------------------------------------------------------------------------------
# dynamic per-token / per-channel max quantisers
# ---------------------------------------------------------------------------------------------


def qmax_dynamic(x: torch.Tensor, num_bits: int = 8, reduce_dim: int = -1) -> torch.Tensor:
    """QMaxDynamic.forward (fms_mo/quant/quantizers.py:3531-3534), also PerTokenMax.forward
    (:3492-3498): ``x.div(s).round().mul(s)`` with ``s = clamp(amax, 1e-5) / levels``; no clamp of
    the rounded codes."""
    levels = 2 ** (num_bits - 1) - 1
    amax = x.abs().max(dim=reduce_dim, keepdim=True)[0]
    scales = amax.clamp(min=1e-5).div(levels)
    return x.div(scales).round().mul(scales)


def qa_dynamic_max_qfunc(x: torch.Tensor, nbits: int = 8, reduce_dim: int = -1):
    """QLinearINT8Deploy.qa_dynamic_max_qfunc (fms_mo/modules/linear.py:1085-1100): returns
    ``(int8 codes, input_scale)``.  The rounded quotient is cast straight to int8 (no clamp)."""
    amax = x.abs().max(dim=reduce_dim, keepdim=True)[0]
    levels = 2 ** (nbits - 1) - 1
    input_scale = amax.clamp(min=1e-5).div(levels)
    return torch.round(x / input_scale).to(torch.int8), input_scale


def qa_raw_qfunc(x: torch.Tensor, input_scale: torch.Tensor, input_zp: torch.Tensor, use_sym_act: bool) -> torch.Tensor:
    """QLinearINT8Deploy.qa_raw_qfunc (fms_mo/modules/linear.py:1061-1071)."""
    y = torch.clamp((x / input_scale + input_zp - 128 + use_sym_act).round(), -128, 127)
    return y.to(torch.int8)


def qa_fmo_mo_qfunc(
    x: torch.Tensor, cv: torch.Tensor, cvn: torch.Tensor, quant_stepsize: torch.Tensor, quant_zero_point: torch.Tensor,
    use_sym_act: bool,
) -> torch.Tensor:  # fmt: skip
    """QLinearINT8Deploy.qa_fmo_mo_qfunc (fms_mo/modules/linear.py:1073-1083): clamp, then round."""
    y = torch.round(x.clamp(cvn, cv) / quant_stepsize - quant_zero_point) - (128 - use_sym_act)
    return y.to(torch.int8)


# ---------------------------------------------------------------------------------------------
# per-channel weight quantisers
# ---------------------------------------------------------------------------------------------
SAWB_COEFFS = {103: (2.6, -1.71), 403: (12.035, -12.03), 803: (31.76, -35.04)}  # quantizers.py:635-641
SAWB_CODE = {8: 803, 4: 403, 2: 103}  # quantizers.py:518


def sawb_clip_perch(w: torch.Tensor, num_bits: int) -> torch.Tensor:
    """sawb_params_code(perCh=True) (fms_mo/quant/quantizers.py:648-655)."""
    c0, c1 = SAWB_COEFFS[SAWB_CODE[num_bits]]
    reduce_dim = list(range(1, w.dim()))
    mu = torch.mean(w.abs(), dim=reduce_dim)
    std = torch.mean(w**2, dim=reduce_dim).sqrt()
    return c1 * mu + c0 * std


def perch_fake_quant(w: torch.Tensor, clip: torch.Tensor, num_bits: int, dequantize: bool = True) -> torch.Tensor:
    """The quantise step shared by SAWBPlusZeroPerChSTE.forward (fms_mo/quant/quantizers.py:539-567)
    and QmaxPerChSTE.forward (:3199-3220): ``scale = clip * 2 / (2^b - 2)``, then
    ``torch.fake_quantize_per_channel_affine`` on the fp32 copy with zero_point 0 and the symmetric
    integer range, cast to the clip dtype.  ``dequantize=False`` follows the SAWB branch
    (``torch.quantize_per_channel(...).int_repr().clamp``)."""
    int_l = -(2 ** (num_bits - 1)) + 1
    int_u = -int_l
    scale = clip * 2 / (2**num_bits - 2)
    zero_point = torch.zeros_like(scale)
    if dequantize:
        return torch.fake_quantize_per_channel_affine(
            w.float(), scale.float(), zero_point.float(), axis=0, quant_min=int_l, quant_max=int_u
        ).to(clip.dtype)
    return torch.quantize_per_channel(w, scale, zero_point, 0, torch.qint8).int_repr().clamp(int_l, int_u)


def sawb_perch(w: torch.Tensor, num_bits: int = 8, dequantize: bool = True):
    """SAWB(perCh, align_zero=True) in training mode: returns ``(quantised, clip_val)``."""
    clip = sawb_clip_perch(w, num_bits)
    return perch_fake_quant(w, clip, num_bits, dequantize), clip


def qmax_perch(w: torch.Tensor, num_bits: int = 8):
    """Qmax(perCh) in training mode on its first call (fms_mo/quant/quantizers.py:3050-3115):
    clip = per-row absmax, quantised with QmaxPerChSTE and cast back to the input dtype.
    Returns ``(quantised, clip_val)``."""
    clip = torch.max(w.abs().reshape([w.shape[0], -1]), dim=1).values
    return perch_fake_quant(w, clip, num_bits).to(w.dtype), clip


def sawb_clip_pertensor(w: torch.Tensor, num_bits: int) -> torch.Tensor:
    """sawb_params_code(perCh=False) (fms_mo/quant/quantizers.py:657-671) with the fallback of
    SAWBPlusZeroSTE.forward (:482-487): a non-positive clip becomes max|w|; returned with shape [1]."""
    c0, c1 = SAWB_COEFFS[SAWB_CODE[num_bits]]
    x = w.flatten()
    mu = x.abs().mean()
    std = x.mul(x).mean().sqrt()
    clip = c1 * mu + c0 * std
    if clip <= 0:
        clip = w.abs().max()
    return clip.unsqueeze(0)


def pertensor_sym_fake_quant(w: torch.Tensor, clip: torch.Tensor, num_bits: int, align_zero: bool = True, dequantize: bool = True):
    """The quantise step shared by SAWBPlusZeroSTE.forward (fms_mo/quant/quantizers.py:488-495) and
    QmaxSTE.forward (:3168-3183) with linear_quantize / linear_dequantize (:2561-2585, :2622-2633)."""
    scale = (2**num_bits - 2) if align_zero else (2**num_bits - 1)
    clip = clip.to(w.dtype)
    out = w.mul(1 / clip).clamp(-1, 1).mul(0.5).add(0.5)
    out = torch.round(scale * out - 0.0)
    if dequantize:
        out = (out + 0.0) / scale
        return (2 * out - 1) * clip
    return out - scale / 2


def to_fp8_scaled_rows(x: torch.Tensor):
    """to_fp8_scaled_perToken / to_fp8_scaled_perCh on a 2-D tensor with emulate=True, e4m3
    (fms_mo/quant/quantizers.py:5336-5420): returns ``(fake-quantised x, scale multiplier)``."""
    amax = torch.max(torch.abs(x), dim=-1, keepdim=True)[0]
    return _fp8_scaled(x, amax)


def to_fp8_scaled_tensor(x: torch.Tensor):
    """to_fp8_scaled, emulate=True, e4m3 (fms_mo/quant/quantizers.py:5352-5372)."""
    return _fp8_scaled(x, torch.max(torch.abs(x)))


def _fp8_scaled(x, amax):
    res = 448.0 / torch.clamp(amax, min=1e-12)
    if x.dtype is torch.float16:
        res = torch.clamp(res, max=torch.finfo(torch.float16).max)
    scale = torch.empty_like(amax, dtype=x.dtype)
    scale.copy_(res)
    return (to_fp8_saturated(x * scale) / scale).to(x.dtype), scale


def to_fp8_saturated(x: torch.Tensor) -> torch.Tensor:
    """to_fp8_saturated, emulate=True, e4m3 (fms_mo/quant/quantizers.py:5316-5333)."""
    return x.clamp(min=-448.0, max=448.0).to(torch.float8_e4m3fn).to(x.dtype)


# ---------------------------------------------------------------------------------------------
# PACT+ two-sided
# ---------------------------------------------------------------------------------------------
def _pact2_params(x: torch.Tensor, clip_val: torch.Tensor, clip_valn: torch.Tensor, num_bits: int, align_zero: bool):
    cv, cvn = clip_val.to(x.dtype), clip_valn.to(x.dtype)
    n_levels = 2**num_bits - 1
    scale = n_levels / (cv - cvn)
    stepsize = 1.0 / scale
    zp = cvn * scale
    if align_zero:
        zp = torch.round(zp)
    return cv, cvn, n_levels, stepsize, zp


def pact2plus_fwd(x: torch.Tensor, clip_val: torch.Tensor, clip_valn: torch.Tensor, num_bits: int = 8, align_zero: bool = True):
    """PACTplus2STE.forward with dequantize=True, use_PT_native_Qfunc=False
    (fms_mo/quant/quantizers.py:1962-2055)."""
    cv, cvn, _, stepsize, zp = _pact2_params(x, clip_val, clip_valn, num_bits, align_zero)
    y = torch.minimum(x, cv)
    y = torch.maximum(y, cvn)
    y = torch.round(y / stepsize - zp)
    return (y + zp) * stepsize


def pact2plus_bwd(
    x: torch.Tensor, grad_out: torch.Tensor, clip_val: torch.Tensor, clip_valn: torch.Tensor, num_bits: int = 8,
    align_zero: bool = True,
):  # fmt: skip
    """PACTplus2STE.backward (fms_mo/quant/quantizers.py:2058-2102): returns
    ``(grad_x, grad_clip_val, grad_clip_valn)`` with the two clip gradients as 0-dim tensors."""
    cv, cvn, n_levels, stepsize, _ = _pact2_params(x, clip_val, clip_valn, num_bits, align_zero)
    z = (x - cvn) / stepsize
    delz = (z - torch.round(z)) / n_levels
    zeros = torch.zeros_like(grad_out)
    gx = torch.where(x <= cvn, zeros, grad_out)
    gx = torch.where(x >= cv, zeros, gx)
    ga = -grad_out * delz
    gan = -ga
    ga = torch.where(x <= cvn, zeros, ga)
    ga = torch.where(x >= cv, grad_out, ga)
    gan = torch.where(x >= cv, zeros, gan)
    gan = torch.where(x <= cvn, grad_out, gan)
    return gx, ga.sum(), gan.sum()


def pact_one_sided_fwd(x, clip_val, num_bits=8):
    """PACTplusSTE.forward, dequantize=True (fms_mo/quant/quantizers.py:1018-1042)."""
    cv = clip_val.to(x.dtype)
    stepsize = 1.0 / ((2**num_bits - 1) / cv)
    return torch.round(torch.clamp(x, torch.zeros_like(cv), cv) / stepsize) * stepsize


def pact_one_sided_bwd(x, grad_out, clip_val, num_bits=8):
    """PACTplusSTE.backward (fms_mo/quant/quantizers.py:1044-1070): ``(grad_x, grad_clip_val)``."""
    cv = clip_val.to(x.dtype)
    n_levels = 2**num_bits - 1
    stepsize = 1.0 / (n_levels / cv)
    z = x / stepsize
    delz = (z - torch.round(z)) / n_levels
    ga = -grad_out * delz
    zeros = torch.zeros_like(grad_out)
    gx = torch.where(x <= 0, zeros, grad_out)
    gx = torch.where(x >= cv, zeros, gx)
    ga = torch.where(x <= 0, zeros, ga)
    ga = torch.where(x >= cv, grad_out, ga)
    return gx, ga.sum()


def pact_sym_fwd(x, clip_val, num_bits=8, intg_zp=True):
    """PACTplusSymSTE_rev1.forward, dequantize=True (fms_mo/quant/quantizers.py:1077-1116)."""
    cv = clip_val.to(x.dtype)
    n_levels = 2**num_bits - 2 if intg_zp else 2**num_bits - 1
    stepsize = 1.0 / (n_levels / (2 * cv))
    out = torch.where(x > cv, torch.ones_like(x) * cv, x)
    out = torch.where(out < -cv, torch.ones_like(x) * -cv, out)
    return torch.round((out + cv) / stepsize) * stepsize - cv


def pact_sym_bwd(x, grad_out, clip_val, num_bits=8, intg_zp=True):
    """PACTplusSymSTE_rev1.backward with out-of-range gradients clipped (fms_mo/quant/quantizers.py:1118-1154)."""
    cv = clip_val.to(x.dtype)
    n_levels = 2**num_bits - 2 if intg_zp else 2**num_bits - 1
    stepsize = 1.0 / (n_levels / (2 * cv))
    z = (x + cv) / stepsize
    delz = 2 * (torch.round(z) - z) / n_levels
    zeros = torch.zeros_like(grad_out)
    gx = torch.where(x <= -cv, zeros, grad_out)
    gx = torch.where(x >= cv, zeros, gx)
    ga = torch.ones_like(grad_out) * delz
    ga = torch.where(x <= -cv, -torch.ones_like(gx), ga)
    ga = torch.where(x >= cv, torch.ones_like(gx), ga)
    return gx, (ga * grad_out).sum()


# ---------------------------------------------------------------------------------------------
# FP8 scaling of the FP8 linear
# ---------------------------------------------------------------------------------------------
FP8_E4M3_MAX = 448.0
DL8_MIN = 0.0087890625


def fp8_dyn_quant(t: torch.Tensor, per_tensor: bool = False, dl8_flush: bool = False):
    """The scaling of LinearFuncFPxFwdBwd.forward (fms_mo/modules/linear.py:1939-1953):
    ``scale = clamp(amax / 448, 1e-5)`` along dim 1 (or the whole tensor), then
    ``(t / scale).to(float8_e4m3fn)``.  Returns ``(fp8 tensor, scale)``."""
    reduce_dim = None if per_tensor else 1
    scale = (t.abs().amax(dim=reduce_dim, keepdim=True) / FP8_E4M3_MAX).clamp(min=1e-5)
    q = (t / scale).to(torch.float8_e4m3fn)
    if dl8_flush:
        q32 = q.to(torch.float32)
        q32.masked_fill_(q32.abs() < DL8_MIN, 0)
        q = q32.to(torch.float8_e4m3fn)
    return q, scale
