"""CPU restatement of the quantized batched matmul (fms_mo/modules/bmm.py).  Test infrastructure only: nothing in the
package may import it.  Pinned bit for bit against outputs of the reference itself (tests/golden/bmm.pt, made by
tests/golden/make_golden.py::gen_bmm).
"""

from __future__ import annotations

import torch

from . import quantizers as OQ


def fake_quant_operand(x: torch.Tensor, mode: str, num_bits: int, clip_val: torch.Tensor, clip_valn, one_sided: bool, align_zero: bool = True):
    """The activation quantizer QBmm picks for an operand (fms_mo/modules/bmm.py:137-147 through
    get_activation_quantizer, fms_mo/quant/quantizers.py:80-107, 155-163): one-sided PACT+, two-sided PACT+ or
    symmetric PACT+."""
    if num_bits in (16, 32):
        return x
    if mode == "pactsym+":
        return OQ.pact_sym_fwd(x, clip_val, num_bits, intg_zp=align_zero)
    if mode == "pact+" and one_sided:
        return OQ.pact_one_sided_fwd(x, clip_val, num_bits)
    if mode == "pact+":
        return OQ.pact2plus_fwd(x, clip_val, clip_valn, num_bits, align_zero)
    raise NotImplementedError(mode)


def qbmm_fake(m1, m2, q1: dict, q2: dict, replace_bmm: bool = True):
    """QBmm.forward (fms_mo/modules/bmm.py:183-226): quantise both operands, then matmul, or bmm on the operands
    flattened to three dimensions."""
    qm1 = fake_quant_operand(m1, **q1)
    qm2 = fake_quant_operand(m2, **q2)
    if replace_bmm:
        return torch.matmul(qm1, qm2)
    head = qm1.shape[:2]
    if qm1.dim() > 3:
        qm1 = qm1.reshape(-1, qm1.shape[-2], qm1.shape[-1])
    if qm2.dim() > 3:
        qm2 = qm2.reshape(-1, qm2.shape[-2], qm2.shape[-1])
    out = torch.bmm(qm1, qm2)
    return out.reshape(*head, *out.shape[1:])


def deploy_buffers(clip_val1, clip_valn1, num_bits1: int, mode1: str, clip_val2, num_bits2: int):
    """QBmmINT8Deploy.from_fms_mo (fms_mo/modules/bmm.py:645-671): scales and zero points from the clip values.
    ``num_bits1`` is the quantizer's own width (7 when a one-sided m1 gave up a bit)."""
    cvn = -clip_val1 if (num_bits1 == 7 or "sym" in mode1) else (clip_valn1 if clip_valn1 is not None else torch.zeros_like(clip_val1))
    m1_scale = (clip_val1 - cvn) / (2**num_bits1 - 1)
    m2_scale = clip_val2 * 2 / (2**num_bits2 - 2)
    return dict(m1_scale=m1_scale, m1_zp=torch.round(-cvn / m1_scale).to(torch.int), m2_scale=m2_scale,
                m2_zp=torch.zeros_like(m2_scale, dtype=torch.int), m1_clip_val=clip_val1, m1_clip_valn=cvn * (128 / 127),
                m2_clip_val=clip_val2, m2_clip_valn=-clip_val2 * (128 / 127))  # fmt: skip


def qfunc_raw(x, scale, zp):
    """fms_mo/modules/bmm.py:690-702."""
    return torch.clamp((x / scale + zp).round(), -128, 127).to(torch.int8)


def qbmm_int8_deploy(m1, m2, buf: dict):
    """QBmmINT8Deploy.forward (fms_mo/modules/bmm.py:719-752).  The reference multiplies fp16 copies of the codes; the
    restatement sums the integer products exactly and rounds the sum once to fp16, which is what a float matmul
    with fp32 accumulation returns while the sums stay below 2^24 (sums beyond 65504 become infinities in both).
    The correction term keeps the reference's sum over dimension 0 of m2's codes."""
    m1_i8 = qfunc_raw(m1, buf["m1_scale"], buf["m1_zp"] - 128)
    m2_i8 = qfunc_raw(m2, buf["m2_scale"], buf["m2_zp"])
    acc = torch.matmul(m1_i8.double(), m2_i8.double())
    corr_term = buf["m1_scale"].float() * (buf["m1_zp"] - 128) * m2_i8.sum(dim=0) * buf["m2_scale"].float()
    x = acc.to(torch.float16) * buf["m1_scale"] * buf["m2_scale"] - corr_term
    return x.to(m1.dtype)
