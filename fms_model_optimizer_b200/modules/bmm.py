"""Quantized batched matmul: the step either side of the quantized Linears in an attention block.

``QBmm`` mirrors fms_mo/modules/bmm.py:26-228 (fake quantisation of both operands, then ``torch.matmul`` / ``torch.bmm``
exactly as the reference calls them); its quantizers are this package's CUDA kernels.  ``QBmmINT8Deploy`` mirrors
fms_mo/modules/bmm.py:607-758 with one difference the reference asks for itself ("Haven't implemented any batched
CUTLASS matmul, hence use torch.matmul to simulate"): the product of the int8 codes runs as an integer batched GEMM on
the tcgen05 kernels (``ops.bmm_i8``) instead of a float matmul on fp16 copies of the codes.  The value it returns is the
reference's: the exact integer sum rounded once to fp16 (what a float matmul with fp32 accumulation returns for sums
below 2^24), then the reference's own expression for scales and correction term, evaluated by the same PyTorch operators
so that every dtype promotion is the reference's.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import _lib as L
from .. import ops
from ..quant.quantizers import get_activation_quantizer


class _Bypass(nn.Module):
    """Qbypass (fms_mo/quant/quantizers.py): operands of 16 or 32 bits pass through."""

    def forward(self, x):
        return x


class QBmm(nn.Module):
    """Fake-quantized ``m1 @ m2`` (fms_mo/modules/bmm.py:26-228).  Constructor keywords, attribute and parameter names
    (``quantize_m1.clip_val`` ...) follow the reference, ``qcfg`` included.  Not provided: the calibration pass
    (``qmodel_calibration_new`` > 0, a ``Qdynamic`` observer) and quantizer modes outside this package's families
    (``pact+``, ``pactsym+``, ``max`` / ``maxsym``, ``fp8_*``); both raise at construction."""

    def __init__(self, num_bits_m1=32, qm1_mode=None, num_bits_m2=32, qm2_mode=None, m1_unidirectional=False,
                 m2_unidirectional=False, m1_bounded=False, m2_bounded=False, replaceBmm=True, **kwargs):  # fmt: skip
        super().__init__()
        qcfg = kwargs.pop("qcfg")
        self.replaceBmm = replaceBmm
        self.num_bits_m1 = num_bits_m1
        self.nbits_kvcache = kwargs.get("nbits_kvcache", num_bits_m2 if qcfg.get("nbits_kvcache", None) is None else qcfg.get("nbits_kvcache"))
        self.num_bits_m2 = self.nbits_kvcache
        self.m1_unidirectional, self.m2_unidirectional = m1_unidirectional, m2_unidirectional
        self.m1_bounded, self.m2_bounded = m1_bounded, m2_bounded
        self.qm1_mode, self.qm2_mode = qm1_mode, qm2_mode
        self.m1_clip_init_val = kwargs.get("m1_clip_init_val", qcfg.get("m1_clip_init_val", 1.0))
        self.m1_clip_init_valn = kwargs.get("m1_clip_init_valn", qcfg.get("m1_clip_init_valn", -1.0))
        self.m2_clip_init_val = kwargs.get("m2_clip_init_val", qcfg.get("m2_clip_init_val", 1.0))
        self.m2_clip_init_valn = kwargs.get("m2_clip_init_valn", qcfg.get("m2_clip_init_valn", -1.0))
        self.non_neg = kwargs.get("non_neg", qcfg.get("non_neg", False))
        self.align_zero = kwargs.get("align_zero", qcfg.get("align_zero", True))
        self.sym_7bits_bmm = kwargs.get("sym_7bits_bmm", qcfg.get("sym_7bits_bmm", False))
        self.extend_act_range = kwargs.get("extend_act_range", qcfg.get("extend_act_range", False))
        if qcfg.get("qmodel_calibration_new", 0) > 0:
            raise NotImplementedError("QBmm on B200: the calibration pass (qmodel_calibration_new > 0) is not provided")
        self.register_buffer("calib_counter", torch.tensor(0))
        self.register_buffer("num_module_called", torch.tensor(0))
        self.qcfg = qcfg
        self.symmetric = False
        if self.sym_7bits_bmm:
            if self.m1_unidirectional:
                self.num_bits_m1 -= 1
            elif self.m2_unidirectional:
                self.num_bits_m2 -= 1
            else:
                self.symmetric = True
                assert "sym" in qm1_mode and "sym" in qm2_mode, "should use one of the symmetric quantizers for qbmm modules"
        self.quantize_m1 = self._make(self.num_bits_m1, qm1_mode, m1_bounded, self.m1_clip_init_val, self.m1_clip_init_valn, m1_unidirectional)
        self.quantize_m2 = self._make(self.num_bits_m2, qm2_mode, m2_bounded, self.m2_clip_init_val, self.m2_clip_init_valn, m2_unidirectional)

    def _make(self, nbits, mode, bounded, cv, cvn, unidirectional):
        if nbits in (32, 16):
            return _Bypass()
        if bounded and "fp8" not in mode:
            raise NotImplementedError("QBmm on B200: bounded operands (the min-max quantizer) are not provided")
        return get_activation_quantizer(mode, nbits=nbits, clip_val=cv, clip_valn=cvn, non_neg=unidirectional, align_zero=self.align_zero,
                                        extend_act_range=bool(self.extend_act_range))  # fmt: skip

    def forward(self, m1, m2):
        qm1, qm2 = self.quantize_m1(m1), self.quantize_m2(m2)
        if self.replaceBmm:
            output = torch.matmul(qm1, qm2)
        else:
            org_batch_header = qm1.shape[:2]
            if len(qm1.shape) > 3:
                qm1 = qm1.reshape([-1, qm1.shape[-2], qm1.shape[-1]])
            if len(qm2.shape) > 3:
                qm2 = qm2.reshape([-1, qm2.shape[-2], qm2.shape[-1]])
            output = torch.bmm(qm1, qm2)
            output = output.reshape([*org_batch_header, *output.shape[1:]])
        self.num_module_called += 1
        return output

    def extra_repr(self):
        return f"nbits_m1,m2={self.num_bits_m1},{self.num_bits_m2}, qm1,qm2_mode={self.qm1_mode},{self.qm2_mode}"


class QBmmINT8Deploy(nn.Module):
    """INT8 ``m1 @ m2`` (fms_mo/modules/bmm.py:607-758): m1 treated as activations (asymmetric range stored as uint8
    codes minus 128), m2 as weights (symmetric), one static scale per operand.  Buffers (``m1_scale``, ``m1_zp``,
    ``m2_scale``, ``m2_zp``, ``m1_clip_val`` ...) carry the reference's names and values, so state dicts interchange."""

    def __init__(self):
        super().__init__()
        self.num_bits_m1 = self.num_bits_m2 = 8
        self.use_int_kernel = "b200"
        self.use_PT_native_Qfunc = False
        self._host = None

    @classmethod
    def from_fms_mo(cls, fms_mo_qbmm, **kwargs):
        """Same arithmetic on the clip values as fms_mo/modules/bmm.py:618-673.  ``fms_mo_qbmm`` is this package's QBmm or
        the reference's (only its attributes and quantizer parameters are read)."""
        assert fms_mo_qbmm.num_bits_m1 in [7, 8] and fms_mo_qbmm.num_bits_m2 == 8, "Only support 8bit QBmm!"
        target_device = kwargs.get("target_device", kwargs.get("device", next(fms_mo_qbmm.parameters()).device))
        qbmm_int = cls().to(target_device)
        qbmm_int.num_bits_m1, qbmm_int.num_bits_m2 = fms_mo_qbmm.num_bits_m1, fms_mo_qbmm.num_bits_m2
        qcfg = getattr(fms_mo_qbmm, "qcfg", None)
        qbmm_int.use_PT_native_Qfunc = qcfg.get("use_PT_native_Qfunc", False) if qcfg else False
        with torch.no_grad():
            Qa, Qw = fms_mo_qbmm.quantize_m1, fms_mo_qbmm.quantize_m2
            cvn_ext_ratio = 128 / 127
            if qbmm_int.num_bits_m1 == 7 or "sym" in fms_mo_qbmm.qm1_mode:
                Qa_cvn = -Qa.clip_val
            else:
                Qa_cvn = getattr(Qa, "clip_valn", torch.zeros_like(Qa.clip_val))
            m1_scale = (Qa.clip_val - Qa_cvn) / (2**Qa.num_bits - 1)
            m2_scale = Qw.clip_val * 2 / (2**Qw.num_bits - 2)
            qbmm_int.register_buffer("m1_scale", m1_scale.detach().clone())
            qbmm_int.register_buffer("m1_zp", torch.round(-Qa_cvn / m1_scale).to(torch.int))
            qbmm_int.register_buffer("m2_scale", m2_scale.detach().clone())
            qbmm_int.register_buffer("m2_zp", torch.zeros_like(m2_scale, dtype=torch.int))
            qbmm_int.register_buffer("m1_clip_val", Qa.clip_val.detach().clone())
            qbmm_int.register_buffer("m1_clip_valn", Qa_cvn.detach() * cvn_ext_ratio)
            qbmm_int.register_buffer("m2_clip_val", Qw.clip_val.detach().clone())
            qbmm_int.register_buffer("m2_clip_valn", -Qw.clip_val.detach() * cvn_ext_ratio)
        return qbmm_int.to(target_device)

    def _get_name(self):
        return "QBmmINT8Deploy"

    def extra_repr(self) -> str:
        return f"nbits_m1,m2={self.num_bits_m1},{self.num_bits_m2}, use_int_kernel={self.use_int_kernel}"

    def _host_scalars(self):
        """Scales and zero points as host numbers, read once per version of the buffers (the quantise kernel takes them
        as launch arguments)."""
        key = tuple((b.data_ptr(), b._version) for b in (self.m1_scale, self.m1_zp, self.m2_scale, self.m2_zp))
        if self._host is None or self._host[0] != key:
            self._host = (key, float(self.m1_scale.float().item()), int(self.m1_zp.item()) - 128, float(self.m2_scale.float().item()),
                          int(self.m2_zp.item()))  # fmt: skip
        return self._host[1:]

    def _codes(self, x, scale_t, scale, zp):
        """``clamp((x / scale + zp).round(), -128, 127).to(int8)`` (qfunc_raw, fms_mo/modules/bmm.py:690-702) over the rows of
        ``x``.  With an fp32 scale the division happens in fp32 whatever x's dtype (a one-element tensor is not a scalar for
        PyTorch's promotion) and the fused kernel applies; a 16-bit scale makes PyTorch round the quotient and the sum to
        16 bits, and the expression is then evaluated by the same PyTorch operators."""
        if scale_t.dtype == torch.float32 and x.dtype in (torch.float32, torch.float16, torch.bfloat16):
            rows = x.reshape(-1, x.shape[-1])
            codes, _, _ = ops.act_quant(rows, mode=L.Q_I8_STATIC, native_chain=0, scale0=scale, zp0=float(zp), shift=0.0)
            return codes.view(x.shape)
        zp_t = torch.tensor([zp], dtype=torch.int, device=x.device)
        return torch.clamp((x / scale_t + zp_t).round(), -128, 127).to(torch.int8)

    def forward(self, m1: torch.Tensor, m2: torch.Tensor) -> torch.Tensor:
        """``[..., m, k] @ [..., k, n] -> [..., m, n]`` with equal leading dimensions."""
        if not m1.is_cuda:
            raise RuntimeError("QBmmINT8Deploy runs on a CUDA device (there is no CPU fallback)")
        if m1.shape[:-2] != m2.shape[:-2] or m1.shape[-1] != m2.shape[-2]:
            raise RuntimeError("QBmmINT8Deploy takes m1 [..., m, k] and m2 [..., k, n] with equal leading dimensions")
        with torch.no_grad():
            s1, zp1, s2, zp2 = self._host_scalars()
            lead = m1.shape[:-2]
            m, k, n = m1.shape[-2], m1.shape[-1], m2.shape[-1]
            # m2 as [.., n, k] with k contiguous: free when m2 is the transposed view of a [.., n, k] tensor (q @ k^T)
            m2_nk = m2.transpose(-1, -2).contiguous()
            m1_i8 = self._codes(m1.contiguous(), self.m1_scale, s1, zp1)
            m2_i8_nk = self._codes(m2_nk, self.m2_scale, s2, zp2)
            acc = ops.bmm_i8(m1_i8.reshape(-1, m, k), m2_i8_nk.reshape(-1, n, k)).view(*lead, m, n)
            x = acc.to(torch.float16) * self.m1_scale * self.m2_scale
            if zp1 != 0:
                # the reference's correction term as it stands there (fms_mo/modules/bmm.py:741-746), the sum over
                # dimension 0 of m2's codes included
                m2_i8 = m2_i8_nk.transpose(-1, -2)
                corr_term = self.m1_scale.float() * (self.m1_zp - 128) * m2_i8.sum(dim=0) * self.m2_scale.float()
                x = x - corr_term
        return x.to(m1.dtype)
