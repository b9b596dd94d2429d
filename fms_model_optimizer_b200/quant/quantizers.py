"""QAT / DQ quantizer modules on the B200 kernels.

Same class names, constructor arguments and ``clip_val`` / ``clip_valn`` attribute names as the
quantizers they stand in for (fms_mo/quant/quantizers.py), restricted to the ones on the quantized
Linear's path: PACT2 with PACT+ gradients (activations), SAWB+ per channel and Qmax per channel
(weights), QMaxDynamic / PerTokenMax (dynamic per-token activations).  Forward and backward run as
single CUDA kernels; there is no CPU path.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import _lib as L
from .. import ops

SAWB_COEFFS = {8: (31.76, -35.04), 4: (12.035, -12.03), 2: (2.6, -1.71)}  # codes 803 / 403 / 103


class PACTplus2STE(torch.autograd.Function):
    """PACT+ two-sided fake quantisation with straight-through gradients
    (fms_mo/quant/quantizers.py:1949-2102), dequantize=True."""

    @staticmethod
    def forward(ctx, input_tensor, clip_val, clip_valn, num_bits, dequantize, inplace, intg_zp, use_PT_native_Qfunc):
        if not dequantize or use_PT_native_Qfunc or inplace or intg_zp not in (0, 1, False, True):
            raise NotImplementedError("PACTplus2STE on B200: dequantize=True, align_zero in {0,1}, out of place only")
        ctx.save_for_backward(input_tensor, clip_val, clip_valn)
        ctx.num_bits = num_bits
        ctx.align_zero = bool(intg_zp)
        return ops.pact2_fwd(input_tensor, clip_val, clip_valn, num_bits, bool(intg_zp))

    @staticmethod
    def backward(ctx, grad_output):
        x, clip_val, clip_valn = ctx.saved_tensors
        gx, gclip = ops.pact2_bwd(x, grad_output, clip_val, clip_valn, ctx.num_bits, ctx.align_zero)
        ga = gclip[0].to(clip_val.dtype).expand_as(clip_val)
        gan = gclip[1].to(clip_valn.dtype).expand_as(clip_valn)
        return gx.view_as(x), ga, gan, None, None, None, None, None


class PACT2(nn.Module):
    """Two-sided PACT (fms_mo/quant/quantizers.py:1397-1484) with the PACT+ gradient rule."""

    def __init__(self, num_bits, init_clip_valn=-8.0, init_clip_val=8.0, dequantize=True, inplace=False,
                 cggrad=False, pcq_w=False, grad_scale=False, pact_plus=False, **kwargs):  # fmt: skip
        super().__init__()
        if cggrad or pcq_w or grad_scale or not pact_plus:
            raise NotImplementedError("PACT2 on B200 provides the pact_plus=True quantizer")
        self.num_bits = num_bits
        if isinstance(init_clip_val, torch.Tensor) and isinstance(init_clip_valn, torch.Tensor):
            self.clip_val = nn.Parameter(init_clip_val)
            self.clip_valn = nn.Parameter(init_clip_valn)
        elif not isinstance(init_clip_val, torch.Tensor) and not isinstance(init_clip_valn, torch.Tensor):
            self.clip_val = nn.Parameter(torch.Tensor([init_clip_val]))
            self.clip_valn = nn.Parameter(torch.Tensor([init_clip_valn]))
        else:
            raise ValueError("FMS: init_clip_val and init_clip_valn  should be the same instance type.")
        self.dequantize = dequantize
        self.inplace = inplace
        self.pact_plus = pact_plus
        self.align_zero = kwargs.get("align_zero", False)
        self.use_PT_native_Qfunc = kwargs.get("use_PT_native_Qfunc", False)
        self.quantizer = PACTplus2STE

    def forward(self, input_tensor):
        return self.quantizer.apply(input_tensor, self.clip_val, self.clip_valn, self.num_bits, self.dequantize,
                                    self.inplace, self.align_zero, self.use_PT_native_Qfunc)  # fmt: skip

    def __repr__(self):
        return (f"{self.__class__.__name__}(num_bits={self.num_bits}, pos-clip={self.clip_val[0]:.4f}, "
                f"neg-clip={self.clip_valn[0]:.4f},quantizer={self.quantizer})")  # fmt: skip


class _PactOneClipSTE(torch.autograd.Function):
    """One-sided PACT+ (PACTplusSTE, fms_mo/quant/quantizers.py:1016-1070) and symmetric PACT+
    (PACTplusSymSTE_rev1, :1073-1154): a single learnable clip value."""

    @staticmethod
    def forward(ctx, input_tensor, clip_val, num_bits, variant, intg_zp):
        ctx.save_for_backward(input_tensor, clip_val)
        ctx.cfg = (num_bits, variant, bool(intg_zp))
        return ops.pact2_fwd(input_tensor, clip_val, None, num_bits, bool(intg_zp), variant)

    @staticmethod
    def backward(ctx, grad_output):
        x, clip_val = ctx.saved_tensors
        num_bits, variant, intg_zp = ctx.cfg
        gx, gclip = ops.pact2_bwd(x, grad_output, clip_val, None, num_bits, intg_zp, variant)
        return gx.view_as(x), gclip[0].to(clip_val.dtype).expand_as(clip_val), None, None, None


class PACT(nn.Module):
    """One-sided PACT with the PACT+ gradient rule (fms_mo/quant/quantizers.py:791-844), for
    non-negative activations."""

    def __init__(self, num_bits, init_clip_val, init_clip_valn=0, dequantize=True, inplace=False, cggrad=False,
                 grad_scale=False, pact_plus=False):  # fmt: skip
        super().__init__()
        if cggrad or grad_scale or not pact_plus or not dequantize or inplace:
            raise NotImplementedError("PACT on B200 provides the pact_plus=True, dequantize=True quantizer")
        self.num_bits = num_bits
        self.clip_val = nn.Parameter(init_clip_val if isinstance(init_clip_val, torch.Tensor) else torch.Tensor([init_clip_val]))
        self.dequantize = dequantize
        self.inplace = inplace
        self.quantizer = _PactOneClipSTE

    def forward(self, input_tensor):
        return self.quantizer.apply(input_tensor, self.clip_val, self.num_bits, L.PACT_ONE_SIDED, False)


class PACTplusSym(nn.Module):
    """Two-sided symmetric PACT+ (fms_mo/quant/quantizers.py:1247-1304)."""

    def __init__(self, num_bits, init_clip_val, dequantize=True, inplace=False, intg_zp=False, OORgradnoclip=False,
                 extend_act_range=False):  # fmt: skip
        super().__init__()
        if extend_act_range or OORgradnoclip or not dequantize or inplace:
            raise NotImplementedError("PACTplusSym on B200: dequantize=True, out-of-range gradients clipped")
        self.num_bits = num_bits
        self.clip_val = nn.Parameter(init_clip_val if isinstance(init_clip_val, torch.Tensor) else torch.Tensor([init_clip_val]))
        self.dequantize = dequantize
        self.inplace = inplace
        self.intg_zp = intg_zp
        self.OORgradnoclip = OORgradnoclip
        self.quantizer = _PactOneClipSTE
        self.quantizer_name = "PACT+sym"

    def forward(self, input_tensor):
        return self.quantizer.apply(input_tensor, self.clip_val, self.num_bits, L.PACT_SYMMETRIC, self.intg_zp)


class _PerChSTE(torch.autograd.Function):
    """Per-channel symmetric fake quantisation with identity gradient: the quantise step of
    SAWBPlusZeroPerChSTE (fms_mo/quant/quantizers.py:503-572) and QmaxPerChSTE (:3190-3224)."""

    @staticmethod
    def forward(ctx, w, num_bits, mode, clip_buf, dequantize):
        c0, c1 = SAWB_COEFFS.get(num_bits, (0.0, 0.0))
        w2 = w.reshape(w.shape[0], -1)
        dq, codes, clip = ops.weight_fq_perch(
            w2, num_bits=num_bits, mode=mode, clip=(clip_buf if mode == L.W_GIVEN else None), want_dq=dequantize,
            want_codes=not dequantize, c0=c0, c1=c1,
            clip_dtype=(clip_buf.dtype if mode == L.W_GIVEN else None),
        )  # fmt: skip
        if mode != L.W_GIVEN:
            clip_buf.copy_(clip.to(clip_buf.dtype))
        return dq.view_as(w) if dequantize else codes.view_as(w)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output.clone(), None, None, None, None


class _PerTensorSTE(torch.autograd.Function):
    """Per-tensor symmetric fake quantisation with identity gradient: SAWBPlusZeroSTE
    (fms_mo/quant/quantizers.py:455-500) and QmaxSTE (:3159-3187)."""

    @staticmethod
    def forward(ctx, x, num_bits, mode, clip_buf, dequantize, align_zero):
        c0, c1 = SAWB_COEFFS.get(num_bits, (0.0, 0.0))
        if mode == L.W_SAWB and num_bits not in SAWB_COEFFS:
            mode = L.W_MAX
        out, clip = ops.tensor_fq(
            x, kind=L.PT_INT_SYM, mode=mode, num_bits=num_bits, clip=(clip_buf if mode == L.W_GIVEN else None),
            align_zero=align_zero, dequantize=dequantize, c0=c0, c1=c1,
        )  # fmt: skip
        if mode != L.W_GIVEN:
            clip_buf.copy_(clip.to(clip_buf.dtype))
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None, None, None, None, None


class SAWB(nn.Module):
    """SAWB+ with zero alignment (fms_mo/quant/quantizers.py:377-452), per output channel
    (SAWBPlusZeroPerChSTE, :503-572) or per tensor (SAWBPlusZeroSTE, :455-500): in training mode the
    clip value is recomputed from mean|w| and sqrt(mean w^2), in eval mode the stored ``clip_val`` is used."""

    def __init__(self, num_bits, dequantize=True, inplace=False, align_zero=False, clipSTE=True, perCh=False, interp=False):
        super().__init__()
        if num_bits not in [2, 4, 8]:
            raise ValueError("FMS: SAWB supports 2, 4, and 8-bit quantization only.")
        if not (clipSTE and align_zero) or inplace:
            raise NotImplementedError("SAWB on B200 provides the sawb+ quantizers (clipSTE, align_zero)")
        self.num_bits = num_bits
        self.dequantize = dequantize
        self.inplace = inplace
        self.align_zero = align_zero
        self.clipSTE = clipSTE
        self.perCh = perCh
        self.interp = interp
        self.quantizer = _PerChSTE if perCh else _PerTensorSTE
        self.register_buffer("clip_val", torch.zeros(perCh) if perCh else torch.Tensor([0.0]))

    def forward(self, input_tensor: torch.Tensor) -> torch.Tensor:
        mode = L.W_SAWB if self.training else L.W_GIVEN
        if self.perCh:
            return self.quantizer.apply(input_tensor, self.num_bits, mode, self.clip_val, self.dequantize)
        return self.quantizer.apply(input_tensor, self.num_bits, mode, self.clip_val, self.dequantize, True)

    def __repr__(self):
        return f"{self.__class__.__name__}(num_bits={self.num_bits}, quantizer={self.quantizer})"


class Qmax(nn.Module):
    """Symmetric max quantizer (fms_mo/quant/quantizers.py:2990-3141), per output channel (QmaxPerChSTE,
    :3190-3224) or per tensor (QmaxSTE, :3159-3187): training uses the fresh absmax and keeps a moving
    average (factor 0.1) in ``clip_val``; eval uses the stored value."""

    def __init__(self, num_bits, dequantize=True, inplace=False, align_zero=False, clipSTE=True, minmax=False,
                 perCh=None, perGp=None, extend_act_range=False):  # fmt: skip
        super().__init__()
        if minmax or perGp or extend_act_range or inplace or (perCh and not dequantize):
            raise NotImplementedError("Qmax on B200 provides the symmetric per-channel and per-tensor quantizers")
        self.num_bits = num_bits
        self.dequantize = dequantize
        self.align_zero = align_zero
        self.perCh = perCh
        self.movAvgFac = 0.1
        self.Niter = 0
        self.quantizer_name = "Qmax"
        self.register_buffer("clip_val", torch.zeros(perCh) if perCh else torch.Tensor([0.0]))
        self.register_buffer("clip_valn", torch.zeros(perCh) if perCh else torch.Tensor([0.0]))

    def _quantise(self, x, mode, clip):
        if self.perCh:
            return _PerChSTE.apply(x, self.num_bits, mode, clip, True)
        return _PerTensorSTE.apply(x, self.num_bits, mode, clip, self.dequantize, self.align_zero)

    def forward(self, input_tensor):
        if self.training:
            fresh = torch.empty_like(self.clip_val, dtype=torch.float32)
            out = self._quantise(input_tensor, L.W_MAX, fresh)
            with torch.no_grad():
                new = fresh.to(input_tensor.dtype)
                if self.Niter == 0:
                    self.clip_val.copy_(new)
                    self.clip_valn.copy_(-new)
                self.clip_val.copy_(self.clip_val * (1.0 - self.movAvgFac) + new * self.movAvgFac)
                self.clip_valn.copy_(self.clip_valn * (1.0 - self.movAvgFac) + (-new) * self.movAvgFac)
        else:
            out = self._quantise(input_tensor, L.W_GIVEN, self.clip_val)
        self.Niter += 1
        return out

    def __repr__(self):
        return f"Qmax(num_bits={self.num_bits}, " + (f"per channel of {self.perCh})" if self.perCh else "per tensor)")


class QMaxDynamic(nn.Module):
    """Dynamic symmetric per-token fake quantisation (fms_mo/quant/quantizers.py:3504-3537):
    ``x.div(s).round().mul(s)`` with ``s = clamp(amax, 1e-5) / levels`` along the last dimension."""

    def __init__(self, num_bits, dim=-1):
        super().__init__()
        self.num_bits = num_bits
        self.levels = 2 ** (self.num_bits - 1) - 1
        if dim not in (-1, "perToken", "per_token", "per_Token"):
            raise NotImplementedError("QMaxDynamic on B200 reduces over the last dimension (per token)")
        self.reduce_dim = -1

    def forward(self, input_tensor):
        x2 = input_tensor.reshape(-1, input_tensor.shape[-1])
        native = 0 if x2.dtype == torch.float32 else 3
        _, _, dq = ops.act_quant(x2, mode=L.Q_I8_DYN, native_chain=native, levels=self.levels, want_codes=False, want_dq=True)
        return dq.view_as(input_tensor)

    def __repr__(self):
        return f"{self.__class__.__name__}(num_bits={self.num_bits}, quantizer=)"


class PerTokenMax(QMaxDynamic):
    """fms_mo/quant/quantizers.py:3479-3501: same arithmetic as QMaxDynamic; also records the
    per-token clip values."""

    def __init__(self, num_bits):
        super().__init__(num_bits, -1)
        self.register_buffer("clip_val", torch.Tensor([0.0]))
        self.register_buffer("clip_valn", torch.Tensor([0.0]))


class _Fp8FakeSTE(torch.autograd.Function):
    """e4m3 quantise-dequantise with identity gradient."""

    @staticmethod
    def forward(ctx, x, variant):
        if variant == "row":
            x2 = x.reshape(-1, x.shape[-1])
            native = 0 if x2.dtype == torch.float32 else 3
            _, _, dq = ops.act_quant(x2, mode=L.Q_F8_FAKE_SCALED, native_chain=native, want_codes=False, want_dq=True,
                                     dyn_eps=1e-12)  # fmt: skip
            return dq.view_as(x)
        if variant == "tensor":
            return ops.tensor_fq(x, kind=L.PT_F8_SCALED, mode=L.W_MAX)[0]
        return ops.tensor_fq(x, kind=L.PT_F8_SAT, mode=L.W_GIVEN)[0]

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


class to_fp8(nn.Module):  # noqa: N801  (the reference's class name)
    """FP8 e4m3 quantise-dequantise in the tensor dtype (fms_mo/quant/quantizers.py:5422-5488 with
    to_fp8_saturated / to_fp8_scaled / to_fp8_scaled_perCh / to_fp8_scaled_perToken, :5316-5420):
    ``emulate=True`` only.  The reference's e5m2 branch cannot be constructed (it names a dtype that
    does not exist), so only e4m3 is provided."""

    def __init__(self, n_bits: int = 8, q_mode: str = "fp8_e4m3_sat", perCh=None, perToken: bool = False, emulate: bool = True):
        super().__init__()
        assert n_bits == 8, "only for 8-bit floating point conversion"
        if "e4m3" not in q_mode:
            raise ValueError("FP8 on B200 provides e4m3 (the reference's e5m2 quantizer cannot be constructed)")
        if not emulate:
            raise NotImplementedError("to_fp8 on B200 provides emulate=True; real FP8 tensors come from LinearFPxAcc")
        self.q_mode = q_mode
        self.float8_dtype = torch.float8_e4m3fn
        self.emulate = emulate
        self.perCh = perCh
        self.perToken = perToken
        self.register_buffer("scale", torch.zeros(perCh) if perCh else torch.Tensor([0.0]))

    def forward(self, x: torch.Tensor):
        if self.perCh:
            if x.dim() != 2:
                raise RuntimeError("per-channel FP8 quantisation expects a [out, in] weight")
            return _Fp8FakeSTE.apply(x, "row")
        if self.perToken:
            return _Fp8FakeSTE.apply(x, "row")
        if "_sat" in self.q_mode:
            return _Fp8FakeSTE.apply(x, "sat")
        if "_scale" in self.q_mode:
            return _Fp8FakeSTE.apply(x, "tensor")
        return None

    def __repr__(self):
        return f"{self.__class__.__name__}(q_mode={self.q_mode}, emulate={self.emulate})"


def get_activation_quantizer(qa_mode="pact+", nbits=8, clip_val=None, clip_valn=None, non_neg=False, align_zero=True, **_):
    """Subset of get_activation_quantizer (fms_mo/quant/quantizers.py:46-226) for the modes on the
    quantized Linear's path."""
    if qa_mode == "pact+" and non_neg:
        return PACT(nbits, init_clip_val=clip_val, init_clip_valn=clip_valn, dequantize=True, inplace=False, pact_plus=True)
    if qa_mode == "pactsym+":
        return PACTplusSym(nbits, init_clip_val=clip_val, dequantize=True, inplace=False, intg_zp=align_zero)
    if qa_mode == "pact+" and not non_neg:
        return PACT2(nbits, init_clip_valn=clip_valn, init_clip_val=clip_val, dequantize=True, inplace=False,
                     pact_plus=True, align_zero=align_zero)  # fmt: skip
    if "max" in qa_mode and ("pertoken" in qa_mode or "perToken" in qa_mode):
        return QMaxDynamic(nbits, dim=-1)
    if "max" in qa_mode and "min" not in qa_mode and "per_channel" not in qa_mode and "perCh" not in qa_mode:
        return Qmax(nbits, align_zero=True if "sym" in qa_mode else align_zero, minmax=False)
    if "fp8" in qa_mode and "custom" not in qa_mode:
        return to_fp8(nbits, q_mode=qa_mode, perToken="perToken" in qa_mode, emulate=True)
    raise NotImplementedError(f"activation quantizer {qa_mode!r} is not on the B200 quantized-Linear path")


def get_weight_quantizer(qw_mode="sawb+", nbits=8, w_shape=None, align_zero=True, clip_val=None, **_):
    """Subset of get_weight_quantizer (fms_mo/quant/quantizers.py:229-374)."""
    cout = w_shape[0] if w_shape is not None else None
    if "sawb" in qw_mode and "+" in qw_mode and "interp" not in qw_mode:
        return SAWB(nbits, dequantize=True, inplace=False, align_zero=True, clipSTE=True, perCh=cout if "perCh" in qw_mode else False)
    if "max" in qw_mode and "min" not in qw_mode and "perGp" not in qw_mode:
        return Qmax(nbits, align_zero=align_zero, minmax=False, perCh=cout if "perCh" in qw_mode else None)
    if qw_mode == "pact+":
        return PACTplusSym(nbits, init_clip_val=clip_val, dequantize=True, inplace=False, intg_zp=align_zero)
    if "fp8" in qw_mode and "custom" not in qw_mode:
        return to_fp8(nbits, q_mode=qw_mode, emulate=True, perCh=cout if "perCh" in qw_mode else False)
    raise NotImplementedError(f"weight quantizer {qw_mode!r} is not on the B200 quantized-Linear path")
