"""Deploy-time quantized Linear modules on the B200 kernels.

``QLinearINT8Deploy`` and ``LinearFPxAcc`` keep the class names, constructors (``from_fms_mo``,
``from_torch_iW``, ``from_nn``), keyword arguments, buffer names and numerics of the modules they
stand in for (fms_mo/modules/linear.py:708-1338 and :1892-2124) but run their forward as two fused
kernels: one row-wise quantise pass and one tcgen05 GEMM with the dequantise chain in its epilogue.
There is no CPU path: the modules raise if their tensors are not on a CUDA device.
"""

from __future__ import annotations

import json
from typing import Optional

import torch
from torch import nn

from .. import _lib as L
from .. import ops
from ..quant.quantizers import get_activation_quantizer, get_weight_quantizer

_FLOATS = (torch.float32, torch.float16, torch.bfloat16)


def _promote(a: torch.dtype, b: torch.dtype) -> torch.dtype:
    return torch.promote_types(a, b)


class QLinearINT8Deploy(nn.Linear):
    """W8A8 integer Linear: quantise -> int8 GEMM -> dequantise, as one quantise kernel plus one GEMM.

    Mirrors QLinearINT8Deploy of the reference (fms_mo/modules/linear.py:708).  ``weight`` is int8
    ``[out, in]``; buffers ``input_scale, input_zp, w_scale, w_zp, smoothq_scale, corr_term, bias``
    carry the same values, so state dicts are interchangeable.  ``use_int_kernel`` is always
    ``"b200"``; chunked accumulation (``chunk_size``, ``truncate_lsb``, ``max_acc_bits``) is done
    inside the GEMM, as with the reference's ``"triton"`` setting."""

    @classmethod
    def from_fms_mo(cls, fms_mo_qlinear, **kwargs):
        """Converts a QLinear (the reference's, or any module with the same attributes) into a
        deploy module.  Same keyword arguments as the reference's from_fms_mo
        (fms_mo/modules/linear.py:717-920): ``max_acc_bits, truncate_lsb, chunk_size,
        use_dynamic_max_act_Qfunc, use_PT_native_Qfunc, recalc_clipvals, target_device``."""
        assert all(
            getattr(fms_mo_qlinear, a_or_w) in [4, 8] for a_or_w in ["num_bits_feature", "num_bits_weight"]
        ), "Please check nbits setting!"
        tar_dev = kwargs.get("target_device", kwargs.get("device", next(fms_mo_qlinear.parameters()).device))
        w_dtype = fms_mo_qlinear.weight.dtype
        q = cls(fms_mo_qlinear.in_features, fms_mo_qlinear.out_features, bias=fms_mo_qlinear.bias is not None, device="meta")
        q.use_int_kernel = "b200"
        q.usePTnativeQfunc = kwargs.get("use_PT_native_Qfunc", False)
        q.useDynMaxQfunc = kwargs.get("use_dynamic_max_act_Qfunc", False)
        q.useSymAct = "sym" in fms_mo_qlinear.qa_mode or fms_mo_qlinear.qa_mode in ["pertokenmax", "max"]
        q.max_acc_bits = kwargs.get("max_acc_bits", 32)
        q.truncate_lsb = kwargs.get("truncate_lsb", 0)
        q.chunk_size = kwargs.get("chunk_size", 100000)
        q.acc_dtype = torch.float16
        q.nbits_a = fms_mo_qlinear.num_bits_feature
        q.nbits_w = fms_mo_qlinear.num_bits_weight
        w_levels = 2**q.nbits_w - 2
        a_levels = 2**q.nbits_a - 1 - q.useSymAct

        with torch.no_grad():
            Qa = fms_mo_qlinear.quantize_feature
            Qw = fms_mo_qlinear.quantize_weight
            if kwargs.get("recalc_clipvals", True):
                Qw(fms_mo_qlinear.weight)
            w_cv = Qw.clip_val
            a_cv = getattr(Qa, "clip_val", torch.tensor(8.0, device=tar_dev))
            a_cvn = getattr(Qa, "clip_valn", torch.tensor(-8.0, device=tar_dev))
            q.cvs = [a_cv, a_cvn, w_cv]

            smoothq_scale = torch.tensor([1.0], device=tar_dev, dtype=w_dtype)
            if getattr(fms_mo_qlinear, "smoothq", False):
                a_scale = fms_mo_qlinear.smoothq_act_scale
                w_sq = fms_mo_qlinear.weight.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
                alpha = fms_mo_qlinear.smoothq_alpha
                if torch.all(a_scale != 0).item():
                    smoothq_scale = (a_scale**alpha / w_sq ** (1.0 - alpha)).clamp(min=1e-5).to(a_scale.dtype)

            input_scale = torch.tensor(1.0, device=tar_dev)
            w_scale = w_cv * 2 / w_levels
            q.use_fake_zero_shift = False
            if q.useDynMaxQfunc in [-1, -2]:
                input_zero_point = torch.tensor(128 - q.useSymAct, device=tar_dev)
            elif 0 < q.useDynMaxQfunc < 65:
                # per-tensor dynamic scale with a fake zero shift; the scale is computed at run time
                q.use_fake_zero_shift = True
                input_zero_point = torch.tensor(q.useDynMaxQfunc, device=tar_dev)
            elif q.usePTnativeQfunc:
                input_scale = torch.tensor([(a_cv - a_cvn) / a_levels], device=tar_dev)
                input_zero_point = torch.round(-a_cvn / input_scale)
            else:
                quant_scale = a_levels / torch.tensor([a_cv - a_cvn], device=tar_dev)
                quant_stepsize = 1.0 / quant_scale
                quant_zero_point = torch.round(a_cvn * quant_scale)
                input_scale = quant_stepsize
                input_zero_point = -quant_zero_point
                w_scale = 1.0 / (w_levels / (w_cv * 2))
                q.register_buffer("quant_scale", quant_scale)
                q.register_buffer("quant_stepsize", quant_stepsize)
                q.register_buffer("quant_zero_point", quant_zero_point)
            w_zp = torch.zeros_like(w_scale, dtype=torch.int)
            input_zero_point = input_zero_point.to(torch.int)
            q.register_buffer("input_scale", input_scale)
            q.register_buffer("input_zp", input_zero_point)
            q.register_buffer("w_scale", w_scale)
            q.register_buffer("w_zp", w_zp)
            q.register_buffer("smoothq_scale", smoothq_scale)

            if type(Qw).__name__ == "SAWB":
                Qw.dequantize = False
                w_int8 = Qw(fms_mo_qlinear.weight.float() * smoothq_scale)
            else:
                w_int8 = (
                    torch.round((fms_mo_qlinear.weight * smoothq_scale).t() / w_scale)
                    .clamp(-w_levels / 2, w_levels / 2)
                    .t()
                )
            w_int8 = w_int8.to(torch.int)
            q.weight = nn.Parameter(w_int8.to(torch.int8), requires_grad=False)

            if q.useSymAct:
                corr_term_int = 0
                if q.use_fake_zero_shift:
                    corr_term_int = input_zero_point * (w_int8.sum(dim=1))
            else:
                corr_term_int = (input_zero_point - 128) * (w_int8.sum(dim=1))
            q.register_buffer("corr_term", corr_term_int * w_scale.float() * input_scale.float())
            q.org_model_has_bias = fms_mo_qlinear.bias is not None
            if q.org_model_has_bias:
                new_bias = fms_mo_qlinear.bias.float() - q.corr_term
            else:
                new_bias = -q.corr_term
            if q.use_fake_zero_shift:
                new_bias += q.corr_term  # applied in forward, times the run-time input scale
            delattr(q, "bias")
            q.register_buffer("bias", new_bias.to(w_dtype))

        q.set_matmul_op()
        return q.to(tar_dev)

    @classmethod
    def from_torch_iW(cls, nnlin_iW, prec, a_cv, a_cvn, w_cv, zero_shift, **kwargs):
        """Builds a deploy module from an ``nn.Linear`` that already holds integer weights
        (fms_mo/modules/linear.py:922-1038): static per-tensor activation quantisation."""
        assert prec == "int8", "Only support INT8 for now."
        target_device = kwargs.get("target_device", kwargs.get("device", next(nnlin_iW.parameters()).device))
        q = cls(nnlin_iW.in_features, nnlin_iW.out_features, bias=nnlin_iW.bias is not None, device=target_device)
        q.nbits_a = 8
        q.nbits_w = 8
        q.acc_dtype = kwargs.get("acc_dtype", torch.float)
        q.usePTnativeQfunc = kwargs.get("use_PT_native_Qfunc", True)
        q.useDynMaxQfunc = False
        q.use_fake_zero_shift = False
        q.useSymAct = False
        q.use_int_kernel = "b200"
        q.weight = nn.Parameter(nnlin_iW.weight.to(torch.int8), requires_grad=False)
        q.max_acc_bits = kwargs.get("max_acc_bits", 32)
        q.truncate_lsb = kwargs.get("truncate_lsb", False)
        q.chunk_size = kwargs.get("chunk_size", 100000)
        with torch.no_grad():
            if q.usePTnativeQfunc:
                input_scale = torch.Tensor([(a_cv - a_cvn) / (2**q.nbits_a - 1)])
                input_zero_point = torch.round(-a_cvn / input_scale).to(torch.int)
                w_scale = torch.Tensor([w_cv * 2 / (2**q.nbits_w - 2)])
            else:
                quant_scale = (2**q.nbits_a - 1) / torch.Tensor([a_cv - a_cvn])
                quant_stepsize = 1.0 / quant_scale
                quant_zero_point = torch.round(a_cvn * quant_scale)
                input_scale = quant_stepsize
                input_zero_point = -quant_zero_point
                w_scale = 1.0 / ((2**q.nbits_a - 2) / torch.Tensor([w_cv * 2]))
                q.register_buffer("quant_scale", quant_scale)
                q.register_buffer("quant_stepsize", quant_stepsize)
                q.register_buffer("quant_zero_point", quant_zero_point)
            q.register_buffer("input_scale", input_scale)
            q.register_buffer("input_zp", input_zero_point)
            q.register_buffer("w_scale", w_scale)
            q.register_buffer("w_zp", torch.zeros_like(w_scale, dtype=torch.int))
            q.register_buffer("smoothq_scale", torch.tensor([1.0]))
            q.cvs = [a_cv, a_cvn, w_cv]
            zero_s = torch.Tensor(json.loads(zero_shift)) if isinstance(zero_shift, str) else torch.Tensor([zero_shift])
            corr_term = (input_zero_point - 128) * zero_s * w_scale * input_scale
            q.register_buffer("corr_term", corr_term)
            q.register_buffer("zero_shift", zero_s)
            if nnlin_iW.bias is not None:
                q.bias = nn.Parameter((nnlin_iW.bias - corr_term.to(target_device)).to(q.acc_dtype), requires_grad=False)
                q.org_mod_has_bias = True
            else:
                delattr(q, "bias")
                q.register_buffer("bias", -corr_term.to(q.acc_dtype))
                q.org_mod_has_bias = False
        q.set_matmul_op()
        return q.to(target_device)

    # ------------------------------------------------------------------------------------------
    def set_matmul_op(self):
        """The reference picks and registers its matmul callable here (fms_mo/modules/linear.py:1213);
        on B200 the only kernel is ``torch.ops.qlin_b200.imatmul``."""
        self.imatmul = torch.ops.qlin_b200.imatmul
        self._cache = None

    def _prepared(self, dev: torch.device):
        """fp32 views of the per-channel vectors the kernels take, rebuilt when buffers move."""
        bufs = (self.w_scale, self.bias, self.smoothq_scale)
        # in-place updates (load_state_dict, buffer.copy_) keep the address and bump the version counter
        key = tuple((b.data_ptr(), b._version, b.dtype) for b in bufs) + (str(dev),)
        if self._cache is None or self._cache[0] != key:
            sq = self.smoothq_scale
            use_sq = bool(torch.all(sq != 1).item())
            self._cache = (
                key,
                dict(
                    w_scale=self.w_scale.detach().float().reshape(-1).contiguous(),
                    bias=self.bias.detach().float().reshape(-1).contiguous(),
                    smooth=(sq.detach().float().reshape(-1).contiguous() if use_sq else None),
                    smooth_rcp=(ops.smooth_reciprocal(sq.detach().float()) if use_sq else None),
                ),
            )
        return self._cache[1]

    def _get_name(self):
        return "QLinear_INT8"

    def extra_repr(self) -> str:
        s = f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}, int_kernel={self.use_int_kernel}"
        if self.truncate_lsb > 0 or self.max_acc_bits < 32:
            s += f", acc_bits={self.max_acc_bits}, trun_lsb={self.truncate_lsb}"
        return s

    def __getstate__(self):
        state = self.__dict__.copy()
        state.pop("imatmul", None)
        state["_cache"] = None
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self.set_matmul_op()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """QLinearINT8Deploy.forward + iaddmm_int (fms_mo/modules/linear.py:1309-1338, :1115-1188).
        The dtype in which each step of the reference's eager chain would run is worked out from
        the dtypes of ``x`` and of the buffers, and the kernels round at the same places."""
        if not x.is_cuda:
            raise RuntimeError("QLinearINT8Deploy(b200) runs on CUDA tensors only")
        with torch.no_grad():
            org_dtype = x.dtype
            tar_shape = tuple(x.shape[:-1]) + (self.weight.shape[0],)
            x2 = x.reshape(-1, x.shape[-1])
            prep = self._prepared(x.device)
            smooth = prep["smooth"]
            chain = x2.dtype if smooth is None else _promote(x2.dtype, self.smoothq_scale.dtype)
            kw = {}
            # `x / smoothq_scale` is rounded to the dtype of x when the scale has that dtype (or promotes to it); the
            # static quantisers then divide by their fp32 scale buffers in fp32 (fms_mo/modules/linear.py:1330, :1061-1083)
            smooth_native = 1 if (smooth is not None and chain == x2.dtype and chain != torch.float32) else 0
            if self.useDynMaxQfunc in [-1, -2]:
                if self.useDynMaxQfunc == -2:
                    raise NotImplementedError("per-channel (dim=-2) dynamic activation quantisation")
                # qa_dynamic_max_qfunc runs in `chain`; bit 0: the division by smoothq_scale rounds to
                # the dtype of x, bit 1: the quantise chain does
                native = smooth_native | (2 if (chain == x2.dtype and chain != torch.float32) else 0)
                if smooth is None or self.smoothq_scale.dtype == x2.dtype:
                    native |= 4  # the smoothing scales are values of the activation dtype
                codes, in_scale, _ = ops.act_quant(
                    x2, mode=L.Q_I8_DYN, smooth=smooth, smooth_rcp=prep["smooth_rcp"], native_chain=native,
                    levels=2 ** (self.nbits_a - 1) - 1
                )
                scale_dtype = chain
            elif self.use_fake_zero_shift:
                # qa_dyn_max_fake_zero_shift (fms_mo/modules/linear.py:1102-1113): one scale for the whole tensor,
                # amax / (127 - zp), codes shifted by zp; the largest per-row scale is that scale (rounding is monotonic)
                zp = int(self.input_zp)
                native = smooth_native | (2 if (chain == x2.dtype and chain != torch.float32) else 0)
                if smooth is None or self.smoothq_scale.dtype == x2.dtype:
                    native |= 4
                kq = dict(smooth=smooth, smooth_rcp=prep["smooth_rcp"], native_chain=native)
                _, row_scale, _ = ops.act_quant(x2, mode=L.Q_I8_DYN, levels=2 ** (self.nbits_a - 1) - 1 - zp, want_codes=False, **kq)
                in_scale = row_scale.max().reshape(1)
                codes, _, _ = ops.act_quant(x2, mode=L.Q_I8_GIVEN_SCALE, scale_in=in_scale, zp0=float(zp), **kq)
                # iaddmm_int (:1179-1182): bias - input_scale * corr_term, formed in fp32
                kw["bias"] = prep["bias"] - in_scale * self.corr_term.detach().float().reshape(-1)
                scale_dtype = self.w_scale.dtype if self.w_scale.dim() > 0 else chain  # a 0-dim scale takes the other operand's dtype
            elif self.usePTnativeQfunc:
                # qa_raw_qfunc divides by the input_scale buffer: the chain runs in the promoted dtype of the two, which is
                # the dtype of x for a module converted from a 16-bit model (its scale buffers carry the model's dtype)
                st = _promote(chain, self.input_scale.dtype)
                smooth_native |= 2 if (st == x2.dtype and st != torch.float32) else 0
                codes, in_scale, _ = ops.act_quant(
                    x2, mode=L.Q_I8_STATIC, smooth=smooth, smooth_rcp=prep["smooth_rcp"], native_chain=smooth_native,
                    scale0=float(self.input_scale), zp0=float(self.input_zp), shift=128.0, add2=float(self.useSymAct),
                )  # fmt: skip
                in_scale = self.input_scale.detach().float().reshape(-1)
                scale_dtype = self.input_scale.dtype
            else:
                st = _promote(chain, self.quant_stepsize.dtype)
                smooth_native |= 2 if (st == x2.dtype and st != torch.float32) else 0
                codes, in_scale, _ = ops.act_quant(
                    x2, mode=L.Q_I8_STATIC_CLAMP_FIRST, smooth=smooth, smooth_rcp=prep["smooth_rcp"], native_chain=smooth_native,
                    scale0=float(self.quant_stepsize), zp0=float(self.quant_zero_point), lo=float(self.cvs[1]), hi=float(self.cvs[0]),
                    shift=float(128 - self.useSymAct),
                )  # fmt: skip
                in_scale = self.input_scale.detach().float().reshape(-1)
                scale_dtype = self.input_scale.dtype
            prod_dtype = _promote(scale_dtype, self.w_scale.dtype)
            out = ops.gemm(
                codes, self.weight,
                chunk_k=_normalised_chunk(self.chunk_size), trun_bits=int(self.truncate_lsb), max_acc_bits=self.max_acc_bits,
                epilogue=L.EPI_SCALE_PROD, row_scale=in_scale, col_scale=prep["w_scale"], bias=kw.pop("bias", prep["bias"]),
                prod_round=(None if prod_dtype == torch.float32 else prod_dtype), scale_round=torch.float16,
                acc_round=(None if self.acc_dtype == torch.float32 else self.acc_dtype), out_dtype=org_dtype, **kw,
            )  # fmt: skip
            return out.reshape(tar_shape)


def _normalised_chunk(chunk_size: int) -> int:
    """Chunk size as tl_matmul_chunk_truncate normalises it for 8-bit operands
    (fms_mo/custom_ext_kernels/triton_kernels.py:550-555)."""
    pow2 = chunk_size > 0 and (chunk_size & (chunk_size - 1)) == 0
    return max(chunk_size, 32) if pow2 else 32


def _fp8_chunk(chunk_size):
    chunk = _normalised_chunk(int(chunk_size)) if int(chunk_size) != 8 else 8
    if chunk == 8:
        raise NotImplementedError("chunk_size=8 is provided by ops.tl_matmul_chunk_truncate only")
    return chunk


class _LinearFPxFwdBwd(torch.autograd.Function):
    """LinearFuncFPxFwdBwd (fms_mo/modules/linear.py:1892-2058).  Forward: e4m3 codes of x and W with per-token /
    per-channel or per-tensor scales, fp32-accumulating tcgen05 GEMM with optional chunk truncation, ``* x_scale * w_scale``
    and bias in the epilogue.  Backward (per-tensor scaling only, as in the reference, whose per-token branch cannot
    broadcast its scales): e5m2 codes of x, W and grad_output with one scale each, two e5m2 GEMMs; the bias gradient is the
    column sum of the scaled e5m2 gradient codes, which is what the reference returns."""

    @staticmethod
    def forward(ctx, x, weight, bias, trun_bits, chunk_size, fp8_dyn, clamp_acc_to_dl16, wq_ws):
        org_dtype = x.dtype
        tar_shape = x.shape[:-1] + (weight.shape[0],)
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.cfg = (trun_bits, chunk_size, fp8_dyn, bool(clamp_acc_to_dl16), bias.dtype if bias is not None else None)
        native = 0 if org_dtype == torch.float32 else 3
        if fp8_dyn == "per_token":
            xq, xs, _ = ops.act_quant(x2, mode=L.Q_F8_DYN, native_chain=native, dl8_flush=clamp_acc_to_dl16)
            wq, ws = wq_ws
        else:
            xq, xs = ops.fp8_quant_per_tensor(x2, dl8_flush=clamp_acc_to_dl16)
            wq, ws = ops.fp8_quant_per_tensor(weight.detach(), dl8_flush=clamp_acc_to_dl16)
        rnd = None if org_dtype == torch.float32 else org_dtype
        out = ops.gemm(
            xq, wq, chunk_k=_fp8_chunk(chunk_size), trun_bits=(14 if clamp_acc_to_dl16 else int(trun_bits)),
            clamp_dl16=bool(clamp_acc_to_dl16), epilogue=L.EPI_SCALE_SEQ, row_scale=xs, col_scale=ws,
            bias=(bias.detach().to(org_dtype) if bias is not None else None), mid_round=rnd, acc_round=rnd, out_dtype=org_dtype,
        )  # fmt: skip
        return out.reshape(tar_shape)

    @staticmethod
    def backward(ctx, grad_output):
        x2, weight = ctx.saved_tensors
        trun_bits, chunk_size, fp8_dyn, dl16, bias_dtype = ctx.cfg
        if fp8_dyn != "per_tensor":
            raise NotImplementedError("the backward of the FP8 Linear runs with dynamic_fp8='per_tensor' only (so does the reference's)")
        dtype_input = x2.dtype
        out_dim, in_dim = weight.shape
        g2 = grad_output.reshape(-1, out_dim).to(dtype_input)
        xq, xs = ops.fp8_quant_per_tensor(x2, e5m2=True, eps=0.0, dl8_flush=dl16)
        wq, ws = ops.fp8_quant_per_tensor(weight.detach(), e5m2=True, eps=0.0, dl8_flush=dl16)
        gq, gs = ops.fp8_quant_per_tensor(g2, e5m2=True, eps=0.0, dl8_flush=dl16)
        kw = dict(chunk_k=_fp8_chunk(chunk_size), trun_bits=(14 if dl16 else int(trun_bits)), clamp_dl16=dl16, epilogue=L.EPI_SCALE_SEQ)

        def t8(c):  # both GEMM operands are K-major: transpose the one-byte codes
            return c.view(torch.uint8).t().contiguous().view(torch.float8_e5m2)

        # grad_weight[n, k] = sum_m g[m, n] x[m, k];  grad_input[m, k] = sum_n g[m, n] w[n, k]
        grad_weight = ops.gemm(t8(gq), t8(xq), row_scale=gs, col_scale=xs, out_dtype=weight.dtype, **kw)
        grad_input = ops.gemm(gq, t8(wq), row_scale=gs, col_scale=ws, out_dtype=dtype_input, **kw)
        grad_input = grad_input.reshape(grad_output.shape[:-1] + (in_dim,))
        grad_bias = gq.float().sum(0).to(bias_dtype) if bias_dtype is not None else None
        return grad_input, grad_weight, grad_bias, None, None, None, None, None


class LinearFPxAcc(nn.Linear):
    """FP8 Linear with dynamic scales and optional reduced-precision accumulation, mirroring LinearFPxAcc /
    LinearFuncFPxFwdBwd of the reference (fms_mo/modules/linear.py:1892-2124): e4m3 forward with per-token / per-channel
    scales (W's codes cached until the weight changes) or per-tensor scales, e5m2 backward with per-tensor scales."""

    @classmethod
    def from_nn(cls, nnlin, trun_bits=0, **kwargs):
        target_device = kwargs.get("target_device", kwargs.get("device", next(nnlin.parameters()).device))
        lin = cls(nnlin.in_features, nnlin.out_features, bias=nnlin.bias is not None, device="meta")
        lin.weight = nnlin.weight
        lin.trun_bits = trun_bits
        lin.chunk_size = kwargs.get("chunk_size", False)
        lin.fp8_dyn = kwargs.get("dynamic_fp8", False)
        lin.clamp_acc_to_dl16 = kwargs.get("clamp_acc_to_dl16", False)
        lin._wq = None
        if nnlin.bias is not None:
            lin.bias = nnlin.bias
        return lin.to(target_device)

    def _quantised_weight(self):
        w = self.weight
        key = (w.data_ptr(), w._version, w.dtype, str(w.device))
        if getattr(self, "_wq", None) is None or self._wq[0] != key:
            native = 0 if w.dtype == torch.float32 else 3
            wq, ws, _ = ops.act_quant(w.detach(), mode=L.Q_F8_DYN, native_chain=native, dl8_flush=self.clamp_acc_to_dl16)
            self._wq = (key, wq, ws)
        return self._wq[1], self._wq[2]

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if not inputs.is_cuda:
            raise RuntimeError("LinearFPxAcc(b200) runs on CUDA tensors only")
        if self.fp8_dyn not in ("per_token", "per_tensor"):
            raise NotImplementedError("the B200 FP8 Linear provides dynamic_fp8='per_token' or 'per_tensor'")
        assert inputs.dtype in _FLOATS
        wq_ws = self._quantised_weight() if self.fp8_dyn == "per_token" else None
        return _LinearFPxFwdBwd.apply(inputs, self.weight, self.bias, self.trun_bits, self.chunk_size, self.fp8_dyn,
                                      self.clamp_acc_to_dl16, wq_ws)  # fmt: skip

    def extra_repr(self) -> str:
        s = f"{self.in_features},{self.out_features}"
        if self.bias is not None:
            s += f",bias={self.bias is not None}"
        if self.trun_bits > 0:
            s += f",trun_bits={self.trun_bits}"
        if self.fp8_dyn:
            s += f",fp8_dyn={self.fp8_dyn}"
        if self.clamp_acc_to_dl16:
            s += ",use_DL16_acc"
        return s + f",chunk_size={self.chunk_size}"


class QLinearCublasI8I32NT(nn.Linear):
    """Static per-tensor activation quantisation, int8 x int8 -> int32 GEMM, ``input_scale * w_scale * acc + bias``
    (QLinearCublasI8I32NT of the reference, fms_mo/modules/linear.py:1341-1537; the GEMM replaces
    ``mygemm::gemm_nt_i8i32`` / ``cutlass_gemm::i8i32nt``).  ``weight`` is int8 ``[out, in]``; with uint8
    activations the zero-point correction ``w_scale * input_scale * (zp - 128) * sum_k W`` is folded into ``bias``."""

    @classmethod
    def from_reference(cls, ref_qlinear, input_scale, input_zero_point, input_dtype, forceSymA=False):
        """fms_mo/modules/linear.py:1349-1426: from a ``torch.ao.nn.quantized.reference.Linear`` with per-channel weight
        quantisation.  uint8 activations are either made symmetric (``forceSymA``: a new scale ``2 max|range| / 253``, zero
        point 0) or kept, with the zero-point correction folded into the bias."""
        q = cls(ref_qlinear.in_features, ref_qlinear.out_features)
        q.forceSymA = forceSymA
        q.input_dtype = input_dtype
        q.register_buffer("input_scale", input_scale)
        q.register_buffer("input_zp", input_zero_point)
        qweight = ref_qlinear.float().get_quantized_weight()
        if ref_qlinear.weight_qscheme not in [torch.per_channel_symmetric, torch.per_channel_affine]:
            raise RuntimeError("QLinear_cublas only supports perCh for now. ")
        q.register_buffer("w_scale", qweight.q_per_channel_scales().float())
        q.register_buffer("w_zp", qweight.q_per_channel_zero_points())
        q.weight = nn.Parameter(qweight.int_repr(), requires_grad=False)
        q.bias = nn.Parameter(ref_qlinear.bias, requires_grad=False)
        if input_dtype == torch.quint8:
            if forceSymA:
                a_min = -input_zero_point * input_scale
                a_max = (255 - input_zero_point) * input_scale
                a_max_new = max(abs(a_min), abs(a_max))
                q.input_scale.copy_((2 * a_max_new) / (255 - 2))
                q.input_zp.copy_(0)
                q.input_dtype = torch.qint8
            else:
                corr_term = q.w_scale * input_scale * (input_zero_point - 128) * q.weight.sum(dim=1)
                q.bias = nn.Parameter(ref_qlinear.bias - corr_term.to(ref_qlinear.bias.dtype), requires_grad=False)
        return q

    @classmethod
    def from_fms_mo(cls, fms_mo_qlinear, **kwargs):
        """fms_mo/modules/linear.py:1427-1490: activation scale / zero point from the PACT clip values, per-channel
        weight scale ``clip * 2 / (2^b - 2)``, integer weights from the weight quantizer run without dequantisation."""
        assert fms_mo_qlinear.num_bits_feature in [4, 8] and fms_mo_qlinear.num_bits_weight in [4, 8], "Please check nbits setting!"
        target_device = kwargs.get("target_device", next(fms_mo_qlinear.parameters()).device)
        q = cls(fms_mo_qlinear.in_features, fms_mo_qlinear.out_features, device="meta")
        q.input_dtype = torch.quint8
        q.forceSymA = False
        with torch.no_grad():
            # The handful of scalar / per-channel conversions run on the host: torch's CUDA kernels divide
            # by a Python scalar through its reciprocal, the CPU kernels (and IEEE) divide.
            Qa = fms_mo_qlinear.quantize_feature
            a_cv, a_cvn = Qa.clip_val.detach().cpu(), Qa.clip_valn.detach().cpu()
            input_scale = (a_cv - a_cvn) / (2**Qa.num_bits - 1)
            input_zero_point = torch.round(-a_cvn / input_scale).to(torch.int)
            q.register_buffer("input_scale", input_scale)
            q.register_buffer("input_zp", input_zero_point)
            Qw = fms_mo_qlinear.quantize_weight
            w_scale = Qw.clip_val.detach().cpu() * 2 / (2**Qw.num_bits - 2)
            q.register_buffer("w_scale", w_scale.float())
            q.register_buffer("w_zp", torch.zeros_like(w_scale, dtype=torch.int))
            Qw.dequantize = False
            q.weight = nn.Parameter(Qw(fms_mo_qlinear.weight.float()).to(torch.int8), requires_grad=False)
            corr_term = q.w_scale * input_scale * (input_zero_point - 128) * q.weight.sum(dim=1).cpu()
            corr_term = corr_term.to(fms_mo_qlinear.bias.dtype)
            q.bias = nn.Parameter(fms_mo_qlinear.bias.detach().cpu() - corr_term, requires_grad=False)
        return q.to(target_device)

    def _get_name(self):
        return "QuantizedLinear_cublasi8i32"

    def _quantise(self, x2):
        native = 3 if (x2.dtype != torch.float32 and self.input_scale.dtype == x2.dtype) else 0
        if not hasattr(self, "_host_scalars"):  # read once: the module's scale and zero point never change
            self._host_scalars = (float(self.input_scale.reshape(-1)[0].item()), float(self.input_zp.reshape(-1)[0].item()))
        s0, zp0 = self._host_scalars
        lo, hi, shift = (0.0, 255.0, 128.0) if self.input_dtype == torch.quint8 else (-127.0, 127.0, 0.0)
        codes, _, _ = ops.act_quant(x2, mode=L.Q_I8_STATIC_ROUND_FIRST, native_chain=native, scale0=s0, zp0=zp0, lo=lo, hi=hi, shift=shift)
        return codes

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            in_dtype = x.dtype
            if in_dtype not in _FLOATS:
                raise RuntimeError(f"unsupported activation dtype {in_dtype}")
            tar_shape = x.shape[:-1] + (self.weight.shape[0],)
            codes = self._quantise(x.reshape(-1, x.shape[-1]))
            out = ops.gemm(codes, self.weight, epilogue=L.EPI_SCALE_PROD, row_scale=self.input_scale.reshape(-1)[:1],
                           col_scale=self.w_scale, bias=self.bias, out_dtype=in_dtype)  # fmt: skip
        return out.reshape(tar_shape)


class QLinearCutlassI8I32NT(QLinearCublasI8I32NT):
    """fms_mo/modules/linear.py:1540-1583: the same module; both of the reference's library GEMMs are
    replaced by the one tcgen05 GEMM here."""

    def _get_name(self):
        return "QuantizedLinear_cutlassi8i32"


class _LinearINT8FwdFP32Bwd(torch.autograd.Function):
    """LinearFuncINT8FwdFP32Bwd (fms_mo/modules/linear.py:2127-2223): forward through the int8 chunk-
    truncating GEMM with per-token / per-channel max scales (no lower clamp on the scales), backward
    with plain matmuls in the activation dtype."""

    @staticmethod
    def forward(ctx, x, weight, bias, lsb_trun_bits, chunk_size, max_acc_bits):
        assert x.dtype in _FLOATS
        org_dtype = x.dtype
        tar_shape = x.shape[:-1] + (weight.shape[0],)
        x2 = x.reshape(-1, x.shape[-1])
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.save_for_backward(x2, weight)
        native = 0 if org_dtype == torch.float32 else 3
        xq, xs, _ = ops.act_quant(x2, mode=L.Q_I8_DYN, native_chain=native, dyn_eps=0.0)
        wn = 0 if weight.dtype == torch.float32 else 3
        wq, ws, _ = ops.act_quant(weight.detach(), mode=L.Q_I8_DYN, native_chain=wn, dyn_eps=0.0)
        rnd = None if org_dtype == torch.float32 else org_dtype
        out = ops.gemm(
            xq, wq, chunk_k=_normalised_chunk(int(chunk_size)), trun_bits=int(lsb_trun_bits), max_acc_bits=int(max_acc_bits),
            epilogue=L.EPI_SCALE_SEQ, row_scale=xs, col_scale=ws, bias=(bias.detach().to(org_dtype) if bias is not None else None),
            mid_round=rnd, acc_round=rnd, out_dtype=org_dtype,
        )  # fmt: skip
        return out.reshape(tar_shape)

    @staticmethod
    def backward(ctx, grad_output):
        x2, weight = ctx.saved_tensors
        dtype_grad = x2.dtype
        g2 = grad_output.reshape(-1, weight.shape[0]).to(dtype_grad)
        grad_weight = torch.matmul(g2.transpose(0, 1).contiguous(), x2.to(dtype_grad)).to(weight.dtype)
        grad_input = torch.matmul(g2, weight.to(dtype_grad)).reshape(grad_output.shape[:-1] + (weight.shape[1],)).to(x2.dtype)
        grad_bias = g2.sum(0).to(ctx.bias_dtype) if ctx.has_bias else None
        return grad_input, grad_weight, grad_bias, None, None, None


class QLinearINT8Train(nn.Linear):
    """Linear that runs its forward on the int8 GEMM (with optional LSB truncation / narrow
    accumulator) and its backward in floating point: QLinearINT8Train of the reference
    (fms_mo/modules/linear.py:2227-2285)."""

    @classmethod
    def from_fms_mo(cls, nnlin, lsb_trun_bits=0, **kwargs):
        target_device = kwargs.get("target_device", kwargs.get("device", next(nnlin.parameters()).device))
        lin = cls(nnlin.in_features, nnlin.out_features, bias=nnlin.bias is not None, device="meta")
        lin.weight = nnlin.weight
        lin.lsb_trun_bits = lsb_trun_bits
        lin.chunk_size = kwargs.get("chunk_size", 64)
        lin.max_acc_bits = kwargs.get("max_acc_bits", 32)
        if nnlin.bias is not None:
            lin.bias = nnlin.bias
        return lin.to(target_device)

    def forward(self, inputs):
        return _LinearINT8FwdFP32Bwd.apply(inputs, self.weight, self.bias, self.lsb_trun_bits, self.chunk_size, self.max_acc_bits)

    def extra_repr(self) -> str:
        s = f"{self.in_features},{self.out_features},bias={self.bias is not None},chunk_size={self.chunk_size}"
        if self.lsb_trun_bits > 0:
            s += f",lsb_trun={self.lsb_trun_bits}"
        if self.max_acc_bits < 32:
            s += f",max_acc_bits={self.max_acc_bits}"
        return s


class QLinear(nn.Linear):
    """Fake-quant Linear for QAT / DQ (fms_mo/modules/linear.py:51-393, forward :248-305):
    ``F.linear(Qa(x / s), Qw(W * s), bias)`` with the SmoothQuant scale ``s`` of :345-368.  The two
    quantizers run as single CUDA kernels (forward and backward); the matmul itself stays a plain
    library GEMM, as in the reference."""

    def __init__(self, in_features, out_features, bias=True, num_bits_feature=32, qa_mode=None, num_bits_weight=32,
                 qw_mode=None, **kwargs):  # fmt: skip
        super().__init__(in_features, out_features, bias, device=kwargs.get("device", "cuda"))
        qcfg = kwargs.pop("qcfg", {})
        self.num_bits_feature = num_bits_feature
        self.num_bits_weight = num_bits_weight
        self.qa_mode = qa_mode
        self.qw_mode = qw_mode
        self.act_clip_init_val = kwargs.get("act_clip_init_val", qcfg.get("act_clip_init_val", 8.0))
        self.act_clip_init_valn = kwargs.get("act_clip_init_valn", qcfg.get("act_clip_init_valn", -8.0))
        self.non_neg = kwargs.get("non_neg", False)
        self.align_zero = kwargs.get("align_zero", qcfg.get("align_zero", True))
        self.register_buffer("num_module_called", torch.tensor(0))
        self.quantize_feature = nn.Identity()
        if num_bits_feature not in [32, 16]:
            self.quantize_feature = get_activation_quantizer(
                qa_mode, nbits=num_bits_feature, clip_val=self.act_clip_init_val, clip_valn=self.act_clip_init_valn,
                non_neg=self.non_neg, align_zero=self.align_zero,
            )  # fmt: skip
        self.quantize_weight = nn.Identity()
        if num_bits_weight not in [32, 16]:
            self.quantize_weight = get_weight_quantizer(
                qw_mode, nbits=num_bits_weight, align_zero=self.align_zero, w_shape=self.weight.shape
            )
        self.smoothq = qcfg.get("smoothq", False)
        if self.smoothq:
            self.register_buffer("smoothq_act_scale", torch.zeros(self.weight.shape[1], device=self.weight.device))
            self.register_buffer(
                "smoothq_alpha",
                torch.tensor([qcfg.get("smoothq_alpha", 0.5)], dtype=torch.float32, device=self.weight.device),
            )
        self._sq_is_zero = None
        # the quantizers create their clip values on the CPU; keep them with the weight
        self.quantize_feature.to(self.weight.device)
        self.quantize_weight.to(self.weight.device)

    def set_act_scale(self, act_scale):
        assert act_scale.shape[0] == self.weight.shape[1], "scale applies to per-channel"
        self.smoothq_act_scale.copy_(act_scale)
        self._sq_is_zero = None

    def get_smoothq_scale(self, x):
        if self._sq_is_zero is None:  # resolved once, not with a device sync in every forward
            self._sq_is_zero = self.smoothq_act_scale.sum().item() == 0.0
        if self._sq_is_zero:
            return torch.tensor([1.0]).to(x.dtype).to(x.device)
        weight_scale = self.weight.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
        alpha = float(self.smoothq_alpha.item()) if isinstance(self.smoothq_alpha, torch.Tensor) else self.smoothq_alpha
        return (self.smoothq_act_scale.pow(alpha) / weight_scale.pow(1.0 - alpha)).clamp(min=1e-5).to(x.dtype)

    def forward(self, x):
        if self.smoothq:
            scale = self.get_smoothq_scale(x)
            qinput = self.quantize_feature(x / scale).to(x.dtype)
            qweight = self.quantize_weight(self.weight * scale).to(self.weight.dtype)
        else:  # the reference divides and multiplies by a tensor holding 1.0 here: the identity, bit for bit
            qinput = self.quantize_feature(x).to(x.dtype)
            qweight = self.quantize_weight(self.weight).to(self.weight.dtype)
        output = nn.functional.linear(qinput, qweight, self.bias)
        self.num_module_called += 1
        return output


def lower_qmodel_b200(model: nn.Module, use_dyn_max_act=False, max_acc_bits=32, clamp_acc_to_dl16=False,
                      num_lsb_to_truncate=0, chunk_size=32, layer_to_exclude=None):  # fmt: skip
    """In-place lowering with the signature of lower_qmodel_triton
    (fms_mo/custom_ext_kernels/utils.py:869-959): every QLinear (this package's, or the reference's --
    matched by class name so the reference need not be importable) becomes a QLinearINT8Deploy, every
    plain ``nn.Linear`` a LinearFPxAcc with per-token (``use_dyn_max_act`` -1 / -2) or per-tensor FP8 scaling.
    With ``use_dyn_max_act=False`` the reference would run plain Linears through its 16-bit truncating matmul; the
    B200 FP8 Linear has no unscaled mode, so those layers are left as they are (they stay ``nn.Linear``)."""
    fp_dyn = "per_token" if use_dyn_max_act in [-1, -2] else "per_tensor" if use_dyn_max_act else False
    if layer_to_exclude is None:
        layer_to_exclude = []
    elif isinstance(layer_to_exclude, str):
        layer_to_exclude = [layer_to_exclude]
    elif not isinstance(layer_to_exclude, (list, tuple)):
        raise RuntimeError("layer_to_exclude has to be either str, list, or tuple.")
    for name, m in list(model.named_modules()):
        is_q = type(m).__name__ == "QLinear"
        if not (is_q or type(m) is nn.Linear) or name in layer_to_exclude:
            continue
        if not is_q and not fp_dyn:
            continue
        parent_name, _, module_name = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        if is_q:
            new_lin = QLinearINT8Deploy.from_fms_mo(
                m, use_int_kernel="b200", use_dynamic_max_act_Qfunc=use_dyn_max_act, max_acc_bits=max_acc_bits,
                truncate_lsb=num_lsb_to_truncate, chunk_size=chunk_size,
            )  # fmt: skip
        else:
            new_lin = LinearFPxAcc.from_nn(
                m, trun_bits=num_lsb_to_truncate, chunk_size=chunk_size, dynamic_fp8=fp_dyn,
                clamp_acc_to_dl16=clamp_acc_to_dl16,
            )  # fmt: skip
        setattr(parent, module_name, new_lin)
    return model
