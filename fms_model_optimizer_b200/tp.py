"""W8A8 Linear layers sharded column- or row-parallel across the GPUs of one node.

The sharding follows the tables the reference registers for its int8 Linear
(fms_mo/aiu_addons/i8i8/i8i8_aiu_linear.py:304-389): a column-parallel layer splits the output
features (int8 weight rows, per-channel weight scales, bias) and replicates the SmoothQuant scale;
a row-parallel layer splits the input features (weight columns and the SmoothQuant scale),
replicates the weight scales and keeps the bias on rank 0.  One process drives one GPU; the only
data-path collectives are the ones at the shard boundary of a row-parallel layer:

  * an all-reduce(MAX) of the per-token quantisation scales ([tokens] fp32), so that the int8
    activation codes are the ones the unsharded layer would produce, and
  * an all-reduce(SUM) of the dequantised partial outputs.

Everything else is the single-GPU path of ``ops``: one row-quantise kernel and one tcgen05 GEMM with
the dequantise epilogue per layer.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops


def shard_range(total: int, world: int, rank: int) -> slice:
    """Contiguous equal split; ``total`` must divide by ``world``."""
    if total % world != 0:
        raise ValueError(f"cannot shard {total} over {world} ranks")
    step = total // world
    return slice(rank * step, (rank + 1) * step)


def shard_w8a8(weight_i8: torch.Tensor, w_scale: torch.Tensor, smooth: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               mode: str, world: int, rank: int):
    """Returns this rank's ``(weight, w_scale, smooth, bias)`` of an unsharded W8A8 Linear.
    ``mode`` is ``"column"`` (split out features), ``"row"`` (split in features) or ``"replicate"``."""
    if mode == "replicate" or world == 1:
        return weight_i8, w_scale, smooth, bias
    n, k = weight_i8.shape
    if mode == "column":
        r = shard_range(n, world, rank)
        return weight_i8[r].contiguous(), w_scale[r].contiguous(), smooth, (bias[r].contiguous() if bias is not None else None)
    if mode == "row":
        r = shard_range(k, world, rank)
        return (weight_i8[:, r].contiguous(), w_scale, (smooth[r].contiguous() if smooth is not None else None),
                (bias if rank == 0 else None))  # fmt: skip
    raise ValueError(f"unknown shard mode {mode!r}")


class ScaleExchange:
    """How the shards of a row-parallel Linear agree on the per-token scales without a collective: every shard stores
    the scales of its slice of the row into slot ``rank`` of a ``[world][tokens]`` fp32 array on every GPU (plain stores
    to the peers' arenas, or one ``multimem.st`` when ``bases`` holds the arena's multicast address), and after the
    flag barrier each shard takes the maximum over the slots."""

    def __init__(self, barrier, bases, slots_off: int, rank: int, slots: torch.Tensor, multimem: bool = False):
        self.barrier, self.bases, self.slots_off, self.rank, self.slots, self.multimem = barrier, bases, slots_off, rank, slots, multimem


class W8A8Linear:
    """A (possibly sharded) W8A8 Linear with per-token dynamic activation quantisation, SmoothQuant
    and per-channel weight scales: the arithmetic of QLinearINT8Deploy.forward
    (fms_mo/modules/linear.py:1309-1338, :1115-1188) for bf16 / fp16 activations.

    ``quant_fn`` / ``gemm_fn`` default to the CUDA kernels; tests of the sharding logic on CPU ranks
    substitute the oracle's arithmetic."""

    def __init__(self, weight_i8, w_scale, smooth=None, bias=None, mode="replicate", group=None,
                 quant_fn: Optional[Callable] = None, gemm_fn: Optional[Callable] = None):  # fmt: skip
        self.weight = weight_i8
        # dtype the reference's buffer would have: `input_scale * w_scale` is formed in the promoted
        # dtype of the two before it is cast to fp16 (linear.py:1186)
        self.w_scale_dtype = w_scale.dtype
        self.w_scale = w_scale.float().contiguous()
        self.smooth = smooth.float().contiguous() if smooth is not None else None
        self.smooth_rcp = ops.smooth_reciprocal(self.smooth) if (self.smooth is not None and self.smooth.is_cuda) else None
        # true when every smoothing scale is a bf16 value (the reference casts it to the activation dtype)
        self.smooth_is_bf16 = bool(((self.smooth.view(torch.int32) & 0xFFFF) == 0).all().item()) if self.smooth is not None else True
        self.bias = bias.float().contiguous() if bias is not None else None
        self.mode = mode
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None or (dist.is_available() and dist.is_initialized())) else 1
        self.quant_fn = quant_fn or _cuda_quant
        self.gemm_fn = gemm_fn or _cuda_gemm
        self.max_ctas = None  # cap on the GEMM's grid (None: ops.GEMM_MAX_CTAS), set by a caller that overlaps streams

    def _q(self, x2, given_scale):
        if self.quant_fn is _cuda_quant:
            return _cuda_quant(x2, self.smooth, given_scale, self.smooth_rcp, self.smooth_is_bf16)
        return self.quant_fn(x2, self.smooth, given_scale)

    def quantise(self, x2: torch.Tensor):
        """Per-token int8 codes and scales of ``x2 / smooth``.  For a row-parallel shard the scale is
        the maximum over the ranks, which is the unsharded layer's scale."""
        if self.mode == "row" and self.world > 1:
            _, scale = self._q(x2, None)
            dist.all_reduce(scale, op=dist.ReduceOp.MAX, group=self.group)
            codes, _ = self._q(x2, scale)
            return codes, scale
        return self._q(x2, None)

    def quantise_fused(self, x2: torch.Tensor, prologue: int = L.BLOCK_PLAIN, r: Optional[torch.Tensor] = None, exchange=None,
                       keep_h: Optional[list] = None):
        """Per-token codes and scales of ``prologue(x2, r) / smooth`` for bf16 rows through the fused kernel
        (``ops.block_quant``); a row-parallel shard takes two passes around the MAX all-reduce of the scales.
        ``exchange`` (a ``ScaleExchange``) replaces that all-reduce: the first pass stores this shard's scales into slot
        ``rank`` on every GPU, and after the barrier the second pass takes the maximum over the slots itself.
        ``keep_h``: a list that receives the bf16 row the Linear sees (``prologue(x2, r)``), for tests."""
        rcp = [self.smooth_rcp]
        want_h = keep_h is not None
        if exchange is not None:
            T = x2.shape[0]
            world = exchange.barrier.arena.world
            ops.block_quant(x2, prologue=prologue, r=r, smooth_rcps=rcp, mode=L.BLOCK_SCALE_ONLY,
                            dst=(exchange.bases, [0], [exchange.slots_off + exchange.rank * T * 4], 0), dst_multimem=exchange.multimem)
            exchange.barrier.wait()
            (codes,), (scale,), _, h = ops.block_quant(x2, prologue=prologue, r=r, smooth_rcps=rcp, mode=L.BLOCK_GIVEN_SCALE,
                                                       scale_in=exchange.slots, scale_in_parts=world, scale_in_stride=T, want_h=want_h)
            if want_h:
                keep_h.append(h)
            return codes, scale
        if self.mode == "row" and self.world > 1:
            _, (scale,), _, _ = ops.block_quant(x2, prologue=prologue, r=r, smooth_rcps=rcp, mode=L.BLOCK_SCALE_ONLY)
            dist.all_reduce(scale, op=dist.ReduceOp.MAX, group=self.group)
            (codes,), _, _, h = ops.block_quant(x2, prologue=prologue, r=r, smooth_rcps=rcp, mode=L.BLOCK_GIVEN_SCALE, scale_in=scale,
                                                want_h=want_h)
            if want_h:
                keep_h.append(h)
            return codes, scale
        (codes,), (scale,), _, h = ops.block_quant(x2, prologue=prologue, r=r, smooth_rcps=rcp, want_h=want_h)
        if want_h:
            keep_h.append(h)
        return codes, scale

    def scatter(self, quantised, bases, rows_per_rank: int, row0: int, act_dtype: torch.dtype) -> None:
        """Row-parallel shard without a collective: the GEMM epilogue stores the partial output rows of token block
        ``i`` into ``bases[i]`` (rank i's receive buffer, mapped through ``peer.PeerArena``) at row ``row0`` onwards.
        The owner of a token block later sums the ``world`` partials (``ops.block_quant`` with ``r_parts``)."""
        codes, scale = quantised
        prod_dtype = torch.promote_types(act_dtype, self.w_scale_dtype)
        kw = {} if self.gemm_fn is not _cuda_gemm else {"max_ctas": self.max_ctas}
        self.gemm_fn(codes, self.weight, scale, self.w_scale, self.bias, act_dtype, prod_dtype, scatter=(bases, rows_per_rank, row0), **kw)

    def __call__(self, x2: Optional[torch.Tensor], quantised=None, act_dtype: Optional[torch.dtype] = None,
                 reduce: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``quantised=(codes, scale)`` skips the quantiser (a fused kernel upstream produced them for the
        activation dtype ``act_dtype``; for a row-parallel shard the scale must already be the maximum over ranks).
        ``reduce=False`` returns a row-parallel shard's partial output (the caller exchanges it)."""
        codes, scale = quantised if quantised is not None else self.quantise(x2)
        act_dtype = act_dtype if x2 is None else x2.dtype
        prod_dtype = torch.promote_types(act_dtype, self.w_scale_dtype)
        kw = {} if self.gemm_fn is not _cuda_gemm else {"max_ctas": self.max_ctas}
        if out is not None:
            kw["out"] = out
        out = self.gemm_fn(codes, self.weight, scale, self.w_scale, self.bias, act_dtype, prod_dtype, **kw)
        if reduce and self.mode == "row" and self.world > 1:
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out


def _cuda_quant(x2, smooth, given_scale, smooth_rcp=None, smooth_is_bf16=False):
    native = 0 if x2.dtype == torch.float32 else 3
    if x2.dtype == torch.bfloat16 and smooth_is_bf16:
        native |= 4
    if given_scale is None:
        codes, scale, _ = ops.act_quant(x2, mode=L.Q_I8_DYN, smooth=smooth, smooth_rcp=smooth_rcp, native_chain=native)
    else:
        codes, scale, _ = ops.act_quant(x2, mode=L.Q_I8_GIVEN_SCALE, smooth=smooth, smooth_rcp=smooth_rcp, native_chain=native,
                                        scale_in=given_scale)
        scale = given_scale
    return codes, scale


def _cuda_gemm(codes, weight, scale, w_scale, bias, out_dtype, prod_dtype, scatter=None, out=None, max_ctas=None):
    # (acc.float() * (input_scale * w_scale).to(fp16) + bias).to(fp16).to(out_dtype), linear.py:1185-1188, :1338
    return ops.gemm(codes, weight, epilogue=L.EPI_SCALE_PROD, row_scale=scale, col_scale=w_scale, bias=bias,
                    prod_round=(None if prod_dtype == torch.float32 else prod_dtype), scale_round=torch.float16,
                    acc_round=torch.float16, out_dtype=out_dtype, scatter=scatter, out=out, max_ctas=max_ctas)  # fmt: skip
