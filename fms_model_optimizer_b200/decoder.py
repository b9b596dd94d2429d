"""A Llama-shaped decoder whose Linears are W8A8 SmoothQuant INT8, on one GPU or sharded over the GPUs of a node.

This is the model harness around the quantized-Linear path: embedding, RMSNorm, rotary embedding, attention and
SwiGLU are plumbing; the seven Linears of every layer run ``QLinearINT8Deploy``'s arithmetic
(fms_mo/modules/linear.py:1309-1338, :1115-1188) on this library's kernels.  Three ways to run the same model:

* ``surface="fused"`` (default): ``tp.W8A8Linear`` fed by the fused block kernels (residual add + RMSNorm / SiLU*up +
  per-token quantisation for all Linears that share an input, one pass over the activations).
* ``surface="modules"``: the drop-in route a user of the reference takes: ``QLinear`` modules lowered with
  ``lower_qmodel_b200`` to ``QLinearINT8Deploy`` (fms_mo/dq.py:262-272 does the same with ``lower_qmodel_triton``),
  norms and activations as PyTorch ops.  One GPU only.
* sharded (``world > 1``): weights split column-parallel (q, k, v, gate, up) and row-parallel (o, down) following the
  reference's tables (fms_mo/aiu_addons/i8i8/i8i8_aiu_linear.py:304-389), one process per GPU.  ``exchange`` picks how
  the shard boundary is crossed:
    - ``"multimem"``: the residual stream is split by tokens.  A row-parallel GEMM writes its partial output to its
      own GPU's copy of a buffer that all GPUs have bound to one NVLink multicast object; the owner of a token block
      reads the sum of all copies with ``multimem.ld_reduce`` inside the fused norm + quantise kernel (the reduction
      happens in the switch) and writes the int8 codes for the following column-parallel Linears into every GPU's
      code buffer with one ``multimem.st``.  Flag barriers order the phases; no collective carries activations.
    - ``"stores"``: the same token split without the switch: the GEMM epilogue stores each token block's partial rows
      into its owner's receive slots, the owner sums them, and codes are replicated by one plain store per peer.
    - ``"allreduce"``: the textbook scheme, NCCL all-reduce of the partial outputs and of the per-token scales.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _lib as L
from . import ops, tp

LLAMA3_8B = dict(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256, rope_theta=500000.0,
                 batch=8, seq=2048)  # fmt: skip

LINEARS = ("q", "k", "v", "o", "gate", "up", "down")


def linear_shapes(cfg):
    """name -> (out features, in features, shard mode) of the seven Linears of a layer."""
    H, hd = cfg["hidden"], cfg["head_dim"]
    return dict(q=(cfg["q_heads"] * hd, H, "column"), k=(cfg["kv_heads"] * hd, H, "column"), v=(cfg["kv_heads"] * hd, H, "column"),
                o=(H, cfg["q_heads"] * hd, "row"), gate=(cfg["ffn"], H, "column"), up=(cfg["ffn"], H, "column"),
                down=(H, cfg["ffn"], "row"))  # fmt: skip


def decoder_linear_ops(cfg, tokens, layers=None):
    """Multiply-add operations (2 per MAC) of the decoder's Linears for ``tokens`` tokens."""
    per_layer = sum(n * k for n, k, _ in linear_shapes(cfg).values())
    return 2.0 * per_layer * tokens * (layers if layers is not None else cfg["layers"])


def synth_weight(n, k, seed, dev, dtype=torch.bfloat16):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(n, k, generator=g, device=dev) * 0.02).to(dtype)


def synth_act_scale(k, seed, dev, dtype=torch.bfloat16):
    """Stand-in for a calibrated SmoothQuant activation scale: 4.0 with 1 % outlier channels 20 times larger."""
    g = torch.Generator(device=dev).manual_seed(seed + 7919)
    act = torch.full((k,), 4.0, device=dev)
    idx = torch.randperm(k, generator=g, device=dev)[: max(1, k // 100)]
    act[idx] *= 20
    return act.to(dtype)


def w8a8_from_float(w, act, alpha=0.5):
    """Float Linear weight [n, k] -> (int8 codes, per-channel scales, SmoothQuant scale) the way
    QLinearINT8Deploy.from_fms_mo does it (fms_mo/modules/linear.py:799-871) for a max-per-channel weight quantizer."""
    dtype = w.dtype
    w_sq = w.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
    alpha = torch.tensor([alpha], dtype=act.dtype, device=act.device)  # the module keeps alpha as a one-element buffer
    smooth = (act**alpha / w_sq ** (1.0 - alpha)).clamp(min=1e-5).to(dtype)
    ws = w * smooth
    cv_new = ws.abs().max(dim=1).values
    # the clip values a max-per-channel weight quantizer holds after its first training-mode forward: the fresh row
    # maxima passed once through its moving average (fms_mo/quant/quantizers.py:3098-3128)
    w_cv = (cv_new * (1.0 - 0.1) + cv_new * 0.1).to(dtype)
    w_scale = w_cv * 2 / 254  # in the weight dtype, as the module's buffer would be
    codes = torch.round(ws.t() / w_scale).clamp(-127, 127).t().to(torch.int8).contiguous()
    return codes, w_scale, smooth.reshape(-1).float()


def synth_w8a8(n, k, seed, dev, dtype=torch.bfloat16):
    """Random-init Linear [n, k] (N(0, 0.02)) with synthetic activation scales, as W8A8 SmoothQuant buffers (alpha 0.5)."""
    return w8a8_from_float(synth_weight(n, k, seed, dev, dtype), synth_act_scale(k, seed, dev, dtype))


@torch.no_grad()
def calibrate_act_scales(cfg, dev, ids, layers=None):
    """The SmoothQuant calibration pass for the decoder: one forward of the float (bf16) model on ``ids`` [batch, seq] with
    the per-input-channel absolute maxima of every Linear's input recorded on the device (``ops.col_absmax``, the
    statistic of fms_mo/quant/ptq.py:2586-2596).  The float weights are the seeded ones the quantized decoder is built
    from; they are generated layer by layer and dropped again.  Returns ``{(layer, name): fp32 [in_features]}``."""
    B, S = ids.shape
    H, hd = cfg["hidden"], cfg["head_dim"]
    nl = layers if layers is not None else cfg["layers"]
    g = torch.Generator(device=dev).manual_seed(4)
    embed = (torch.randn(cfg["vocab"], H, generator=g, device=dev) * 0.02).bfloat16()
    inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, hd, 2, device=dev).float() / hd))
    ang = torch.outer(torch.arange(S, device=dev).float(), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    ones = torch.ones(H, device=dev, dtype=torch.bfloat16)
    x = F.embedding(ids, embed).view(B * S, H)
    scales = {}
    names = list(linear_shapes(cfg).items())
    for li in range(nl):
        w = {name: synth_weight(n, k, 1000 * li + ni, dev) for ni, (name, (n, k, _)) in enumerate(names)}
        h = F.rms_norm(x, (H,), ones, 1e-5)
        for name in ("q", "k", "v"):
            scales[(li, name)] = ops.col_absmax(h)
        q = ops.rope_(F.linear(h, w["q"]).view(B * S, cfg["q_heads"], hd), cos, sin, S)
        k = ops.rope_(F.linear(h, w["k"]).view(B * S, cfg["kv_heads"], hd), cos, sin, S)
        v = F.linear(h, w["v"])
        a = F.scaled_dot_product_attention(q.view(B, S, -1, hd).transpose(1, 2), k.view(B, S, -1, hd).transpose(1, 2),
                                           v.view(B, S, -1, hd).transpose(1, 2), is_causal=True, enable_gqa=True)  # fmt: skip
        a = a.transpose(1, 2).reshape(B * S, -1)
        scales[(li, "o")] = ops.col_absmax(a)
        x = x + F.linear(a, w["o"])
        h = F.rms_norm(x, (H,), ones, 1e-5)
        scales[(li, "gate")] = ops.col_absmax(h)
        scales[(li, "up")] = scales[(li, "gate")]
        m = F.silu(F.linear(h, w["gate"])) * F.linear(h, w["up"])
        scales[(li, "down")] = ops.col_absmax(m)
        x = x + F.linear(m, w["down"])
        del w
    return scales


class _Group:
    """Exchange buffers of one group of sequences (see W8A8Decoder.enable_token_split)."""


class W8A8Decoder:
    def __init__(self, cfg, dev, world=1, rank=0, layers=None, groups=1, exchange="auto", reserve_sms=0, surface="fused",
                 calibrated_act_scales=None):  # fmt: skip
        """``groups``: groups of sequences advanced round-robin on separate streams (sharded runs overlap one group's
        exchange with the other's GEMMs).  ``reserve_sms``: with several groups, SMs left to the kernels that are bound by
        the links (GEMMs are capped at the rest).  ``calibrated_act_scales``: ``{(layer, name): [k] tensor}`` from
        ``calibrate`` instead of the synthetic activation scales."""
        self.cfg, self.dev, self.world, self.rank = cfg, dev, world, rank
        self.groups = max(1, groups)
        self.reserve_sms = reserve_sms
        self.surface = surface
        self.trace: Optional[list] = None  # when a list: (tag, layer, tensor clone) appended along the forward pass
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(self.groups)] if self.groups > 1 else []
        self.sp: Optional[List[_Group]] = None
        self.arena = None
        self.last_hidden = None
        # multimem exchange: read the shards' partial sums with a streaming kernel of its own ("split", many loads in
        # flight per thread) before the fused norm + quantise kernel, or inside that kernel's prologue ("fused")
        self.switch_reduce = "split"
        # segments by which each further group of sequences starts behind the previous one (sharded runs with several
        # groups; two = the embedding and the first norm + quantise + exchange).  Measured at four GPUs: no difference with
        # two groups (46.3 ms either way), 45.6 against 47.9 ms with four.
        self.stagger = 2
        self.k_on_side_stream = False
        if exchange == "auto":
            # measured on 8 x B200: with two GPUs the plain-store scheme wins (every byte crosses one link once either
            # way and the stores ride in the GEMM epilogue); from four GPUs on the switch's reduce / replicate does
            exchange = "none" if world == 1 else ("stores" if world == 2 else "multimem")
        self.exchange = exchange
        H, hd = cfg["hidden"], cfg["head_dim"]
        self.nq, self.nkv = cfg["q_heads"] // world, cfg["kv_heads"] // world
        nl = layers if layers is not None else cfg["layers"]
        if surface == "modules" and world != 1:
            raise RuntimeError("the module surface runs on one GPU")
        self.layers = []
        for li in range(nl):
            lin = {}
            for ni, (name, (n, k, mode)) in enumerate(linear_shapes(cfg).items()):
                seed = 1000 * li + ni
                w = synth_weight(n, k, seed, dev)
                act = calibrated_act_scales[(li, name)].to(dev, torch.bfloat16) if calibrated_act_scales else synth_act_scale(k, seed, dev)
                if surface == "modules":
                    lin[name] = _deploy_module(w, act, dev)
                else:
                    codes, w_scale, smooth = w8a8_from_float(w, act)
                    wt, sc, sm, _ = tp.shard_w8a8(codes, w_scale, smooth, None, mode, world, rank)
                    lin[name] = tp.W8A8Linear(wt, sc, sm, None, mode=mode if (world > 1 and exchange == "allreduce") else "replicate")
                    del codes
                del w
            lin["ln1"] = torch.ones(H, device=dev, dtype=torch.bfloat16)
            lin["ln2"] = torch.ones(H, device=dev, dtype=torch.bfloat16)
            self.layers.append(lin)
        g = torch.Generator(device=dev).manual_seed(4)
        self.embed = (torch.randn(cfg["vocab"], H, generator=g, device=dev) * 0.02).bfloat16()
        self.lm_head = (torch.randn(cfg["vocab"], H, generator=g, device=dev) * 0.02).bfloat16()
        self.norm = torch.ones(H, device=dev, dtype=torch.bfloat16)
        S = cfg["seq"]
        inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, hd, 2, device=dev).float() / hd))
        ang = torch.outer(torch.arange(S, device=dev).float(), inv)
        self.cos, self.sin = ang.cos().contiguous(), ang.sin().contiguous()  # fp32 [S, hd / 2]
        self._apply_sm_partition()

    def _apply_sm_partition(self):
        """With several groups in flight on a sharded run, GEMMs leave ``reserve_sms`` SMs to the exchange kernels of the
        other group (in the plain-store scheme the row-parallel GEMMs are themselves link-bound and get that share)."""
        if self.surface != "fused":
            return
        on = self.world > 1 and self.reserve_sms > 0 and self.groups > 1
        sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        link_bound = ("o", "down") if self.exchange == "stores" else ()
        for lin in self.layers:
            for name in LINEARS:
                lin[name].max_ctas = None if not on else (self.reserve_sms if name in link_bound else sms - self.reserve_sms)

    def reconfigure(self, groups=None, reserve_sms=None, exchange=None):
        """Sharded runs: another number of sequence groups, SM partition or exchange scheme ("multimem" / "stores") on the
        same weights.  Collective: every rank calls it with the same arguments; call ``enable_token_split`` afterwards."""
        self.close()
        self.sp = None
        if groups is not None:
            self.groups = max(1, groups)
            self.streams = [torch.cuda.Stream(device=self.dev) for _ in range(self.groups)] if self.groups > 1 else []
        if reserve_sms is not None:
            self.reserve_sms = reserve_sms
        if exchange is not None:
            if "allreduce" in (exchange, self.exchange) and exchange != self.exchange:
                raise RuntimeError("the NCCL all-reduce scheme shards the Linears differently: build another decoder")
            self.exchange = exchange
        self._apply_sm_partition()

    # ------------------------------------------------------------------------------------------------ helpers
    def _note(self, tag, layer, t):
        if self.trace is not None:
            self.trace.append((tag, layer, t.detach().clone()))

    def _attention(self, q, k, v, B, S):
        hd = self.cfg["head_dim"]
        a = F.scaled_dot_product_attention(q.view(B, S, self.nq, hd).transpose(1, 2), k.view(B, S, self.nkv, hd).transpose(1, 2),
                                           v.view(B, S, self.nkv, hd).transpose(1, 2), is_causal=True, enable_gqa=True)  # fmt: skip
        return a.transpose(1, 2).reshape(B * S, self.nq * hd)

    def _head(self, last):
        """(next-token ids, the normalised hidden state they were computed from) for the last token of every sequence."""
        return (last @ self.lm_head.t()).argmax(-1), last

    # ------------------------------------------------------------------------------------------------ one GPU / NCCL
    def _forward_steps(self, ids):
        """The forward pass of one group of sequences as a generator: it yields after every row-parallel Linear
        (whose all-reduce, if any, has just been queued), so that a driver can advance another group on another
        stream meanwhile.  Returns the next-token ids through StopIteration."""
        cfg = self.cfg
        B, S = ids.shape
        hd, bf = cfg["head_dim"], torch.bfloat16
        x = F.embedding(ids, self.embed).view(B * S, -1)
        pending = None  # output of the last row-parallel Linear, added to the stream by the next fused kernel
        tr = self.trace is not None
        for li, lin in enumerate(self.layers):
            # (x += pending) -> RMSNorm -> per-token int8 codes for q, k, v: one pass over the stream
            cs, ss, xs, h = ops.block_quant(x, prologue=L.BLOCK_NORM, r=pending, norm_w=lin["ln1"], store_sum=True, want_h=tr,
                                            smooth_rcps=[lin["q"].smooth_rcp, lin["k"].smooth_rcp, lin["v"].smooth_rcp])  # fmt: skip
            x = xs if xs is not None else x
            q = lin["q"](None, (cs[0], ss[0]), bf)
            k = lin["k"](None, (cs[1], ss[1]), bf)
            v = lin["v"](None, (cs[2], ss[2]), bf)
            if tr:
                for tag, t in (("x_attn_in", x), ("h_attn", h), ("q", q), ("k", k), ("v", v)):
                    self._note(tag, li, t)
                for name, c_, s_ in zip("qkv", cs, ss):
                    self._note("codes_" + name, li, c_)
                    self._note("scale_" + name, li, s_)
            q = ops.rope_(q.view(B * S, self.nq, hd), self.cos, self.sin, S)
            k = ops.rope_(k.view(B * S, self.nkv, hd), self.cos, self.sin, S)
            del cs, ss
            a = self._attention(q, k, v, B, S)
            qa = lin["o"].quantise_fused(a)
            pending = lin["o"](None, qa, bf)
            if tr:
                for tag, t in (("q_rope", q), ("k_rope", k), ("attn", a), ("codes_o", qa[0]), ("scale_o", qa[1]), ("o", pending)):
                    self._note(tag, li, t)
            yield
            cs, ss, x, h = ops.block_quant(x, prologue=L.BLOCK_NORM, r=pending, norm_w=lin["ln2"], store_sum=True, want_h=tr,
                                           smooth_rcps=[lin["gate"].smooth_rcp, lin["up"].smooth_rcp])  # fmt: skip
            g = lin["gate"](None, (cs[0], ss[0]), bf)
            u = lin["up"](None, (cs[1], ss[1]), bf)
            keep = [] if tr else None
            qd = lin["down"].quantise_fused(g, L.BLOCK_SILU_MUL, u, keep_h=keep)
            pending = lin["down"](None, qd, bf)
            if tr:
                for tag, t in (("x_mlp_in", x), ("h_mlp", h), ("gate", g), ("up", u), ("codes_gate", cs[0]), ("scale_gate", ss[0]),
                               ("codes_up", cs[1]), ("scale_up", ss[1]), ("h_down", keep[0]), ("codes_down", qd[0]), ("scale_down", qd[1]),
                               ("down", pending)):  # fmt: skip
                    self._note(tag, li, t)
            del cs, ss
            yield
        # only the last token of every sequence reaches the head
        x_last, p_last = x.view(B, S, -1)[:, -1].contiguous(), pending.view(B, S, -1)[:, -1].contiguous()
        _, _, x_last, h = ops.block_quant(x_last, prologue=L.BLOCK_NORM, r=p_last, norm_w=self.norm, store_sum=True, smooth_rcps=[], want_h=True)
        self._note("x_final_last", len(self.layers), x_last)
        return self._head(h)

    def _forward_steps_modules(self, ids):
        """The same decoder through the module surface: RMSNorm, SiLU*up and the residual adds as PyTorch ops, every
        Linear a ``QLinearINT8Deploy`` (its own quantise kernel + GEMM)."""
        cfg = self.cfg
        B, S = ids.shape
        hd = cfg["head_dim"]
        x = F.embedding(ids, self.embed).view(B * S, -1)
        for li, lin in enumerate(self.layers):
            self._note("x_attn_in", li, x)
            h = F.rms_norm(x, (x.shape[-1],), lin["ln1"], 1e-5)
            q = ops.rope_(lin["q"](h).view(B * S, self.nq, hd), self.cos, self.sin, S)
            k = ops.rope_(lin["k"](h).view(B * S, self.nkv, hd), self.cos, self.sin, S)
            v = lin["v"](h)
            x = x + lin["o"](self._attention(q, k, v, B, S))
            self._note("x_mlp_in", li, x)
            h = F.rms_norm(x, (x.shape[-1],), lin["ln2"], 1e-5)
            x = x + lin["down"](F.silu(lin["gate"](h)) * lin["up"](h))
            yield
        self._note("x_final", len(self.layers), x)
        h = F.rms_norm(x, (x.shape[-1],), self.norm, 1e-5)
        return self._head(h.view(B, S, -1)[:, -1])

    # ------------------------------------------------------------------------------------------------ token split
    def enable_token_split(self, tokens_per_group, barrier_timeout_s=10.0):
        """Buffers for the sharded forward that keeps the residual stream split by tokens.  Per group of sequences, in an
        arena at the same offsets on every GPU: a bf16 ``[tokens, hidden]`` buffer for the row-parallel Linears' partial
        outputs, the int8 codes and fp32 scales of up to three Linear inputs for all tokens, ``[world][tokens]`` slots
        for the per-token scales of a row-parallel Linear's input, and the barrier's flags."""
        from .peer import PeerBarrier, make_arena

        H, W, T = self.cfg["hidden"], self.world, tokens_per_group
        if T % W != 0 or (T // W) % 128 != 0:
            raise RuntimeError("tokens per rank and group must be a multiple of 128")
        # load the attention library on every rank before the first flag barrier can start counting: a rank that is
        # still reading shared objects from a cold disk must not make its peers' bounded waits run out
        t = torch.zeros(1, 2, 128, self.cfg["head_dim"], dtype=torch.bfloat16, device=self.dev)
        F.scaled_dot_product_attention(t, t, t, is_causal=True)
        torch.cuda.synchronize(self.dev)
        dist.barrier()
        per_group = T * H * 2 + 3 * (T * H + 4 * T + 512) + 4 * W * T + 4096
        self.arena = make_arena(self.groups * per_group + 4096, self.dev, want_multicast=(self.exchange == "multimem"))
        if self.exchange == "multimem" and not getattr(self.arena, "mc_base", 0):
            self.exchange = "stores"  # no NVLink multicast on this node: the plain peer-store scheme
        mm = self.exchange == "multimem"
        self.sp = []
        for _ in range(self.groups):
            g = _Group()
            g.bar = PeerBarrier(self.arena, barrier_timeout_s)
            g.side = torch.cuda.Stream(device=self.dev)
            g.side2 = torch.cuda.Stream(device=self.dev)
            g.T, g.Ts = T, T // W
            g.part_off, part = self.arena.alloc(T * H * 2)
            # multimem: my partial output for all tokens; stores: [world] receive slots for my tokens
            g.part = part.view(torch.bfloat16).view(T, H) if mm else part.view(torch.bfloat16).view(W, T // W, H)
            g.codes_off, g.scale_off, g.codes, g.scales = [], [], [], []
            for _ in range(3):
                off, c = self.arena.alloc(T * H)
                g.codes_off.append(off)
                g.codes.append(c.view(torch.int8).view(T, H))
            for _ in range(3):
                off, sc = self.arena.alloc(4 * T)
                g.scale_off.append(off)
                g.scales.append(sc.view(torch.float32)[:T])
            g.sslot_off, sl = self.arena.alloc(4 * W * T)
            g.sslots = sl.view(torch.float32)[: W * T]
            # multimem: the multicast address, and this GPU's own arena for a plain copy of what its own kernels read next
            g.bases = [self.arena.mc_addr(0), self.arena.addr(self.rank, 0)] if mm else [self.arena.addr(r, 0) for r in range(W)]
            g.part_bases = [self.arena.addr(r, g.part_off) for r in range(W)]
            g.my_part_mc = self.arena.mc_addr(g.part_off + self.rank * g.Ts * H * 2) if mm else 0
            self.sp.append(g)
        self.nvlink_bytes_per_forward = self._exchange_bytes(T)

    def _exchange_bytes(self, T):
        """(bytes leaving this GPU, bytes arriving) over NVLink in one forward pass of all groups, counted from the
        buffers the exchange kernels write and read."""
        H, W, nl = self.cfg["hidden"], self.world, len(self.layers)
        Ts = T // W
        partial_rows_out = (T - Ts) * H * 2        # my partial rows owned by the other ranks
        codes_out = Ts * (H + 4)                   # one code tensor + scales of my tokens
        scales = T * 4                             # per-token scales of a row-parallel input
        if self.exchange == "multimem":
            out_b = 2 * partial_rows_out + 5 * codes_out + 2 * scales
            in_b = 2 * Ts * H * 2 + 5 * (W - 1) * codes_out + 2 * (W - 1) * scales
        else:
            out_b = 2 * partial_rows_out + 5 * (W - 1) * codes_out + 2 * (W - 1) * scales
            in_b = 2 * (W - 1) * Ts * H * 2 + 5 * (W - 1) * codes_out + 2 * (W - 1) * scales
        return out_b * nl * self.groups, in_b * nl * self.groups

    def _forward_steps_split(self, ids, g):
        """Sharded forward with the residual stream split by tokens: this rank owns tokens [rank * Ts, (rank + 1) * Ts)
        of the group.  Two barriers per half layer order the exchange (partials complete -> owners reduce; codes
        landed -> column-parallel GEMMs), one more the per-token scales of the row-parallel input."""
        cfg, W, rank = self.cfg, self.world, self.rank
        B, S = ids.shape
        hd, bf = cfg["head_dim"], torch.bfloat16
        T, Ts, bar = g.T, g.Ts, g.bar
        mm = self.exchange == "multimem"
        x = F.embedding(ids.reshape(-1)[rank * Ts : (rank + 1) * Ts], self.embed)
        H = x.shape[1]
        have_parts = False
        link_ctas = 8 * self.reserve_sms if self.reserve_sms > 0 else 0
        sx = tp.ScaleExchange(bar, g.bases, g.sslot_off, rank, g.sslots, mm)

        def reduce_norm_quant(norm_w, rcps, want_h=False):
            """x += sum over shards of the last row-parallel partials (my tokens); h = RMSNorm(x); codes of h for the
            Linears that follow, into every rank's buffers."""
            n = len(rcps)
            kw = dict(prologue=L.BLOCK_NORM, norm_w=norm_w, smooth_rcps=rcps, sum_into=x, max_ctas=link_ctas, want_h=want_h)
            if n:
                kw["dst"] = (g.bases, g.codes_off[:n], g.scale_off[:n], rank * Ts)
                kw["dst_multimem"] = mm
            if have_parts and mm and self.switch_reduce == "split":
                ops.shard_reduce_(x, g.my_part_mc, max_ctas=2 * self.reserve_sms)
            elif have_parts and mm:
                kw.update(r_ptr=g.my_part_mc, r_multimem=True)
            elif have_parts:
                kw.update(r=g.part[0], r_parts=W, r_part_stride=Ts * H)
            return ops.block_quant(x, **kw)

        def row_parallel(lin_, quantised):
            if mm:  # partial output for all tokens into my copy of the shared buffer; the owners pull the sums
                lin_(None, quantised, bf, out=g.part)
            else:   # the epilogue stores token block i into rank i's receive slot
                lin_.scatter(quantised, g.part_bases, Ts, rank * Ts, bf)
            bar.wait()  # every rank's partials are complete

        for li, lin in enumerate(self.layers):
            yield
            reduce_norm_quant(lin["ln1"], [lin["q"].smooth_rcp, lin["k"].smooth_rcp, lin["v"].smooth_rcp])
            self._note("x_attn_in", li, x)
            bar.wait()  # every rank's codes have landed here
            yield
            # the shards of k and v are narrow (a quarter of q's columns with grouped-query attention): v's GEMM goes to a
            # side stream so that it shares a wave of CTAs with k's instead of taking one of its own
            cur = torch.cuda.current_stream()
            g.side.wait_stream(cur)
            with torch.cuda.stream(g.side):
                v = lin["v"](None, (g.codes[2], g.scales[2]), bf)
            if self.k_on_side_stream:  # with many small groups q's shard does not fill the GPU either: k beside it as well
                g.side2.wait_stream(cur)
                with torch.cuda.stream(g.side2):
                    k = ops.rope_(lin["k"](None, (g.codes[1], g.scales[1]), bf).view(T, self.nkv, hd), self.cos, self.sin, S)
            q = ops.rope_(lin["q"](None, (g.codes[0], g.scales[0]), bf).view(T, self.nq, hd), self.cos, self.sin, S)
            if self.k_on_side_stream:
                cur.wait_stream(g.side2)
                k.record_stream(cur)
            else:
                k = ops.rope_(lin["k"](None, (g.codes[1], g.scales[1]), bf).view(T, self.nkv, hd), self.cos, self.sin, S)
            cur.wait_stream(g.side)
            v.record_stream(cur)
            a = self._attention(q, k, v, B, S)
            row_parallel(lin["o"], lin["o"].quantise_fused(a, exchange=sx))
            have_parts = True
            yield
            reduce_norm_quant(lin["ln2"], [lin["gate"].smooth_rcp, lin["up"].smooth_rcp])
            self._note("x_mlp_in", li, x)
            bar.wait()
            yield
            gt = lin["gate"](None, (g.codes[0], g.scales[0]), bf)
            u = lin["up"](None, (g.codes[1], g.scales[1]), bf)
            row_parallel(lin["down"], lin["down"].quantise_fused(gt, L.BLOCK_SILU_MUL, u, exchange=sx))
        yield
        # final norm of my token slice; the last token of every sequence goes to all ranks through one small all-reduce
        _, _, _, h = reduce_norm_quant(self.norm, [], want_h=True)
        self._note("x_final", len(self.layers), x)
        last = torch.zeros(B, h.shape[1], dtype=bf, device=h.device)
        for b in range(B):
            idx = b * S + S - 1
            if idx // Ts == rank:
                last[b] = h[idx % Ts]
        dist.all_reduce(last)
        bar.wait()  # the exchange buffers are free for the next forward pass
        return self._head(last)

    # ------------------------------------------------------------------------------------------------ driver
    @torch.no_grad()
    def forward(self, ids):
        """Next-token ids [batch]; ``self.last_hidden`` keeps the final normalised hidden state of every sequence's last
        token ([batch, hidden]) for comparisons between the ways of running the model."""
        parts = ids.chunk(self.groups, 0)
        if self.surface == "modules":
            gens = [self._forward_steps_modules(p) for p in parts]
        elif self.sp is not None:
            gens = [self._forward_steps_split(p, self.sp[i]) for i, p in enumerate(parts)]
        else:
            gens = [self._forward_steps(p) for p in parts]
        out, self.last_hidden = self._drive(gens)
        return out

    def _drive(self, gens):
        """Advances the groups round-robin, one segment at a time, each on its own stream."""
        nm = len(gens)
        if nm <= 1:
            try:
                while True:
                    next(gens[0])
            except StopIteration as stop:
                return stop.value
        main = torch.cuda.current_stream()
        results = [None] * nm
        for i in range(nm):
            self.streams[i].wait_stream(main)
        live = list(range(nm))
        if self.stagger > 0:
            # group i starts once group i - 1 has finished its first `stagger` segments: the groups then sit in different
            # phases (one exchanging while another multiplies) instead of all exchanging and all multiplying together
            for i in range(nm - 1):
                with torch.cuda.stream(self.streams[i]):
                    for _ in range(self.stagger):
                        try:
                            next(gens[i])
                        except StopIteration as stop:
                            results[i] = stop.value
                            live.remove(i)
                            break
                self.streams[i + 1].wait_stream(self.streams[i])
        while live:
            for i in list(live):
                with torch.cuda.stream(self.streams[i]):
                    try:
                        next(gens[i])
                    except StopIteration as stop:
                        results[i] = stop.value
                        live.remove(i)
        for i in range(nm):
            main.wait_stream(self.streams[i])
            for t in results[i]:
                t.record_stream(main)
        return tuple(torch.cat(ts) for ts in zip(*results))

    def close(self):
        """Sharded runs: every rank stops touching the exchange buffers before any rank leaves."""
        if self.arena is not None:
            self.arena.close()
            self.arena = None


def _deploy_module(w, act, dev):
    """One Linear of the decoder by the drop-in route: a ``QLinear`` (per-token max activations, max-per-channel weights,
    SmoothQuant alpha 0.5) holding the float weight and the activation scale, one training-mode forward to latch the
    weight clip values (fms_mo/quant/quantizers.py:3098-3104), then ``lower_qmodel_b200`` -> ``QLinearINT8Deploy``."""
    from .modules import QLinear, lower_qmodel_b200

    n, k = w.shape
    holder = torch.nn.Module()
    lin = QLinear(k, n, bias=False, num_bits_feature=8, qa_mode="pertokenmax", num_bits_weight=8, qw_mode="maxperCh",
                  qcfg={"smoothq": True, "smoothq_alpha": 0.5}, device=dev)  # fmt: skip
    with torch.no_grad():
        lin.weight.copy_(w)
    lin = lin.to(w.dtype)
    lin.set_act_scale(act.float())
    lin.train()
    with torch.no_grad():
        lin(torch.zeros(1, k, device=dev, dtype=w.dtype))
    lin.eval()
    holder.lin = lin
    lower_qmodel_b200(holder, use_dyn_max_act=-1)
    return holder.lin
