"""Benchmark of the W8A8 quantized-Linear hot path on B200.

Default workload ("c5"): prefill of a Llama-3-8B-shaped decoder (32 layers, hidden 4096, 32 q / 8 kv
heads of 128, SwiGLU FFN 14336, RMSNorm, RoPE theta 5e5, vocab 128256) whose every Linear inside the
decoder layers is W8A8 SmoothQuant INT8 (alpha 0.5, per-channel weights, per-token activations), on a
batch of 8 x 2048 random token ids.  With N > 1 GPUs the Linears are sharded column / row parallel
(tensor parallel), one process per GPU, NCCL all-reduce at the row-parallel boundaries; the total
work is fixed, so scaling is "strong".

    python bench.py --gpus N --steps K --warmup W                  # this implementation
    python bench.py --impl reference --gpus N --steps K --warmup W # reference CPU fake-quant path

One JSON line is printed by rank 0.  `value` is tokens/s of the whole job with the token ids
already on the device; `e2e` is the same with the ids copied from pinned host memory and the
next-token ids copied back inside the timed region.  `roofline` is the int8 GEMM kernel (all its
launches in the timed region, timed with CUDA events on the launching stream); `cpu_baseline` is
the reference's CPU fake-quant arithmetic (QLinear.forward: per-token / per-channel fake quantise +
F.linear) for one decoder layer on a bounded token sample, extrapolated to the 32 layers.

Other workloads, for single kernels: --workload c1 | c2 | c3 | c5lin (TOPS of one quantized Linear / GEMM;
c5lin is one 16384 x 4096 x 4096 Linear of the c5 decoder).
Weights and activations are synthetic (seeded); nothing is read from disk.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA = dict(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256, rope_theta=500000.0,
             batch=8, seq=2048)  # fmt: skip


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, src="fallback")


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        busy = [v for v in sm if smax and v > 0.3 * smax] or sm
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# synthetic W8A8 decoder
# ------------------------------------------------------------------------------------------------
def synth_w8a8(n, k, seed, dev, dtype=torch.bfloat16):
    """Random-init Linear [n, k] (N(0, 0.02)) turned into W8A8 SmoothQuant buffers the way
    QLinearINT8Deploy.from_fms_mo does it (fms_mo/modules/linear.py:799-871): synthetic activation
    scales (1% outlier channels x20), smoothing scale with alpha 0.5, per-channel max weight scale,
    int8 codes."""
    g = torch.Generator(device=dev).manual_seed(seed)
    w = (torch.randn(n, k, generator=g, device=dev) * 0.02).to(dtype)
    act = torch.full((k,), 4.0, device=dev)
    idx = torch.randperm(k, generator=g, device=dev)[: max(1, k // 100)]
    act[idx] *= 20
    act = act.to(dtype)
    w_sq = w.abs().max(dim=0, keepdim=True)[0].clamp(min=1e-5)
    smooth = (act**0.5 / w_sq**0.5).clamp(min=1e-5).to(dtype)
    ws = w * smooth
    w_cv = ws.abs().max(dim=1).values
    w_scale = w_cv * 2 / 254
    codes = torch.round(ws.t() / w_scale).clamp(-127, 127).t().to(torch.int8).contiguous()
    return codes, w_scale.float(), smooth.reshape(-1).float()


class Decoder:
    """Llama-shaped decoder whose Linears are ``tp.W8A8Linear``; norms, RoPE, attention and SwiGLU
    are plain PyTorch ops on the device (they are not part of the quantized-Linear path)."""

    def __init__(self, cfg, dev, world, rank, layers=None, n_micro=1):
        from fms_model_optimizer_b200 import tp

        self.n_micro = n_micro
        self.rank = rank
        self.sp = None
        self.exchange = "stores"
        self.chain = False
        self.scale_exchange = True
        self.reserve_sms = 0
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(n_micro)] if n_micro > 1 else []

        self.cfg = cfg
        self.dev = dev
        self.world = world
        H, hd = cfg["hidden"], cfg["head_dim"]
        self.nq, self.nkv = cfg["q_heads"] // world, cfg["kv_heads"] // world
        nl = layers if layers is not None else cfg["layers"]
        self.layers = []
        for li in range(nl):
            lin = {}
            for ni, (name, (n, k, mode)) in enumerate(dict(
                q=(cfg["q_heads"] * hd, H, "column"), k=(cfg["kv_heads"] * hd, H, "column"), v=(cfg["kv_heads"] * hd, H, "column"),
                o=(H, cfg["q_heads"] * hd, "row"), gate=(cfg["ffn"], H, "column"), up=(cfg["ffn"], H, "column"),
                down=(H, cfg["ffn"], "row"),
            ).items()):  # fmt: skip
                codes, w_scale, smooth = synth_w8a8(n, k, 1000 * li + ni, dev)
                wt, sc, sm, _ = tp.shard_w8a8(codes, w_scale, smooth, None, mode, world, rank)
                lin[name] = tp.W8A8Linear(wt, sc, sm, None, mode=mode if world > 1 else "replicate")
                del codes
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

    def _forward_steps(self, ids):
        """The forward pass of one group of sequences as a generator: it yields after every row-parallel
        Linear (whose all-reduce has just been queued), so that a driver can advance another group on another
        stream while the collective runs.  Returns the next-token ids through StopIteration."""
        from fms_model_optimizer_b200 import _lib as L
        from fms_model_optimizer_b200 import ops

        cfg = self.cfg
        B, S = ids.shape
        hd = cfg["head_dim"]
        bf = torch.bfloat16
        x = F.embedding(ids, self.embed).view(B * S, -1)
        pending = None  # output of the last row-parallel Linear, added to the stream by the next fused kernel
        for lin in self.layers:
            # (x += pending) -> RMSNorm -> per-token int8 codes for q, k, v: one pass over the stream
            cs, ss, xs, _ = ops.block_quant(x, prologue=L.BLOCK_NORM, r=pending, norm_w=lin["ln1"], store_sum=True,
                                            smooth_rcps=[lin["q"].smooth_rcp, lin["k"].smooth_rcp, lin["v"].smooth_rcp])  # fmt: skip
            x = xs if xs is not None else x
            q = ops.rope_(lin["q"](None, (cs[0], ss[0]), bf).view(B * S, self.nq, hd), self.cos, self.sin, S)
            k = ops.rope_(lin["k"](None, (cs[1], ss[1]), bf).view(B * S, self.nkv, hd), self.cos, self.sin, S)
            v = lin["v"](None, (cs[2], ss[2]), bf)
            del cs, ss
            a = F.scaled_dot_product_attention(q.view(B, S, self.nq, hd).transpose(1, 2), k.view(B, S, self.nkv, hd).transpose(1, 2),
                                               v.view(B, S, self.nkv, hd).transpose(1, 2), is_causal=True, enable_gqa=True)  # fmt: skip
            a = a.transpose(1, 2).reshape(B * S, self.nq * hd)
            pending = lin["o"](None, lin["o"].quantise_fused(a), bf)
            yield
            cs, ss, x, _ = ops.block_quant(x, prologue=L.BLOCK_NORM, r=pending, norm_w=lin["ln2"], store_sum=True,
                                           smooth_rcps=[lin["gate"].smooth_rcp, lin["up"].smooth_rcp])  # fmt: skip
            g = lin["gate"](None, (cs[0], ss[0]), bf)
            u = lin["up"](None, (cs[1], ss[1]), bf)
            del cs, ss
            pending = lin["down"](None, lin["down"].quantise_fused(g, L.BLOCK_SILU_MUL, u), bf)
            yield
        last = x.view(B, S, -1)[:, -1] + pending.view(B, S, -1)[:, -1]
        last = F.rms_norm(last, (last.shape[-1],), self.norm, 1e-5)
        logits = last @ self.lm_head.t()
        return logits.argmax(-1)

    def enable_sequence_parallel(self, tokens_per_group):
        """Buffers for the sharded forward that keeps the residual stream split by tokens: per group of sequences,
        a receive buffer for the row-parallel Linears' partial outputs ([world][tokens / world, hidden] bf16), the
        int8 codes and scales of up to three Linear inputs for all tokens, and a barrier."""
        from fms_model_optimizer_b200.peer import PeerArena, PeerBarrier

        H, W, T = self.cfg["hidden"], self.world, tokens_per_group
        assert T % W == 0 and (T // W) % 128 == 0, "tokens per rank must be a multiple of 128"
        # load the attention library on every rank before the first flag barrier can start counting: a rank that is
        # still reading shared objects from a cold disk must not make its peers' bounded waits run out
        t = torch.zeros(1, 2, 128, self.cfg["head_dim"], dtype=torch.bfloat16, device=self.dev)
        F.scaled_dot_product_attention(t, t, t, is_causal=True)
        torch.cuda.synchronize(self.dev)
        dist.barrier()
        per_group = T * H * 2 + 3 * (T * H + 4 * T) + 4 * W * T + 4096
        self.arena = PeerArena(max(1, self.n_micro) * per_group + 4096, self.dev)
        self.sp = []
        for _ in range(max(1, self.n_micro)):
            g = {"bar": PeerBarrier(self.arena), "T": T, "Ts": T // W}
            g["part_off"], part = self.arena.alloc(T * H * 2)
            g["part"] = part.view(torch.bfloat16).view(W, T // W, H)
            g["codes_off"], g["scale_off"], g["codes"], g["scales"] = [], [], [], []
            for _ in range(3):
                off, c = self.arena.alloc(T * H)
                g["codes_off"].append(off)
                g["codes"].append(c.view(torch.int8).view(T, H))
            for _ in range(3):
                off, sc = self.arena.alloc(4 * T)
                g["scale_off"].append(off)
                g["scales"].append(sc.view(torch.float32)[:T])
            g["sslot_off"], sl = self.arena.alloc(4 * W * T)  # per-token scales of a row-parallel layer, one slot per shard
            g["sslots"] = sl.view(torch.float32)[: W * T]
            g["part_bases"] = [self.arena.addr(r, g["part_off"]) for r in range(W)]
            g["bases"] = [self.arena.addr(r, 0) for r in range(W)]
            if self.exchange == "copies":
                # local staging for the copy engines: this rank's codes and scales of its own tokens, and the
                # partial output of a row-parallel GEMM for all tokens
                Ts = T // W
                g["stage"] = torch.empty(3 * Ts * H + 12 * Ts, dtype=torch.uint8, device=self.dev)
                g["stage_codes_off"] = [o * Ts * H for o in range(3)]
                g["stage_scale_off"] = [3 * Ts * H + o * 4 * Ts for o in range(3)]
                g["po"] = torch.empty(T, H, dtype=torch.bfloat16, device=self.dev)
                assert all(g["codes_off"][o] == g["codes_off"][0] + o * T * H for o in range(3))
                assert all(g["scale_off"][o] == g["scale_off"][0] + o * 4 * T for o in range(3))
            self.sp.append(g)

    def _forward_steps_sp(self, ids, g):
        """Sharded forward with the residual stream split by tokens.  Each rank owns tokens [rank * Ts, (rank + 1) * Ts)
        of the group: it sums the partial outputs the row-parallel GEMMs of all ranks stored into its receive buffer,
        adds them to its slice of the stream, normalises, quantises for the following column-parallel Linears and
        stores those codes into every rank's code buffer.  No collective carries activations; two barriers per
        half layer order the remote stores."""
        from fms_model_optimizer_b200 import _lib as L
        from fms_model_optimizer_b200 import ops

        cfg, W, rank = self.cfg, self.world, self.rank
        B, S = ids.shape
        hd, bf = cfg["head_dim"], torch.bfloat16
        T, Ts, bar = g["T"], g["Ts"], g["bar"]
        x = F.embedding(ids.reshape(-1)[rank * Ts : (rank + 1) * Ts], self.embed)
        parts = None

        H = x.shape[1]
        # per-token scales of the row-parallel layers travel the same way as the activations (peer stores + barrier)
        sx = (bar, g["bases"], g["sslot_off"], rank, g["sslots"]) if self.scale_exchange else None
        copies = self.exchange == "copies"
        arena = self.arena

        def shared_quant(norm_w, lins):
            yield "compute"
            n = len(lins)
            if copies:  # quantise into local staging, then the copy engines place my rows in every rank's buffers
                dst = ([g["stage"].data_ptr()], g["stage_codes_off"][:n], g["stage_scale_off"][:n], 0)
            else:  # the kernel stores to every rank's buffers itself
                dst = (g["bases"], g["codes_off"][:n], g["scale_off"][:n], rank * Ts)
            ops.block_quant(x, prologue=L.BLOCK_NORM, r=(parts[0] if parts is not None else None), r_parts=(W if parts is not None else 0),
                            r_part_stride=Ts * H, norm_w=norm_w, smooth_rcps=[l.smooth_rcp for l in lins], sum_into=x, dst=dst,
                            max_ctas=(4 * self.reserve_sms if not copies else 0))  # fmt: skip
            if copies:
                yield "comm"
                src = g["stage"].data_ptr()
                for p in range(W):
                    arena.copy2d(arena.addr(p, g["codes_off"][0]) + rank * Ts * H, T * H, src, Ts * H, Ts * H, n)
                    arena.copy2d(arena.addr(p, g["scale_off"][0]) + rank * Ts * 4, T * 4, src + 3 * Ts * H, Ts * 4, Ts * 4, n)
            bar.wait()  # every rank's codes have landed here

        def row_parallel(lin_, quantised):
            if not copies:
                yield "compute"
            if copies:
                lin_.gemm_fn(quantised[0], lin_.weight, quantised[1], lin_.w_scale, lin_.bias, bf,
                             torch.promote_types(bf, lin_.w_scale_dtype), out=g["po"])
                yield "comm"
                for p in range(W):
                    arena.copy2d(arena.addr(p, g["part_off"]) + rank * Ts * H * 2, 0, g["po"].data_ptr() + p * Ts * H * 2, 0, Ts * H * 2, 1)
            else:
                lin_.scatter(quantised, g["part_bases"], Ts, rank * Ts, bf)
            bar.wait()  # every rank's partial rows for my tokens have landed

        for lin in self.layers:
            yield from shared_quant(lin["ln1"], [lin["q"], lin["k"], lin["v"]])
            yield "compute"
            q = ops.rope_(lin["q"](None, (g["codes"][0], g["scales"][0]), bf).view(T, self.nq, hd), self.cos, self.sin, S)
            k = ops.rope_(lin["k"](None, (g["codes"][1], g["scales"][1]), bf).view(T, self.nkv, hd), self.cos, self.sin, S)
            v = lin["v"](None, (g["codes"][2], g["scales"][2]), bf)
            a = F.scaled_dot_product_attention(q.view(B, S, self.nq, hd).transpose(1, 2), k.view(B, S, self.nkv, hd).transpose(1, 2),
                                               v.view(B, S, self.nkv, hd).transpose(1, 2), is_causal=True, enable_gqa=True)  # fmt: skip
            a = a.transpose(1, 2).reshape(T, self.nq * hd)
            yield from row_parallel(lin["o"], lin["o"].quantise_fused(a, exchange=sx))
            parts = g["part"]
            yield from shared_quant(lin["ln2"], [lin["gate"], lin["up"]])
            yield "compute"
            gt = lin["gate"](None, (g["codes"][0], g["scales"][0]), bf)
            u = lin["up"](None, (g["codes"][1], g["scales"][1]), bf)
            yield from row_parallel(lin["down"], lin["down"].quantise_fused(gt, L.BLOCK_SILU_MUL, u, exchange=sx))
        yield "compute"
        # final norm of my token slice; the last token of every sequence goes to all ranks through one small all-reduce
        _, _, _, h = ops.block_quant(x, prologue=L.BLOCK_NORM, r=parts[0], r_parts=W, r_part_stride=Ts * x.shape[1], norm_w=self.norm,
                                     smooth_rcps=[], sum_into=x, want_h=True)  # fmt: skip
        last = torch.zeros(B, h.shape[1], dtype=bf, device=h.device)
        for b in range(B):
            idx = b * S + S - 1
            if idx // Ts == rank:
                last[b] = h[idx % Ts]
        dist.all_reduce(last)
        bar.wait()  # the receive buffers are free for the next forward pass
        logits = last @ self.lm_head.t()
        return logits.argmax(-1)

    @torch.no_grad()
    def forward(self, ids):
        nm = self.n_micro
        if self.sp is not None:
            return self._drive([self._forward_steps_sp(part, self.sp[i]) for i, part in enumerate(ids.chunk(max(1, nm), 0))])
        return self._drive([self._forward_steps(part) for part in ids.chunk(max(1, nm), 0)])

    def _drive(self, gens):
        """Advances the groups round-robin, one segment at a time.  A generator announces the kind of its next segment
        ("compute": kernels that fill the SMs; "comm": copy-engine transfers and the barrier that waits for the peers;
        None: unclassified) and issues it when resumed.  Compute segments of all groups are chained through events, so
        they run one after the other while the transfers of the other groups proceed beside them (``self.chain``;
        without it the groups' streams are left to the hardware scheduler)."""
        nm = len(gens)
        if nm <= 1:
            try:
                while True:
                    next(gens[0])
            except StopIteration as stop:
                return stop.value
        main = torch.cuda.current_stream()
        results, pending, token = [None] * nm, [None] * nm, None
        for i in range(nm):
            self.streams[i].wait_stream(main)
        live = list(range(nm))
        while live:
            for i in list(live):
                st = self.streams[i]
                with torch.cuda.stream(st):
                    if self.chain and pending[i] == "compute" and token is not None and token[0] != i:
                        st.wait_event(token[1])
                    issued = pending[i]
                    try:
                        pending[i] = next(gens[i])
                    except StopIteration as stop:
                        results[i] = stop.value
                        live.remove(i)
                    if issued == "compute":
                        ev = torch.cuda.Event()
                        ev.record(st)
                        token = (i, ev)
        for i in range(nm):
            main.wait_stream(self.streams[i])
            results[i].record_stream(main)
        return torch.cat(results)


def decoder_linear_ops(cfg, tokens, layers=None):
    hd, H = cfg["head_dim"], cfg["hidden"]
    per_layer = H * (cfg["q_heads"] * hd) * 2 + 2 * H * (cfg["kv_heads"] * hd) + 3 * H * cfg["ffn"]
    return 2.0 * per_layer * tokens * (layers if layers is not None else cfg["layers"])


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's fake-quant QLinear arithmetic (oracle port)
# ------------------------------------------------------------------------------------------------
def cpu_reference_layer_tokens_per_s(tokens: int, steps: int, warmup: int, cfg=LLAMA):
    """Times the seven QLinear fake-quant forwards of one decoder layer (QLinear.forward,
    fms_mo/modules/linear.py:248-305, with qa_mode pertokenmax / qw_mode maxperCh / SmoothQuant) on
    `tokens` tokens with all host threads and returns (tokens/s of a 32-layer prefill, seconds per
    step, threads).  Only the quantized Linears are timed, as they are the path being replaced."""
    from oracle import qlinear as OL

    torch.set_num_threads(os.cpu_count() or 1)
    hd, H = cfg["head_dim"], cfg["hidden"]
    shapes = [(cfg["q_heads"] * hd, H), (cfg["kv_heads"] * hd, H), (cfg["kv_heads"] * hd, H), (H, cfg["q_heads"] * hd),
              (cfg["ffn"], H), (cfg["ffn"], H), (H, cfg["ffn"])]  # fmt: skip
    g = torch.Generator().manual_seed(4)
    mods = []
    for n, k in shapes:
        w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
        act = torch.full((k,), 4.0).bfloat16()
        sq = OL.smoothq_scale(act, w, 0.5, torch.bfloat16)
        clip = OL.qmax_clip_after_first_train_forward(w * sq)
        x = torch.randn(tokens, k, generator=g).bfloat16()
        mods.append((x, w, sq, clip))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for x, w, sq, clip in mods:
            OL.qlinear_fakequant_forward(x, w, None, sq, clip)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    per_step = sum(times) / len(times)
    return tokens / (per_step * cfg["layers"]), per_step, torch.get_num_threads()


# ------------------------------------------------------------------------------------------------
def run_reference(args, rank):
    if rank != 0:
        return
    tokens = 256
    tps, per_step, threads = cpu_reference_layer_tokens_per_s(tokens, args.steps, max(1, min(args.warmup, 1)))
    sample = (f"one decoder layer (7 QLinear fake-quant forwards, bf16) on {tokens} tokens per step, "
              f"tokens/s = {tokens} / (step time x 32 layers)")  # fmt: skip
    line = {
        "impl": "reference", "metric": "w8a8_llama3_8b_prefill_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "c5: Llama-3-8B-shaped W8A8 prefill 8x2048", "hardware": "host CPU"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def run_c5(args, rank, world, dev):
    from fms_model_optimizer_b200 import ops

    cfg = dict(LLAMA)
    n_micro = args.micro if args.micro > 0 else (2 if world > 2 else 1)
    if n_micro > 1 and world > 1 and args.allreduce:
        ops.GEMM_MAX_CTAS = args.gemm_ctas
    model = Decoder(cfg, dev, world, rank, layers=args.layers, n_micro=n_micro)
    if world > 1 and not args.allreduce:
        model.exchange = args.exchange
        model.chain = args.chain
        if n_micro > 1 and args.reserve_sms > 0 and args.exchange == "stores":
            # SM partition between the groups' streams: kernels bound by the links (row-parallel GEMMs storing to the
            # peers, the quantiser replicating its codes) run on `reserve` SMs, the compute-bound GEMMs on the rest, so a
            # kernel of each kind fits on the GPU at the same time
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            model.reserve_sms = args.reserve_sms
            for lin in model.layers:
                for name, l_ in lin.items():
                    if hasattr(l_, "max_ctas"):
                        l_.max_ctas = args.reserve_sms if name in ("o", "down") else sms - args.reserve_sms
        model.enable_sequence_parallel(cfg["batch"] * cfg["seq"] // n_micro)
    nl = len(model.layers)
    B, S = cfg["batch"], cfg["seq"]
    tokens = B * S
    g = torch.Generator().manual_seed(4)
    ids_host = torch.randint(0, cfg["vocab"], (B, S), generator=g).pin_memory()
    ids_dev = ids_host.to(dev)
    out_host = torch.empty(B, dtype=torch.int64).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        model.forward(ids_dev)
    barrier()
    ops.check_status(dev)

    # One forward pass as a CUDA graph (sharded runs by default): with the step split over several GPUs the kernels
    # get short enough for the host's launch rate to matter.  Collectives, peer stores and barriers are captured too.
    use_graph = args.graph == "on" or (args.graph == "auto" and world > 1)
    static_ids, static_out, graph = ids_dev.clone(), None, None
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = model.forward(static_ids)
            for _ in range(2):
                graph.replay()
        except Exception as e:  # noqa: BLE001 -- every rank runs the same code, so all of them land here together
            print(f"# CUDA graph capture failed ({type(e).__name__}: {e}); timing eager launches instead", file=sys.stderr, flush=True)
            graph = None
            torch.cuda.synchronize()
        barrier()
        ops.check_status(dev)

    def step(ids):
        if graph is None:
            return model.forward(ids)
        if ids is not static_ids:
            static_ids.copy_(ids, non_blocking=True)
        graph.replay()
        return static_out

    # ---- timed region: device-resident inputs.  Eager runs bracket every kernel launch of this library with CUDA
    # events inside the region; graph runs take those per-launch times from eager steps right after it.
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    ops.PROFILE = [] if graph is None else None
    ops.LAUNCHES = 0
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` capture exactly the timed region
    e0.record()
    for _ in range(args.steps):
        step(static_ids)
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if graph is not None:
        ops.PROFILE = []
        ops.LAUNCHES = 0
        for _ in range(args.steps):
            model.forward(ids_dev)
        barrier()
    prof, ops.PROFILE = ops.PROFILE, None
    launches = ops.LAUNCHES
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()

    # ---- end to end: ids from pinned host memory, next-token ids back to the host, every step
    barrier()
    e0.record()
    for _ in range(args.steps):
        ids_d = ids_host.to(dev, non_blocking=True) if graph is None else static_ids.copy_(ids_host, non_blocking=True)
        out = step(ids_d)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = t.item()
    ops.check_status(dev)
    if rank != 0:
        return

    pk = peaks()
    gemm_ms = sum(a.elapsed_time(b) for (name, a, b, work) in prof if name == "gemm")
    gemm_ops = sum(work for (name, a, b, work) in prof if name == "gemm")
    n_gemm = sum(1 for p in prof if p[0] == "gemm")
    quant_ms = sum(a.elapsed_time(b) for (name, a, b, work) in prof if name in ("act_quant", "block_quant"))
    quant_bytes = sum(work for (name, a, b, work) in prof if name in ("act_quant", "block_quant"))
    achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    if args.breakdown:
        groups = {}
        for name, a, b, work in prof:
            t = groups.setdefault((name, work), [0, 0.0])
            t[0] += 1
            t[1] += a.elapsed_time(b)
        for (name, work), (n, t) in sorted(groups.items(), key=lambda kv: -kv[1][1]):
            print(f"# {name:12s} work {work:.3e} launches/step {n / args.steps:6.1f} avg {1e3 * t / n:8.1f} us  "
                  f"total/step {t / args.steps:7.2f} ms", file=sys.stderr, flush=True)
    peak = 2.0 * pk["bf16_sustained"]
    line = {
        "metric": "w8a8_llama3_8b_prefill_tokens_per_s", "value": tokens * args.steps / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {
            "workload": "c5: Llama-3-8B-shaped decoder, all decoder Linears W8A8 SmoothQuant INT8, prefill 8x2048",
            "layers": nl, "global_batch": B, "seq_len": S, "parallelism": f"tp{world}", "sequence_groups_in_flight": n_micro,
            "timed_region": ("eager launches, per-launch CUDA events inside the region" if graph is None else
                             "CUDA graph replays; per-launch CUDA events from the same number of eager steps right after"),
            "shard_exchange": ("none" if world == 1 else "nccl all-reduce" if args.allreduce else
                               f"peer {args.exchange} over NVLink, residual stream split by tokens, flag barriers"),
            "l2": "inputs larger than L2 (activations 134 MB per Linear, weights 7 GB)",
            "linear_tops": decoder_linear_ops(cfg, tokens, nl) * args.steps / (ms * 1e-3) / 1e12,
        },
        "roofline": {
            "bound": "tensor", "kernel": "qlin_gemm_pair_kernel<int8> (all decoder GEMMs have at least 256 rows)", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak if peak else None, "traffic": None, "launches": n_gemm,
            "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({pk['src']}); no 8-bit peak was measured; "
                           f"datasheet dense int8 4500 TOPS -> frac {achieved / 4500.0:.3f}",
            "gemm_share_of_step": gemm_ms / ms if ms else None,
            "act_quant_gbs": quant_bytes / (quant_ms * 1e-3) / 1e9 if quant_ms > 0 else None,
            "act_quant_share_of_step": quant_ms / ms if ms else None,
        },
        "e2e": {"value": tokens * args.steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": ids_host.numel() * ids_host.element_size(), "d2h_bytes_per_step": out_host.numel() * 8},
        "gpu_launches": launches,
        "clocks": clocks,
    }  # fmt: skip
    if world == 1 and not args.no_cpu_baseline:
        tok = 256
        tps, per_step, threads = cpu_reference_layer_tokens_per_s(tok, 2, 1)
        line["cpu_baseline"] = {
            "value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"one decoder layer (7 QLinear fake-quant forwards, bf16) on {tok} tokens, {per_step:.2f} s per step, "
                      f"extrapolated to 32 layers",
        }  # fmt: skip
    print(json.dumps(line), flush=True)


class BertQAT(torch.nn.Module):
    """BERT-base-shaped encoder (12 layers, hidden 768, 12 heads, FFN 3072) whose 72 Linears are this package's QLinear with
    PACT+ activations (clip values +-6) and SAWB+ per-channel weights: BASELINE config 4.  Embeddings, LayerNorm, GELU and
    attention are PyTorch."""

    def __init__(self, dev, layers=12, hidden=768, heads=12, ffn=3072, vocab=30522, seq=128, dtype=torch.bfloat16):
        super().__init__()
        from fms_model_optimizer_b200.modules import QLinear

        def qlin(i, o):
            return QLinear(i, o, bias=True, num_bits_feature=8, qa_mode="pact+", num_bits_weight=8, qw_mode="sawb+perCh",
                           act_clip_init_val=6.0, act_clip_init_valn=-6.0, device=dev)  # fmt: skip

        self.heads = heads
        self.word = torch.nn.Embedding(vocab, hidden, device=dev)
        self.pos = torch.nn.Embedding(seq, hidden, device=dev)
        self.ln0 = torch.nn.LayerNorm(hidden, device=dev)
        self.blocks = torch.nn.ModuleList()
        for _ in range(layers):
            self.blocks.append(torch.nn.ModuleDict(dict(
                q=qlin(hidden, hidden), k=qlin(hidden, hidden), v=qlin(hidden, hidden), o=qlin(hidden, hidden),
                ln1=torch.nn.LayerNorm(hidden, device=dev), up=qlin(hidden, ffn), down=qlin(ffn, hidden),
                ln2=torch.nn.LayerNorm(hidden, device=dev),
            )))  # fmt: skip
        self.to(dtype)

    def forward(self, ids):
        B, S = ids.shape
        x = self.ln0(self.word(ids) + self.pos(torch.arange(S, device=ids.device))[None])
        for blk in self.blocks:
            def heads(t):
                return t.view(B, S, self.heads, -1).transpose(1, 2)
            a = F.scaled_dot_product_attention(heads(blk["q"](x)), heads(blk["k"](x)), heads(blk["v"](x)))
            x = blk["ln1"](x + blk["o"](a.transpose(1, 2).reshape(B, S, -1)))
            x = blk["ln2"](x + blk["down"](F.gelu(blk["up"](x))))
        return x


def run_c4(args, dev):
    """BASELINE config 4: QAT forward + backward of the BERT-base-shaped encoder on a 32 x 128 batch of random token ids
    (seed 3), random-init weights.  One step = forward, a scalar loss, backward (no optimizer step, as the config says)."""
    from fms_model_optimizer_b200 import ops

    torch.manual_seed(3)
    model = BertQAT(dev, layers=args.layers or 12)
    model.train()
    B, S = 32, 128
    ids = torch.randint(0, 30522, (B, S), device=dev)
    params = [p for p in model.parameters() if p.requires_grad]

    def step():
        for p in params:
            p.grad = None
        loss = model(ids).float().pow(2).mean()
        loss.backward()
        return loss

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ops.check_status(dev)
    sampler = ClockSampler(dev.index)
    sampler.start()
    ops.PROFILE, ops.LAUNCHES = [], 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    prof, ops.PROFILE = ops.PROFILE, None
    clocks = sampler.stop()
    by = {}
    for name, a, b, work in prof:
        t = by.setdefault(name, [0, 0.0, 0.0])
        t[0] += 1
        t[1] += a.elapsed_time(b)
        t[2] += work
    mine_ms = sum(t[1] for t in by.values()) / args.steps
    pact = [by.get(k) for k in ("pact2_fwd", "pact2_bwd") if by.get(k)]
    pact_gbs = sum(t[2] for t in pact) / (sum(t[1] for t in pact) * 1e-3) / 1e9 if pact else None
    pk = peaks()
    print(json.dumps({
        "metric": "qat_bert_base_fwd_bwd_tokens_per_s", "value": B * S / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c4: BERT-base-shaped encoder, 72 QLinear (PACT+ 8-bit activations, SAWB+ per-channel 8-bit weights), "
                               "QAT forward + backward, batch 32 x 128", "layers": len(model.blocks),
                   "l2": "activations 6-25 MB per tensor: L2 resident between kernels, as in the real step",
                   "library_kernels_ms_per_step": mine_ms,
                   "launches_per_step": {k: v[0] / args.steps for k, v in by.items()}},
        "roofline": {"bound": "hbm", "kernel": "pact2_fwd / pact2_bwd", "achieved": pact_gbs, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": (pact_gbs / pk["hbm"]) if pact_gbs else None, "traffic": None,
                     "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({pk['src']}); tensors of this workload fit in L2, so the "
                                    "fraction can exceed what HBM alone would allow"},
        "gpu_launches": ops.LAUNCHES, "clocks": clocks,
    }), flush=True)  # fmt: skip


def run_kernel_workload(args, dev):
    """Single-kernel workloads: c1 (W8A8 Linear 2048x4096x4096), c2 (chunk-truncated int8 GEMM
    4096x8192x4096, chunk 64, 8 bits), c3 (FP8 Linear sweep).  Prints one JSON line per shape."""
    from fms_model_optimizer_b200 import _lib as L, ops

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn, steps, warmup):
        for _ in range(max(warmup, 3)):
            fn()
        torch.cuda.synchronize()
        # the call is replayed as a CUDA graph, as a serving loop would run it: for the small shapes the two or three
        # launches of a Linear take less time on the GPU than the host needs to issue them
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        fn = graph.replay
        fn()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / steps

    cases = []
    if args.workload in ("c1", "c5lin"):
        torch.manual_seed(0)
        M, K, N = (2048, 4096, 4096) if args.workload == "c1" else (16384, 4096, 4096)
        x = torch.randn(M, K, device=dev).bfloat16()
        codes, w_scale, smooth = synth_w8a8(N, K, 0, dev)
        from fms_model_optimizer_b200 import tp

        lin = tp.W8A8Linear(codes, w_scale, smooth, torch.zeros(N, device=dev))
        cases.append((f"{args.workload} W8A8 INT8 Linear {M}x{K}x{N} (quantise + GEMM + dequantise)", 2.0 * M * N * K, lambda: lin(x), "int8"))
    elif args.workload == "c2":
        torch.manual_seed(1)
        M, K, N = 4096, 8192, 4096
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        out = torch.empty((M, N), dtype=torch.int32, device=dev)
        cases.append((f"c2 int8 chunk-truncated GEMM {M}x{K}x{N}, chunk 64, 8 bits", 2.0 * M * N * K,
                      lambda: ops.gemm(a, b, out=out, chunk_k=64, trun_bits=8), "int8"))  # fmt: skip
    else:
        torch.manual_seed(2)
        from fms_model_optimizer_b200.modules import LinearFPxAcc

        for M, K, N in ((1, 4096, 14336), (128, 4096, 4096), (8192, 4096, 14336), (8192, 14336, 4096)):
            x = torch.randn(M, K, device=dev).bfloat16()
            lin = torch.nn.Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16)
            q = LinearFPxAcc.from_nn(lin, trun_bits=0, chunk_size=64, dynamic_fp8="per_token")
            with torch.no_grad():
                q(x)
            cases.append((f"c3 FP8 e4m3 Linear {M}x{K}x{N}", 2.0 * M * N * K, (lambda q=q, x=x: q(x)), "fp8"))
    for name, work, fn, dt in cases:
        with torch.no_grad():
            ms = timeit(fn, args.steps, args.warmup)
        tops = work / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "quantized_linear_tops", "value": tops, "unit": "TOPS", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dt, "data": "synthetic",
            "config": {"workload": name, "l2": "256 MB flush between timed launches", "launch": "CUDA graph replay of the call"},
            "roofline": {"bound": "tensor", "achieved": tops, "peak": 2.0 * pk["bf16"], "unit": "TFLOP/s",
                         "frac": tops / (2.0 * pk["bf16"]),
                         # DRAM bytes of the GEMM launch from the ncu capture of this very shape (profiles/qlin_gemm_pair_*)
                         "traffic": (86.8e6 + 97.6e6) if args.workload == "c5lin" else None,
                         "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({pk['src']})"},
        }), flush=True)  # fmt: skip


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c5", "c1", "c2", "c3", "c4", "c5lin"])
    ap.add_argument("--layers", type=int, default=None, help="development only: fewer decoder layers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the forward pass as one CUDA graph in the timed region (auto: sharded runs only)")
    ap.add_argument("--reserve-sms", type=int, default=0, help="sharded runs with several groups: SMs set aside for the kernels that "
                    "are bound by the links (even; 0: no partition)")
    ap.add_argument("--chain", action="store_true", help="sharded runs with several groups: run the groups' compute segments strictly "
                    "one after the other (event chain) so that one group's transfers overlap the other's kernels")
    ap.add_argument("--exchange", default="stores", choices=["stores", "copies"],
                    help="sharded runs: how partial outputs and codes reach the other GPUs: stores from the GEMM epilogue / the "
                    "quantiser, or copy-engine transfers from local staging")
    ap.add_argument("--breakdown", action="store_true", help="development: per-kernel-shape times of the timed region on stderr")
    ap.add_argument("--allreduce", action="store_true", help="sharded runs: NCCL all-reduce of the row-parallel outputs instead of "
                    "remote stores from the GEMM epilogue with the residual stream split by tokens")
    ap.add_argument("--micro", type=int, default=0, help="groups of sequences pipelined on separate streams (0: 2 on more than two GPUs, else 1)")
    ap.add_argument("--gemm-ctas", type=int, default=132, help="CTAs per GEMM while a collective may run beside it (sharded runs)")
    ap.add_argument("--nccl-ctas", type=int, default=16, help="upper bound on the CTAs of a collective (sharded runs)")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU baseline")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        if args.nccl_ctas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.nccl_ctas))
        import datetime

        # a rank that fails must not leave the others waiting for NCCL's default ten minutes
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    try:
        if args.workload == "c4":
            run_c4(args, dev)
        elif args.workload == "c5":
            run_c5(args, rank, world, dev)
        else:
            run_kernel_workload(args, dev)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
