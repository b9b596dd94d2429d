"""Benchmark of the W8A8 quantized-Linear hot path on B200.

Default workload ("c5"): prefill of a Llama-3-8B-shaped decoder (32 layers, hidden 4096, 32 q / 8 kv
heads of 128, SwiGLU FFN 14336, RMSNorm, RoPE theta 5e5, vocab 128256) whose every Linear inside the
decoder layers is W8A8 SmoothQuant INT8 (alpha 0.5, per-channel weights, per-token activations), on a
batch of 8 x 2048 random token ids.  With N > 1 GPUs the Linears are sharded column / row parallel
(tensor parallel), one process per GPU; the total work is fixed, so scaling is "strong".

    python bench.py --gpus N --steps K --warmup W                  # this implementation
    python bench.py --impl reference --gpus N --steps K --warmup W # reference CPU fake-quant path

One JSON line is printed by rank 0.  `value` is tokens/s of the whole job with the token ids already on
the device; `e2e` is the same with the ids copied from pinned host memory and the next-token ids copied
back inside the timed region.  `roofline` is the int8 GEMM kernel (all its launches in one step, timed
with CUDA events on the launching stream in extra steps right after the timed region).  On one GPU the
line also carries `surfaces` (the same decoder built from QLinear -> lower_qmodel_b200 ->
QLinearINT8Deploy modules), `kernels` (every kernel family on the shapes the metric names, INT8 and FP8,
with its bound and fraction of peak), `comparators` (cuBLASLt int8 and fp8 GEMMs through torch, same run)
and `cpu_baseline` (the reference's CPU fake-quant QLinear.forward for one decoder layer on a bounded
token sample).

Other workloads print single lines: --workload c1 | c2 | c3 | c5lin (one quantized Linear / GEMM), c4
(BERT-base-shaped QAT forward + backward).  Weights and activations are synthetic (seeded); nothing is
read from disk.
"""

from __future__ import annotations

import argparse
import json
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

DATASHEET_8BIT_TOPS = 4500.0  # NVIDIA's dense int8 / fp8 figure for one B200
# DRAM bytes per launch of the CTA-pair int8 GEMM on 16384 x 4096 x 4096 with bf16 output from its ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum, profiles/qlin_gemm_pair_int8_c5lin_16384x4096x4096.md), and the
# algorithmic bytes of that launch (A + B + D)
C5LIN_DRAM_BYTES = 86.8e6 + 97.6e6
C5LIN_ALGO_BYTES = 16384 * 4096 + 4096 * 4096 + 16384 * 4096 * 2


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
        return self

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
# CPU arm: the reference's fake-quant QLinear on the host cores
# ------------------------------------------------------------------------------------------------
def _reference_qlinear_class():
    """fms-model-optimizer's own QLinear when the reference was installed under baseline/_ref (it is not part of this
    repository's history), else None."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "fms_mo").is_dir():
        return None
    sys.path.insert(0, str(ref))
    try:
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            from fms_mo.modules.linear import QLinear  # noqa: PLC0415
        return QLinear
    except Exception as e:  # noqa: BLE001
        print(f"# reference import failed ({type(e).__name__}: {e}); timing the port instead", file=sys.stderr, flush=True)
        return None
    finally:
        sys.path.remove(str(ref))


def cpu_layer_tokens_per_s(tokens: int, steps: int, warmup: int):
    """Times the seven fake-quant QLinear forwards of one decoder layer (QLinear.forward, fms_mo/modules/linear.py:248-305,
    qa_mode pertokenmax / qw_mode maxperCh / SmoothQuant, bf16) on `tokens` tokens with all host threads.  Runs the
    reference's own class when it is installed under baseline/_ref (kind "reference"), else the oracle's restatement of
    it (kind "port").  Returns (tokens/s of a 32-layer prefill, seconds per step, threads, kind).  Only the quantized
    Linears are timed, as they are the path being replaced."""
    from fms_model_optimizer_b200.decoder import LLAMA3_8B, linear_shapes

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(4)
    QLinear = _reference_qlinear_class()
    kind = "reference" if QLinear is not None else "port"
    calls = []
    for n, k, _ in linear_shapes(LLAMA3_8B).values():
        w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
        act = torch.full((k,), 4.0).bfloat16()
        x = torch.randn(tokens, k, generator=g).bfloat16()
        if QLinear is not None:
            lin = QLinear(k, n, bias=False, num_bits_feature=8, qa_mode="pertokenmax", num_bits_weight=8, qw_mode="maxperCh",
                          qcfg={"smoothq": True, "smoothq_alpha": 0.5}, device="cpu")  # fmt: skip
            with torch.no_grad():
                lin.weight.copy_(w)
            lin = lin.to(torch.bfloat16)
            lin.set_act_scale(act.float())
            lin.train()
            with torch.no_grad():
                lin(x[:1])  # latches the weight clip values (fms_mo/quant/quantizers.py:3098-3104)
            lin.eval()
            calls.append((lin, x))
        else:
            from oracle import qlinear as OL

            sq = OL.smoothq_scale(act, w, 0.5, torch.bfloat16)
            clip = OL.qmax_clip_after_first_train_forward(w * sq)
            calls.append(((lambda x_, w=w, sq=sq, clip=clip: OL.qlinear_fakequant_forward(x_, w, None, sq, clip)), x))
    times = []
    with torch.no_grad():
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            for fn, x in calls:
                fn(x)
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    return tokens / (per_step * LLAMA3_8B["layers"]), per_step, torch.get_num_threads(), kind


CPU_SAMPLE_TOKENS = 2048


def run_reference(args, rank):
    if rank != 0:
        return
    tokens = CPU_SAMPLE_TOKENS
    tps, per_step, threads, kind = cpu_layer_tokens_per_s(tokens, max(1, args.steps), 1)
    sample = (f"one decoder layer (7 QLinear fake-quant forwards, bf16) on {tokens} tokens per step, "
              f"tokens/s = {tokens} / (step time x 32 layers)")  # fmt: skip
    line = {
        "impl": "reference", "metric": "w8a8_llama3_8b_prefill_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": 1, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "c5: Llama-3-8B-shaped decoder, all decoder Linears W8A8 SmoothQuant INT8, prefill 8x2048",
                   "hardware": "host CPU", "sample": sample},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# single kernels
# ------------------------------------------------------------------------------------------------
class KernelTimer:
    """Times one call as a CUDA graph replay (the way a serving loop issues it: for small shapes the launches of a
    Linear take less GPU time than the host needs to queue them), with a 256 MB write between replays so that nothing
    is served from L2.  Cases that walk through several weight sets larger than L2 in one call need no such write
    (flush=False): every set has been evicted, clean, by the time its turn comes again."""

    def __init__(self, dev):
        self.dev = dev
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self, fn, steps=5, warmup=3, graph=True, flush=True):
        with torch.no_grad():
            for _ in range(max(warmup, 3)):
                fn()
            torch.cuda.synchronize()
            run = fn
            if graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    fn()
                run = g.replay
                run()
                torch.cuda.synchronize()
            tot = 0.0
            for _ in range(steps):
                if flush:
                    self.flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run()
                e1.record()
                torch.cuda.synchronize()
                tot += e0.elapsed_time(e1)
        return tot / steps


def kernel_cases(dev, which, only=""):
    """(name, dtype, bound, work, unit_scale, fn) for the single-kernel workloads: work is operations for tensor-bound
    entries and algorithmic bytes for HBM-bound ones."""
    from fms_model_optimizer_b200 import _lib as L, ops, tp
    from fms_model_optimizer_b200.decoder import synth_w8a8
    from fms_model_optimizer_b200.modules import LinearFPxAcc

    cases = []

    def add(name, dtype, bound, work, fn, graph=True):
        cases.append(dict(name=name, dtype=dtype, bound=bound, work=float(work), fn=fn, graph=graph))

    def wanted(prefix):
        """False when --only names another case: such a case is not even built (its set-up launches kernels too)."""
        return not only or only.startswith(prefix) or prefix.startswith(only)

    if which in ("c1", "c5lin", "all"):
        for tag, (M, K, N) in (("c1", (2048, 4096, 4096)), ("c5lin", (16384, 4096, 4096))):
            if which not in (tag, "all") or not wanted(tag):
                continue
            torch.manual_seed(0)
            x = torch.randn(M, K, device=dev).bfloat16()
            codes, w_scale, smooth = synth_w8a8(N, K, 0, dev)
            lin = tp.W8A8Linear(codes, w_scale, smooth, torch.zeros(N, device=dev))
            add(f"{tag} W8A8 INT8 Linear {M}x{K}x{N} (quantise + GEMM + dequantise)", "int8", "tensor", 2.0 * M * N * K, lambda lin=lin, x=x: lin(x))
    if which in ("c2", "all") and wanted("c2"):
        torch.manual_seed(1)
        M, K, N = 4096, 8192, 4096
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        out = torch.empty((M, N), dtype=torch.int32, device=dev)
        add(f"c2 int8 chunk-truncated GEMM {M}x{K}x{N}, chunk 64, 8 bits", "int8", "tensor", 2.0 * M * N * K,
            lambda a=a, b=b, out=out: ops.gemm(a, b, out=out, chunk_k=64, trun_bits=8))  # fmt: skip
    if which in ("c3", "all"):
        torch.manual_seed(2)
        for M, K, N in ((1, 4096, 14336), (1, 14336, 4096), (128, 4096, 4096), (128, 4096, 14336), (8192, 4096, 14336), (8192, 14336, 4096)):
            if not wanted(f"c3 FP8 e4m3 Linear {M}x{K}x{N}"):
                continue
            x = torch.randn(M, K, device=dev).bfloat16()
            lin = torch.nn.Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(N, K, device=dev))
            q = LinearFPxAcc.from_nn(lin, trun_bits=0, chunk_size=64, dynamic_fp8="per_token")
            with torch.no_grad():
                q(x)
            small = M <= 128
            if small:
                # decode-sized: the weights are the traffic.  One call walks through R independent Linears (R weight sets,
                # together several times L2), so each launch streams its weights from HBM and the fixed cost of timing one
                # tiny launch alone is spread over R of them; the figures are per Linear.
                R = max(8, -(-3 * 126_000_000 // (N * K)))
                qs = [q]
                for _ in range(R - 1):
                    with torch.no_grad():
                        lin.weight.copy_(torch.randn(N, K, device=dev))
                    qs.append(LinearFPxAcc.from_nn(lin, trun_bits=0, chunk_size=64, dynamic_fp8="per_token"))
                    with torch.no_grad():
                        qs[-1](x)
                del lin
                add(f"c3 FP8 e4m3 Linear {M}x{K}x{N} (quantise + GEMM + dequantise), {R} weight sets in rotation", "fp8", "hbm",
                    N * K + M * K * 3 + M * N * 2, (lambda qs=qs, x=x: [qq(x) for qq in qs]))  # fmt: skip
                cases[-1].update(ops=2.0 * M * N * K, calls=R, flush=False)
                continue
            add(f"c3 FP8 e4m3 Linear {M}x{K}x{N} (quantise + GEMM + dequantise)", "fp8", "tensor", 2.0 * M * N * K, (lambda q=q, x=x: q(x)))
    if which == "all":
        for M, K, N in ((16384, 4096, 4096), (8192, 8192, 8192)):
            for kind, dt in (("int8", torch.int8), ("fp8", torch.float8_e4m3fn)):
                a = torch.randint(-100, 100, (M, K), dtype=torch.int8, device=dev)
                b = torch.randint(-100, 100, (N, K), dtype=torch.int8, device=dev)
                if kind == "fp8":
                    a, b = (a.float() / 64).to(dt), (b.float() / 64).to(dt)
                rs, cs = torch.rand(M, device=dev) + 0.5, torch.rand(N, device=dev) + 0.5
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                add(f"GEMM {kind} {M}x{K}x{N}, bf16 output, scale epilogue", kind, "tensor", 2.0 * M * N * K,
                    lambda a=a, b=b, rs=rs, cs=cs, out=out: ops.gemm(a, b, out=out, epilogue=L.EPI_SCALE_SEQ, row_scale=rs, col_scale=cs,
                                                                      out_dtype=torch.bfloat16))  # fmt: skip
        # batched integer matmul of attention shapes (QBmmINT8Deploy): 64 heads of one 2048-token sequence each
        for tag, (Bh, M, N, K) in (("q.k^T", (64, 2048, 2048, 128)), ("p.v", (64, 2048, 128, 2048))):
            a3 = torch.randint(-100, 100, (Bh, M, K), dtype=torch.int8, device=dev)
            b3 = torch.randint(-100, 100, (Bh, N, K), dtype=torch.int8, device=dev)
            byts = Bh * (M * K + N * K + 4 * M * N)
            add(f"bmm_i8 {tag} {Bh}x{M}x{K}x{N}, int32 output, one launch", "int8", "hbm" if tag == "q.k^T" else "tensor",
                byts if tag == "q.k^T" else 2.0 * Bh * M * N * K, lambda a3=a3, b3=b3: ops.bmm_i8(a3, b3))
            cases[-1]["ops"] = 2.0 * Bh * M * N * K
        # HBM-bound kernels on c5 / c4 shaped tensors (larger than L2)
        M, K = 16384, 4096
        x = torch.randn(M, K, device=dev).bfloat16()
        r = torch.randn(M, K, device=dev).bfloat16()
        nw = torch.ones(K, device=dev, dtype=torch.bfloat16)
        rc = [ops.smooth_reciprocal((torch.rand(K, device=dev) + 0.5).bfloat16().float()) for _ in range(3)]
        sm = (torch.rand(K, device=dev) + 0.5).bfloat16().float()
        smr = ops.smooth_reciprocal(sm)
        add(f"act_quant bf16 per-token int8 with SmoothQuant {M}x{K}", "bf16", "hbm", M * K * 3 + 4 * M + 4 * K,
            lambda x=x, sm=sm, smr=smr: ops.act_quant(x, mode=L.Q_I8_DYN, smooth=sm, smooth_rcp=smr, native_chain=7))  # fmt: skip
        add(f"block_quant add+RMSNorm+3 outputs {M}x{K}", "bf16", "hbm", M * K * (2 + 2 + 2 + 3) + 12 * M,
            lambda x=x, r=r, nw=nw, rc=rc: ops.block_quant(x, prologue=L.BLOCK_NORM, r=r, norm_w=nw, smooth_rcps=rc, store_sum=True))  # fmt: skip
        add(f"block_quant add+RMSNorm+2 outputs {M}x{K}", "bf16", "hbm", M * K * (2 + 2 + 2 + 2) + 8 * M,
            lambda x=x, r=r, nw=nw, rc=rc: ops.block_quant(x, prologue=L.BLOCK_NORM, r=r, norm_w=nw, smooth_rcps=rc[:2], store_sum=True))  # fmt: skip
        add(f"block_quant SiLU*up+1 output {M}x{K}", "bf16", "hbm", M * K * (2 + 2 + 1) + 4 * M,
            lambda x=x, r=r, rc=rc: ops.block_quant(x, prologue=L.BLOCK_SILU_MUL, r=r, smooth_rcps=rc[:1]))  # fmt: skip
        add(f"block_quant plain 1 output {M}x{K}", "bf16", "hbm", M * K * (2 + 1) + 4 * M,
            lambda x=x, rc=rc: ops.block_quant(x, prologue=L.BLOCK_PLAIN, smooth_rcps=rc[:1]))  # fmt: skip
        for dt, name in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
            xx = (torch.randn(M, K, device=dev) * 3).to(dt)
            gg = torch.randn(M, K, device=dev).to(dt)
            cv, cvn = torch.tensor([6.0], device=dev), torch.tensor([-6.0], device=dev)
            es = xx.element_size()
            add(f"PACT+ forward {name} {M}x{K}", name, "hbm", 2 * es * M * K, lambda xx=xx, cv=cv, cvn=cvn: ops.pact2_fwd(xx, cv, cvn, 8, True))
            add(f"PACT+ backward {name} {M}x{K}", name, "hbm", 3 * es * M * K, lambda xx=xx, gg=gg, cv=cv, cvn=cvn: ops.pact2_bwd(xx, gg, cv, cvn, 8, True))
            w = (torch.randn(14336, 4096, device=dev) * 0.02).to(dt)
            add(f"SAWB+ per-channel weight fake-quant {name} 14336x4096", name, "hbm", 2 * es * w.numel(),
                lambda w=w: ops.weight_fq_perch(w, num_bits=8, mode=L.W_SAWB, c0=SAWB_C[0], c1=SAWB_C[1]))  # fmt: skip
    return cases


SAWB_C = (31.76, -35.04)  # the 8-bit coefficients of sawb_params_code (fms_mo/quant/quantizers.py:639): clip = c0 * rms + c1 * mean|w|


def comparator_cases(dev):
    """Library GEMMs on the same shapes, same run: cuBLASLt int8 through torch._int_mm (the call the reference's
    ext_kernel_cublas.cpp:172-187 makes) and cuBLASLt fp8 through torch._scaled_mm, both as plain GEMMs."""
    out = []
    for M, K, N in ((16384, 4096, 4096), (8192, 8192, 8192)):
        a = torch.randint(-100, 100, (M, K), dtype=torch.int8, device=dev)
        b = torch.randint(-100, 100, (N, K), dtype=torch.int8, device=dev)
        out.append(dict(name=f"torch._int_mm (cuBLASLt int8 -> int32) {M}x{K}x{N}", dtype="int8", work=2.0 * M * N * K,
                        fn=lambda a=a, b=b: torch._int_mm(a, b.t())))  # fmt: skip
        a8, b8 = (a.float() / 64).to(torch.float8_e4m3fn), (b.float() / 64).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        out.append(dict(name=f"torch._scaled_mm (cuBLASLt e4m3 -> bf16) {M}x{K}x{N}", dtype="fp8", work=2.0 * M * N * K,
                        fn=lambda a8=a8, b8=b8: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)))  # fmt: skip
    return out


def measure_kernels(dev, which="all", steps=5, warmup=3, with_comparators=True, only=""):
    """Runs the single-kernel cases and returns (kernels, comparators): lists of dicts with TOPS or GB/s, the bound and
    the fraction of the stated peak."""
    pk = peaks()
    timer = KernelTimer(dev)
    kernels, comps = [], []
    for c in kernel_cases(dev, which, only):
        if only and only not in c["name"]:
            c["fn"] = None
            continue
        ms = timer(c["fn"], steps, warmup, c["graph"], c.get("flush", True)) / c.get("calls", 1)
        e = {"name": c["name"], "dtype": c["dtype"], "bound": c["bound"], "us": ms * 1e3}
        if not c.get("flush", True):
            e["l2"] = f"{c['calls']} weight sets (several times L2) used in rotation inside one CUDA graph; figures per Linear"
        if c["bound"] == "tensor":
            tops = c["work"] / (ms * 1e-3) / 1e12
            e.update(tops=tops, frac_of_2x_bf16_measured=tops / (2 * pk["bf16"]), frac_of_datasheet_8bit=tops / DATASHEET_8BIT_TOPS)
        else:
            gbs = c["work"] / (ms * 1e-3) / 1e9
            e.update(gbs=gbs, frac_of_hbm_measured=gbs / pk["hbm"], algorithmic_bytes=c["work"])
            if "ops" in c:
                e["tops"] = c["ops"] / (ms * 1e-3) / 1e12
        kernels.append(e)
        c["fn"] = None
    if with_comparators:
        for c in comparator_cases(dev):
            try:
                ms = timer(c["fn"], steps, warmup, True)
                tops = c["work"] / (ms * 1e-3) / 1e12
                comps.append({"name": c["name"], "dtype": c["dtype"], "us": ms * 1e3, "tops": tops,
                              "frac_of_datasheet_8bit": tops / DATASHEET_8BIT_TOPS})  # fmt: skip
            except Exception as e:  # noqa: BLE001 -- a library call this torch build does not offer
                comps.append({"name": c["name"], "unavailable": f"{type(e).__name__}: {e}"[:200]})
            c["fn"] = None
    torch.cuda.empty_cache()
    return kernels, comps


def run_kernel_workload(args, dev):
    """--workload c1 | c2 | c3 | c5lin: one JSON line per shape.  --workload kernels: every single-kernel case (or the ones
    whose name contains --only), one line each; this is also the command the ncu captures under profiles/ run."""
    pk = peaks()
    sampler = ClockSampler(dev.index).start()
    which = "all" if args.workload == "kernels" else args.workload
    kernels, _ = measure_kernels(dev, which, args.steps, args.warmup, with_comparators=False, only=args.only)
    clocks = sampler.stop()
    for e in kernels:
        tensor = e["bound"] == "tensor"
        val = e["tops"] if tensor else e["gbs"]
        peak = 2.0 * pk["bf16"] if tensor else pk["hbm"]
        print(json.dumps({
            "metric": "quantized_linear_tops" if tensor else "quantized_linear_weight_stream_gbs", "value": val,
            "unit": "TOPS" if tensor else "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": e["us"] * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": e["dtype"],
            "data": "synthetic",
            "config": {"workload": e["name"], "l2": e.get("l2", "256 MB flush between timed launches"), "launch": "CUDA graph replay of the call"},
            "roofline": {"bound": e["bound"], "achieved": val, "peak": peak, "unit": "TFLOP/s" if tensor else "GB/s", "frac": val / peak,
                         "traffic": C5LIN_DRAM_BYTES if args.workload == "c5lin" else None,
                         "peak_source": (f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({pk['src']}); datasheet dense 8-bit "
                                         f"{DATASHEET_8BIT_TOPS:.0f} -> frac {val / DATASHEET_8BIT_TOPS:.3f}") if tensor else
                                        f"hbm_gbs of MEASURED_PEAKS.json ({pk['src']})"},
            "clocks": clocks,
        }), flush=True)  # fmt: skip


# ------------------------------------------------------------------------------------------------
# c5: decoder prefill
# ------------------------------------------------------------------------------------------------
def _calibrated_scales(args, cfg, world, dev, ids_dev, layers):
    """SmoothQuant activation scales from one calibration forward of the float model on the first two sequences of the
    batch (``decoder.calibrate_act_scales``); sharded runs take rank 0's vectors so that every shard smooths alike."""
    from fms_model_optimizer_b200.decoder import calibrate_act_scales

    if args.act_scales != "calibrated":
        return None
    scales = calibrate_act_scales(cfg, dev, ids_dev[:2], layers)
    if world > 1:
        keys = sorted(scales)
        flat = torch.cat([scales[k] for k in keys])
        dist.broadcast(flat, src=0)
        off = 0
        for k in keys:
            n = scales[k].numel()
            scales[k] = flat[off : off + n].clone()
            off += n
    torch.cuda.empty_cache()
    return scales


def _check_sharded_against_single(args, cfg, rank, world, dev, ids_dev, groups, scales):
    """Before timing a sharded run: a 2-layer decoder through the sharded path (eager and as a CUDA graph replay) and
    through the one-GPU path (every rank holds the full 2-layer weights), same ids.

    The sharp check is the residual stream after the first attention block (``x_mlp_in`` of layer 0): up to there the
    sharded run computes the same codes and integer accumulators as the one-GPU run, and the only difference is that
    every shard's partial output is rounded to bf16 before the sum -- a relative error of the order of 1e-3; a wrong offset,
    a stale buffer or a missed barrier shows there as an error of order 1.  It must be below 2e-2 (3.3e-3 measured on two GPUs).  From then on a last-
    place difference in a normalised row flips int8 codes and the two runs drift apart like any two roundings of the same
    model (a few per cent after two layers, which is also what a CPU run of the same layers in another order shows);
    the final hidden state is reported and only has to be the same model (below 0.2)."""
    from fms_model_optimizer_b200 import ops
    from fms_model_optimizer_b200.decoder import W8A8Decoder

    single = W8A8Decoder(cfg, dev, 1, 0, layers=2, calibrated_act_scales=scales)
    single.trace = []
    want_ids = single.forward(ids_dev)
    want_h = single.last_hidden.float().clone()
    want_x = [t for tag, li, t in single.trace if tag == "x_mlp_in" and li == 0][0].float()
    del single
    sharded = W8A8Decoder(cfg, dev, world, rank, layers=2, groups=groups, exchange=args.exchange, reserve_sms=args.reserve_sms,
                          calibrated_act_scales=scales)
    if sharded.exchange != "allreduce":
        sharded.enable_token_split(cfg["batch"] * cfg["seq"] // groups)
    res = {"exchange": sharded.exchange}
    T = cfg["batch"] * cfg["seq"]
    for mode in ("eager", "graph"):
        if mode == "graph":
            sharded.trace = None
            static_ids = ids_dev.clone()
            sharded.forward(static_ids)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                got_ids = sharded.forward(static_ids)
            gr.replay()
        else:
            sharded.trace = []
            got_ids = sharded.forward(ids_dev)
        torch.cuda.synchronize()
        ops.check_status(dev)
        err = ((sharded.last_hidden.float() - want_h).norm() / want_h.norm()).item()
        res[mode] = {"final_hidden_rel_err": err, "next_tokens_equal": bool(torch.equal(got_ids, want_ids))}
        if mode == "eager":
            xs = [t for tag, li, t in sharded.trace if tag == "x_mlp_in" and li == 0]  # one per group, in group order
            worst = 0.0
            for gi, t in enumerate(xs):
                if sharded.exchange == "allreduce":  # every rank holds all tokens of the group
                    w = want_x[gi * (T // groups) : (gi + 1) * (T // groups)]
                else:  # this rank's token block of the group
                    Ts = T // groups // world
                    w = want_x[gi * (T // groups) + rank * Ts : gi * (T // groups) + (rank + 1) * Ts]
                worst = max(worst, ((t.float() - w).norm() / w.norm()).item())
            res[mode]["first_exchange_rel_err"] = worst
            if not worst < 2e-2:
                raise RuntimeError(f"sharded forward: residual stream after the first exchange differs from the one-GPU run by {worst}")
        if not err < 0.2:
            raise RuntimeError(f"sharded forward ({mode}) differs from the one-GPU forward: relative error {err}")
    dist.barrier()
    sharded.close()
    del sharded
    torch.cuda.empty_cache()
    return res


def run_c5(args, rank, world, dev):
    from fms_model_optimizer_b200 import ops
    from fms_model_optimizer_b200.decoder import LLAMA3_8B, W8A8Decoder, decoder_linear_ops, linear_shapes

    cfg = dict(LLAMA3_8B)
    # measured on 8 x B200: two groups of sequences in flight up to four GPUs, four groups at eight
    groups = args.groups if args.groups > 0 else (4 if world >= 8 else (2 if world > 1 else 1))
    B, S = cfg["batch"], cfg["seq"]
    tokens = B * S
    g = torch.Generator().manual_seed(4)
    ids_host = torch.randint(0, cfg["vocab"], (B, S), generator=g).pin_memory()
    ids_dev = ids_host.to(dev)
    out_host = torch.empty(B, dtype=torch.int64).pin_memory()

    scales = _calibrated_scales(args, cfg, world, dev, ids_dev, args.layers)
    check = None
    if world > 1 and not args.no_check:
        check = _check_sharded_against_single(args, cfg, rank, world, dev, ids_dev, groups, scales)

    model = W8A8Decoder(cfg, dev, world, rank, layers=args.layers, groups=groups, exchange=args.exchange, reserve_sms=args.reserve_sms,
                        surface=("fused" if args.surface == "both" else args.surface), calibrated_act_scales=scales)  # fmt: skip
    if world > 1 and model.exchange != "allreduce":
        model.enable_token_split(tokens // groups)
    nl = len(model.layers)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """`steps` calls of fn between two CUDA events on the current stream, bracketed by barrier + synchronize; the
        maximum over the ranks, in ms."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

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

    timed_as = "eager launches" if graph is None else "CUDA graph replays"

    def step(ids=None):
        if graph is None:
            return model.forward(static_ids if ids is None else ids)
        if ids is not None and ids is not static_ids:
            static_ids.copy_(ids, non_blocking=True)
        graph.replay()
        return static_out

    # ---- timed region: device-resident inputs, no instrumentation inside
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    ops.PROFILE, ops.LAUNCHES = None, 0
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` capture exactly the timed region
    ms = timed(step, args.steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: ids from pinned host memory, next-token ids back to the host, every step
    def e2e_step():
        ids_d = ids_host.to(dev, non_blocking=True) if graph is None else static_ids.copy_(ids_host, non_blocking=True)
        out = step(ids_d)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_e2e = timed(e2e_step, args.steps)
    ops.check_status(dev)

    # ---- per-launch times: the same number of eager steps with every launch of this library bracketed by CUDA events on
    # its stream (the event pairs cost time, so these steps are not part of `value`)
    ops.PROFILE, ops.LAUNCHES = [], 0
    barrier()
    for _ in range(args.steps):
        model.forward(ids_dev)
    barrier()
    prof, ops.PROFILE = ops.PROFILE, None
    launches = ops.LAUNCHES // args.steps
    ops.check_status(dev)

    head_exchange, head_nvlink = model.exchange, getattr(model, "nvlink_bytes_per_forward", None)
    sweep = []
    if world > 1 and args.sweep and model.exchange != "allreduce":
        # other settings of the sharded run on the same weights: "g<groups>r<reserved SMs>[s]" ("s": plain stores)
        for spec in args.sweep.split(","):
            gi, ri = spec.index("g"), spec.index("r")
            sg, sr = int(spec[gi + 1 : ri]), int(spec[ri + 1 :].rstrip("sfnk").split("t")[0])
            graph = None
            model.reconfigure(groups=sg, reserve_sms=sr, exchange=("stores" if spec.endswith("s") else "multimem"))
            model.switch_reduce = "fused" if spec.endswith("f") else "split"  # "f": the switch reduce inside the norm + quantise kernel
            model.k_on_side_stream = spec.endswith("k")  # "k": the k projection on a second side stream
            model.stagger = 0 if spec.endswith("n") else (int(spec.split("t")[1].rstrip("sfnk")) if "t" in spec else 2)  # "n": groups start together; "t<k>": k segments apart
            model.enable_token_split(tokens // sg)
            for _ in range(3):
                model.forward(ids_dev)
            barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                model.forward(static_ids)
            gr.replay()
            ms_v = timed(gr.replay, args.steps) / args.steps
            ops.check_status(dev)
            sweep.append({"groups": sg, "reserve_sms": sr, "exchange": model.exchange, "switch_reduce": model.switch_reduce, "stagger": model.stagger, "k_on_side_stream": model.k_on_side_stream, "ms_per_step": ms_v, "tokens_per_s": tokens / (ms_v * 1e-3)})
            del gr

    surfaces = None
    if world == 1 and args.surface == "both":
        # the same decoder by the drop-in route: QLinear -> lower_qmodel_b200 -> QLinearINT8Deploy, unfused norms
        graph = None
        model.layers.clear()
        torch.cuda.empty_cache()
        surfaces = {"fused": {"tokens_per_s": tokens * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
                              "what": "tp.W8A8Linear fed by the fused block kernels (the headline)"}}  # fmt: skip
        try:
            mod = W8A8Decoder(cfg, dev, 1, 0, layers=args.layers, surface="modules", calibrated_act_scales=scales)
            for _ in range(3):
                mod.forward(ids_dev)
            n_mod = max(2, args.steps // 2)
            ms_mod = timed(lambda: mod.forward(ids_dev), n_mod) / n_mod
            surfaces["modules"] = {"tokens_per_s": tokens / (ms_mod * 1e-3), "ms_per_step": ms_mod,
                                   "what": "QLinear -> lower_qmodel_b200 -> QLinearINT8Deploy per Linear; RMSNorm, SiLU*up, residual adds "
                                           "as PyTorch ops"}  # fmt: skip
            del mod
        except Exception as e:  # noqa: BLE001 -- the headline stands on its own
            surfaces["modules"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()
    if world > 1:
        model.close()
    if rank != 0:
        return

    pk = peaks()
    gemm_ms = sum(a.elapsed_time(b) for (name, a, b, work) in prof if name == "gemm")
    gemm_ops = sum(work for (name, a, b, work) in prof if name == "gemm")
    n_gemm = sum(1 for p in prof if p[0] == "gemm")
    quant_ms = sum(a.elapsed_time(b) for (name, a, b, work) in prof if name in ("act_quant", "block_quant"))
    quant_bytes = sum(work for (name, a, b, work) in prof if name in ("act_quant", "block_quant"))
    bar_ms = sum(a.elapsed_time(b) for (name, a, b, work) in prof if name == "barrier")
    prof_ms = sum(a.elapsed_time(b) for (name, a, b, work) in prof)
    achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    if args.breakdown:
        by = {}
        for name, a, b, work in prof:
            t = by.setdefault((name, work), [0, 0.0])
            t[0] += 1
            t[1] += a.elapsed_time(b)
        for (name, work), (n, t) in sorted(by.items(), key=lambda kv: -kv[1][1]):
            print(f"# {name:12s} work {work:.3e} launches/step {n / args.steps:6.1f} avg {1e3 * t / n:8.1f} us  "
                  f"total/step {t / args.steps:7.2f} ms", file=sys.stderr, flush=True)
    # algorithmic bytes of the GEMM launches of one step on this rank (A codes + B codes + bf16 output)
    algo = 0.0
    for n, k, mode in linear_shapes(cfg).values():
        n_r, k_r = (n // world, k) if mode == "column" else (n, k // world)
        algo += tokens * k_r + n_r * k_r + tokens * n_r * 2
    traffic = algo / 7 * (C5LIN_DRAM_BYTES / C5LIN_ALGO_BYTES)  # seven GEMM launches per layer
    peak = 2.0 * pk["bf16_sustained"]
    line = {
        "metric": "w8a8_llama3_8b_prefill_tokens_per_s", "value": tokens * args.steps / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {
            "workload": "c5: Llama-3-8B-shaped decoder, all decoder Linears W8A8 SmoothQuant INT8, prefill 8x2048",
            "layers": nl, "global_batch": B, "seq_len": S, "parallelism": f"tp{world}", "sequence_groups_in_flight": groups,
            "surface": model.surface,
            "smoothquant_act_scales": ("per-channel absmax from one calibration forward of the float model on 2 x 2048 tokens of the batch "
                                       "(qlin_col_absmax)" if scales is not None else "synthetic: 4.0 with 1 % outlier channels x20"),
            "timed_region": timed_as + ", no instrumentation; per-launch CUDA events (roofline, shares) from the same number of eager steps right after",
            "shard_exchange": {"none": "none", "allreduce": "nccl all-reduce",
                               "multimem": "token-split residual stream; partial sums reduced in the NVLink switch (multimem.ld_reduce), "
                                           "codes replicated with multimem.st, flag barriers",
                               "stores": "token-split residual stream; plain peer stores over NVLink, flag barriers"}[head_exchange],
            "reserve_sms": args.reserve_sms,
            "l2": "inputs larger than L2 (activations 134 MB per Linear, weights 7 GB)",
            "linear_tops": decoder_linear_ops(cfg, tokens, nl) * args.steps / (ms * 1e-3) / 1e12,
        },
        "roofline": {
            "bound": "tensor", "kernel": "qlin_gemm_pair_kernel<int8> (all decoder GEMMs have at least 256 rows)", "achieved": achieved,
            "peak": DATASHEET_8BIT_TOPS, "unit": "TFLOP/s", "frac": achieved / DATASHEET_8BIT_TOPS, "traffic": traffic, "launches": n_gemm // args.steps,
            "peak_source": "datasheet dense INT8 of the B200 (4500 TOPS at 1965 MHz): MEASURED_PEAKS.json holds no 8-bit tensor peak; "
                           "frac_of_2x_bf16_sustained_measured uses twice its bf16_tflops_sustained as a measured proxy, and on one GPU "
                           "`comparators` gives cuBLASLt int8 in the same run",
            "frac_of_2x_bf16_sustained_measured": achieved / peak if peak else None,
            "peak_2x_bf16_sustained_measured": peak, "peak_measured_source": pk["src"],
            "traffic_source": "average DRAM bytes per GEMM launch, scaled from the ncu capture of the 16384x4096x4096 launch "
                              "(184.4 MB measured for 218.1 MB algorithmic: part of the output is still in L2 when the kernel ends) "
                              "by each shape's algorithmic bytes",
            "gemm_ms_per_step": gemm_ms / args.steps,
            "act_quant_gbs": quant_bytes / (quant_ms * 1e-3) / 1e9 if quant_ms > 0 else None,
            "act_quant_ms_per_step": quant_ms / args.steps,
            "shares_of_instrumented_kernel_time": {"gemm": gemm_ms / prof_ms, "quantise": quant_ms / prof_ms, "barrier": bar_ms / prof_ms} if prof_ms else None,
        },
        "e2e": {"value": tokens * args.steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": ids_host.numel() * ids_host.element_size(), "d2h_bytes_per_step": out_host.numel() * 8},
        "gpu_launches": launches * args.steps,
        "clocks": clocks,
    }  # fmt: skip
    if world > 1 and head_exchange in ("multimem", "stores"):
        out_b, in_b = head_nvlink
        line["nvlink"] = {
            "bytes_out_per_step": out_b, "bytes_in_per_step": in_b,
            "achieved_gbs_in": in_b / (ms / args.steps * 1e-3) / 1e9, "achieved_gbs_out": out_b / (ms / args.steps * 1e-3) / 1e9,
            "link_bound_ms_per_step_at_770_gbs": max(out_b, in_b) / 770e9 * 1e3,
            "barrier_ms_per_step_eager": bar_ms / args.steps,
            "barriers_per_step": sum(1 for p in prof if p[0] == "barrier") // args.steps,
        }  # fmt: skip
    if check is not None:
        line["sharded_vs_single_gpu"] = check
    if sweep:
        line["sweep"] = sweep
    if surfaces is not None:
        line["surfaces"] = surfaces
    if world == 1 and not args.no_kernels:
        try:
            line["kernels"], line["comparators"] = measure_kernels(dev, "all", 5, 3)
        except Exception as e:  # noqa: BLE001 -- the headline stands on its own
            line["kernels"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if world == 1 and not args.no_cpu_baseline:
        tps, per_step, threads, kind = cpu_layer_tokens_per_s(CPU_SAMPLE_TOKENS, 2, 1)
        line["cpu_baseline"] = {
            "value": tps, "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"one decoder layer (7 QLinear fake-quant forwards, bf16) on {CPU_SAMPLE_TOKENS} tokens, {per_step:.2f} s per step, "
                      f"extrapolated to 32 layers",
        }  # fmt: skip
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# c4: QAT encoder
# ------------------------------------------------------------------------------------------------
class BertQAT(torch.nn.Module):
    """BERT-base-shaped encoder (12 layers, hidden 768, 12 heads, FFN 3072) whose 72 Linears are this package's QLinear with
    PACT+ activations (clip values +-6) and SAWB+ per-channel weights.  Embeddings, LayerNorm, GELU and attention are PyTorch."""

    def __init__(self, dev, layers=12, hidden=768, heads=12, ffn=3072, vocab=30522, seq=128, dtype=torch.float32):
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
    """QAT forward + backward of the BERT-base-shaped encoder on a 32 x 128 batch of random token ids (seed 3), random-init
    weights, fp32.  One step = forward, the scalar loss (out * G).sum() with a seeded G, backward (no optimizer step: the
    workload is stated as forward + backward)."""
    from fms_model_optimizer_b200 import ops

    torch.manual_seed(3)
    dtype = torch.bfloat16 if args.c4_dtype == "bf16" else torch.float32
    model = BertQAT(dev, layers=args.layers or 12, dtype=dtype)
    model.train()
    B, S = 32, 128
    ids = torch.randint(0, 30522, (B, S), device=dev)
    G = torch.randn(B, S, 768, device=dev).to(dtype)
    params = [p for p in model.parameters() if p.requires_grad]

    def step():
        for p in params:
            p.grad = None
        loss = (model(ids) * G).sum()
        loss.backward()
        return loss

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ops.check_status(dev)
    sampler = ClockSampler(dev.index).start()
    ops.PROFILE, ops.LAUNCHES = None, 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    launches = ops.LAUNCHES
    ops.PROFILE = []
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    prof, ops.PROFILE = ops.PROFILE, None
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
        "vs_baseline": None, "dtype": args.c4_dtype, "data": "synthetic",
        "config": {"workload": "c4: BERT-base-shaped encoder, 72 QLinear (PACT+ 8-bit activations, SAWB+ per-channel 8-bit weights), "
                               "QAT forward + backward, batch 32 x 128, loss (out * G).sum()", "layers": len(model.blocks),
                   "l2": "activations 6-25 MB per tensor: L2 resident between kernels, as in the real step",
                   "library_kernels_ms_per_step": mine_ms,
                   "launches_per_step": {k: v[0] / args.steps for k, v in by.items()}},
        "roofline": {"bound": "hbm", "kernel": "pact2_fwd / pact2_bwd", "achieved": pact_gbs, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": (pact_gbs / pk["hbm"]) if pact_gbs else None, "traffic": None,
                     "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({pk['src']}); tensors of this workload fit in L2, so the "
                                    "fraction can exceed what HBM alone would allow"},
        "gpu_launches": launches, "clocks": clocks,
    }), flush=True)  # fmt: skip


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c5", "c1", "c2", "c3", "c4", "c5lin", "kernels"])
    ap.add_argument("--only", default="", help="--workload kernels: run only the cases whose name contains this text")
    ap.add_argument("--layers", type=int, default=None, help="development only: fewer layers")
    ap.add_argument("--surface", default="both", choices=["fused", "modules", "both"],
                    help="c5 on one GPU: the fused decoder (headline), the QLinearINT8Deploy module route, or the first timed and "
                         "the second reported beside it")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="c5 on one GPU: skip the single-kernel block")
    ap.add_argument("--no-check", action="store_true", help="sharded runs: skip the 2-layer comparison with the one-GPU forward")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the forward pass as one CUDA graph in the timed region (auto: sharded runs only)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "multimem", "stores", "allreduce"],
                    help="sharded runs: how the shard boundary is crossed (auto: multimem where the node has NVLink multicast, else stores)")
    ap.add_argument("--groups", type=int, default=0, help="groups of sequences pipelined on separate streams (0: 2 on sharded runs, else 1)")
    ap.add_argument("--reserve-sms", type=int, default=-1, help="sharded runs with several groups: SMs left to the link-bound exchange "
                    "kernels, GEMMs capped at the rest (-1: 16 on more than two GPUs, else 0)")
    ap.add_argument("--sweep", default="", help="sharded runs, development: further settings timed on the same weights after the headline, "
                    "comma-separated g<groups>r<reserved SMs>[s], e.g. g2r0,g2r32,g1r0,g2r16s")
    ap.add_argument("--nccl-ctas", type=int, default=16, help="upper bound on the CTAs of a collective (sharded runs)")
    ap.add_argument("--c4-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--act-scales", default="calibrated", choices=["calibrated", "synthetic"],
                    help="c5: SmoothQuant activation scales from a calibration forward of the float model, or synthetic ones")
    ap.add_argument("--breakdown", action="store_true", help="development: per-kernel-shape times on stderr")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.reserve_sms < 0:
        args.reserve_sms = 16 if world > 2 else 0

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
    failed = None
    try:
        if args.workload == "c4":
            run_c4(args, dev)
        elif args.workload == "c5":
            run_c5(args, rank, world, dev)
        else:
            run_kernel_workload(args, dev)
    except BaseException as e:  # noqa: BLE001
        failed = e
        import traceback

        traceback.print_exc()
    finally:
        if world > 1:
            # leave together: no rank may exit while another still sends traffic to memory it had bound to the multicast object
            try:
                torch.cuda.synchronize()
                dist.barrier()
            except Exception:  # noqa: BLE001
                pass
            dist.destroy_process_group()
    if failed is not None:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
