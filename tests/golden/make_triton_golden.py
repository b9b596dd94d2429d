"""Runs fms-model-optimizer's own Triton kernels on a CUDA device and stores their outputs as golden vectors.

    python tests/golden/make_triton_golden.py OUT.pt [path/to/an/installed/fms_mo/parent]

The reference's chunk-truncating matmuls (tl_matmul_chunk_truncate -> imatmul_kernel / matmul_kernel,
fms_mo/custom_ext_kernels/triton_kernels.py:468, :211, :96) need a GPU, so this script cannot run where the other
fixtures are made.  It imports the reference from the given directory (default: baseline/_ref under the repository
root, where the reference was pip-installed; that directory is not part of this repository), drives the kernels on
seeded inputs and saves inputs' seeds, shapes and outputs.  The saved file is what pins the float chunk GEMM of the
oracle and of the CUDA kernels to the reference itself (tests/test_oracle_golden.py, tests/test_gpu_gemm.py).  It also
times the reference kernels on the benchmark's large int8 shape, as the same-box comparator.
"""

from __future__ import annotations

import json
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent


def main():
    out_path = Path(sys.argv[1])
    ref_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else ROOT / "baseline" / "_ref"
    sys.path.insert(0, str(ref_dir))
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from fms_mo.custom_ext_kernels.triton_kernels import tl_matmul_chunk_truncate as ref_mm

    dev = torch.device("cuda", 0)
    out = {"cases": [], "timing": [], "errors": []}

    def guarded(fn):
        """A reference kernel that does not build with the installed Triton is recorded, not fatal: the other kernels
        still give their vectors."""
        def run(*args, **kw):
            try:
                return fn(*args, **kw)
            except Exception as e:  # noqa: BLE001
                msg = f"{type(e).__name__}: {str(e).strip().splitlines()[0] if str(e).strip() else ''}"
                out["errors"].append(dict(what=f"{fn.__name__}{args}{kw}", error=msg[:400]))
                print("FAILED", fn.__name__, args, kw, msg[:200], flush=True)
        return run

    @guarded
    def case(kind, M, K, N, seed, **kw):
        g = torch.Generator().manual_seed(seed)
        if kind == "int8":
            a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
            b_nk = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
        else:
            a = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
            b_nk = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
        c = None
        if kw.pop("with_c", False):
            c = torch.randint(-1000, 1000, (M, N), generator=g).to(torch.int32 if kind == "int8" else torch.float32)
        y = ref_mm(a.to(dev), b_nk.to(dev).t(), c=(c.to(dev) if c is not None else None), **kw)
        torch.cuda.synchronize()
        out["cases"].append(dict(kind=kind, M=M, K=K, N=N, seed=seed, kw=dict(kw), with_c=c is not None, y=y.cpu()))
        print("case", kind, M, K, N, kw, tuple(y.shape), y.dtype, flush=True)

    # int8: plain, truncated, clamped accumulator, truncate-after-accumulate, initial accumulator, ragged sizes
    case("int8", 1024, 1024, 1024, 1, chunk_trun_bits=8, chunk_size=64)
    case("int8", 200, 320, 136, 2, chunk_trun_bits=4, chunk_size=32)
    case("int8", 96, 512, 80, 3, chunk_trun_bits=8, chunk_size=64, max_acc_bits=20)
    case("int8", 96, 512, 80, 4, chunk_trun_bits=8, chunk_size=64, truncate_then_accumulate=False)
    case("int8", 96, 512, 80, 5, chunk_trun_bits=8, chunk_size=128, with_c=True)
    case("int8", 64, 256, 64, 6, chunk_trun_bits=0, chunk_size=64)
    # fp8 e4m3: plain, mantissa truncation, DL16 clamp, truncate-after-accumulate, initial accumulator
    case("fp8", 1024, 1024, 1024, 11, chunk_trun_bits=0, chunk_size=64)
    case("fp8", 1024, 1024, 1024, 12, chunk_trun_bits=8, chunk_size=64)
    case("fp8", 200, 320, 136, 13, chunk_trun_bits=16, chunk_size=32)
    case("fp8", 96, 512, 80, 14, chunk_trun_bits=0, chunk_size=64, clamp_acc_to_dl16=True)
    case("fp8", 96, 512, 80, 15, chunk_trun_bits=12, chunk_size=64, truncate_then_accumulate=False)
    case("fp8", 96, 512, 80, 16, chunk_trun_bits=8, chunk_size=128, with_c=True)

    @guarded
    def timing(kind, M, K, N, **kw):
        if kind == "int8":
            a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
            b = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        else:
            a = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
            b = torch.randn(N, K, device=dev).to(torch.float8_e4m3fn)
        for _ in range(3):
            ref_mm(a, b.t(), **kw)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        n = 5
        for _ in range(n):
            ref_mm(a, b.t(), **kw)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        rec = dict(kind=kind, M=M, K=K, N=N, kw=kw, ms=ms, tops=2.0 * M * N * K / (ms * 1e-3) / 1e12)
        out["timing"].append(rec)
        print("timing", json.dumps(rec), flush=True)

    # the reference kernels as same-box comparator: time after warm-up with CUDA events
    timing("int8", 16384, 4096, 4096, chunk_trun_bits=0, chunk_size=64)
    timing("int8", 4096, 8192, 4096, chunk_trun_bits=8, chunk_size=64)
    timing("fp8", 8192, 4096, 14336, chunk_trun_bits=0, chunk_size=64)
    timing("fp8", 4096, 8192, 4096, chunk_trun_bits=8, chunk_size=64)
    out["versions"] = dict(torch=torch.__version__, triton=__import__("triton").__version__, device=torch.cuda.get_device_name(0),
                           when=time.strftime("%Y-%m-%d"))
    torch.save(out, out_path)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
