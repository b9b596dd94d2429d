"""Builds libqlin_b200.so (the C-ABI library with every CUDA kernel of this package) in-tree.

The library is compiled for sm_100a only with plain ``nvcc``; nothing is JIT-compiled at run time.
``python -m fms_model_optimizer_b200.build_ext`` rebuilds it; ``build()`` is also what
``__graft_entry__.build()`` calls.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libqlin_b200.so"
OBJ_DIR = LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libqlin_b200.so cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


STAMP_PATH = LIB_DIR / "libqlin_b200.stamp"


def source_digest(extra_flags: tuple = ()) -> str:
    """SHA-256 over the compiler flags and the name and content of every file the library is built from.  File times
    say nothing after a checkout or a copy to another machine, so staleness is decided by content."""
    files = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    files.append(PKG_DIR.parent / "include" / "qlin_b200.h")
    h = hashlib.sha256()
    h.update("\0".join([*NVCC_FLAGS, *extra_flags]).encode())
    for f in files:
        h.update(f.name.encode() + b"\0")
        h.update(f.read_bytes())
    return h.hexdigest()


def is_stale() -> bool:
    """True unless the library exists and the digest stored beside it at build time equals the digest of the sources."""
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != source_digest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link ``lib/libqlin_b200.so``.  Returns the library path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=4) as pool:
        objs = list(pool.map(compile_one, _sources()))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
