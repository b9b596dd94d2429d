"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the header declares,
and rejects bad arguments with status codes (no kernel is launched here)."""

import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from fms_model_optimizer_b200 import _lib as L

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "qlin_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qlin_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_symbols()
    assert set(names) == set(L.EXPORTED_SYMBOLS)
    for n in names:
        assert hasattr(lib, n), n
    assert lib.qlin_version() == 100


def test_struct_layouts_match_header_field_order():
    text = HEADER.read_text()
    for struct, cls in (("qlin_gemm_args", L.GemmArgs), ("qlin_quant_args", L.QuantArgs),
                        ("qlin_pact2_args", L.Pact2Args), ("qlin_wfq_args", L.WfqArgs),
                        ("qlin_tensor_fq_args", L.TensorFqArgs), ("qlin_block_quant_args", L.BlockQuantArgs),
                        ("qlin_rope_args", L.RopeArgs), ("qlin_peer_barrier_args", L.PeerBarrierArgs),
                        ("qlin_col_absmax_args", L.ColAbsmaxArgs), ("qlin_shard_reduce_args", L.ShardReduceArgs)):
        body = re.search(r"typedef struct " + struct + r" \{(.*?)\} " + struct, text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.replace("*", " ").split()
            # "const void* a" / "int64_t lda, ldb" / "float scale0, zp0"
            head, _, rest = decl.partition(",")
            first = head.replace("*", " ").split()[-1]
            fields.append(first)
            fields += [r.strip().lstrip("*") for r in rest.split(",") if r.strip()]
        fields = [re.sub(r"\[\d+\]$", "", f) for f in fields]  # arrays: "ldq[3]" is the ctypes field "ldq"
        assert fields == [f[0] for f in cls._fields_], struct


def test_null_and_bad_arguments_are_status_codes():
    lib = L.load()
    assert lib.qlin_gemm(None, None) == L.ERR_NULL
    a = L.GemmArgs()
    assert lib.qlin_gemm(C.byref(a), None) == L.ERR_NULL
    assert b"NULL" in lib.qlin_last_error_string()
    buf = (C.c_char * 4096)()
    base = C.addressof(buf)
    base = (base + 15) // 16 * 16
    a = L.GemmArgs(a=base, b=base, d=base, M=16, N=16, K=32, lda=32, ldb=32, ldd=16, kind=L.DT_F32)
    assert lib.qlin_gemm(C.byref(a), None) == L.ERR_BAD_DTYPE
    a.kind = L.DT_I8
    a.M = -1
    assert lib.qlin_gemm(C.byref(a), None) == L.ERR_BAD_SHAPE
    a.M = 16
    a.lda = 24  # not a multiple of 16 bytes, and smaller than K
    assert lib.qlin_gemm(C.byref(a), None) in (L.ERR_BAD_SHAPE, L.ERR_BAD_ALIGN)
    a.lda = 48
    a.a = base + 1
    a.out_dtype = L.DT_I32
    assert lib.qlin_gemm(C.byref(a), None) == L.ERR_BAD_ALIGN
    a.a = base
    a.chunk_k = 48
    assert lib.qlin_gemm(C.byref(a), None) == L.ERR_UNSUPPORTED
    a.chunk_k = 64
    a.out_dtype = L.DT_F16  # raw int8 output must be int32
    assert lib.qlin_gemm(C.byref(a), None) == L.ERR_BAD_DTYPE
    q = L.QuantArgs()
    assert lib.qlin_act_quant(C.byref(q), None) == L.ERR_NULL
    q = L.QuantArgs(x=base, codes=base, rows=4, cols=16, ldx=16, ldq=16, x_dtype=L.DT_I8, qmax_levels=127)
    assert lib.qlin_act_quant(C.byref(q), None) == L.ERR_BAD_DTYPE
    p = L.Pact2Args(x=base, out=base, clip_val=base, clip_valn=base, numel=4, dtype=L.DT_F32, num_bits=1)
    assert lib.qlin_pact2_fwd(C.byref(p), None) == L.ERR_UNSUPPORTED
    w = L.WfqArgs(w=base, dq_out=base, clip_io=base, rows=2, cols=16, ldw=16, ldo=16, dtype=L.DT_F32, num_bits=3)
    assert lib.qlin_weight_fq_perch(C.byref(w), None) == L.ERR_UNSUPPORTED
    assert lib.qlin_pact2_bwd_workspace_bytes(1 << 20) > 0


def test_no_cpu_fallback():
    from fms_model_optimizer_b200 import ops

    a = torch.zeros(16, 32, dtype=torch.int8)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.gemm(a, a)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.act_quant(torch.zeros(4, 16))


def test_product_never_imports_the_oracle():
    pkg = ROOT / "fms_model_optimizer_b200"
    for f in pkg.rglob("*.py"):
        src = f.read_text()
        assert "import oracle" not in src and "from oracle" not in src, f


def test_struct_sizes_and_offsets_match_a_c_compiler(tmp_path):
    """The header compiled as plain C: sizeof and the offset of every field of every argument block equal the ctypes
    mirror's (field order alone would not catch a wrong type)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    assert gcc, "gcc is part of this build's toolchain"
    structs = (("qlin_gemm_args", L.GemmArgs), ("qlin_quant_args", L.QuantArgs), ("qlin_pact2_args", L.Pact2Args),
               ("qlin_wfq_args", L.WfqArgs), ("qlin_tensor_fq_args", L.TensorFqArgs), ("qlin_block_quant_args", L.BlockQuantArgs),
               ("qlin_rope_args", L.RopeArgs), ("qlin_peer_barrier_args", L.PeerBarrierArgs),
               ("qlin_col_absmax_args", L.ColAbsmaxArgs), ("qlin_shard_reduce_args", L.ShardReduceArgs))  # fmt: skip
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for name, cls in structs:
        lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in cls._fields_:
            lines.append(f'  printf("{name}.{field} %zu\\n", offsetof({name}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-o", str(exe), str(src)], check=True)
    got = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for name, cls in structs:
        assert int(got[name]) == C.sizeof(cls), name
        for field, _ in cls._fields_:
            assert int(got[f"{name}.{field}"]) == getattr(cls, field).offset, f"{name}.{field}"
