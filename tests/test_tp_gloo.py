"""Tensor-parallel sharding of the W8A8 Linear on CPU ranks (gloo, world size 2).

The collectives and the shard arithmetic of ``fms_model_optimizer_b200.tp`` are exercised with the
oracle's CPU arithmetic standing in for the CUDA kernels (the product itself has no CPU path):
a column-parallel layer must reproduce the unsharded layer exactly on its slice of the outputs; a
row-parallel layer must produce the unsharded int8 codes (the scales are max-reduced across ranks)
and an output within fp16 rounding of the partial sums."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_quant(x2, smooth, given_scale):
    from oracle import quantizers as OQ

    xs = x2 if smooth is None else x2 / smooth.to(x2.dtype)
    if given_scale is None:
        codes, scale = OQ.qa_dynamic_max_qfunc(xs)
        return codes, scale.float().reshape(-1)
    s = given_scale.to(x2.dtype).reshape(-1, 1)
    return torch.round(xs / s).to(torch.int8), given_scale


def _oracle_gemm(codes, weight, scale, w_scale, bias, out_dtype, prod_dtype):
    from oracle import gemm as OG

    acc = OG.imatmul_chunk_truncate(codes, weight.t().contiguous(), chunk_size=32)
    s = (scale.reshape(-1, 1).to(prod_dtype) * w_scale.to(prod_dtype)).to(torch.float16)
    out = acc.float() * s
    if bias is not None:
        out = out + bias
    return out.to(torch.float16).to(out_dtype)


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fms_model_optimizer_b200 import tp

        torch.manual_seed(0)
        M, K, N = 24, 128, 64
        x = torch.randn(M, K).bfloat16()
        w = torch.randint(-127, 128, (N, K), dtype=torch.int8)
        w_scale = torch.rand(N) * 1e-3 + 1e-4
        smooth = (torch.rand(K) * 2 + 0.5).bfloat16().float()
        bias = torch.randn(N) * 0.01
        full = tp.W8A8Linear(w, w_scale, smooth, bias, mode="replicate", quant_fn=_oracle_quant, gemm_fn=_oracle_gemm)
        want = full(x)
        want_codes, want_scale = full.quantise(x)
        # column parallel: exact on the rank's output slice
        wt, sc, sm, bs = tp.shard_w8a8(w, w_scale, smooth, bias, "column", world, rank)
        col = tp.W8A8Linear(wt, sc, sm, bs, mode="column", quant_fn=_oracle_quant, gemm_fn=_oracle_gemm)
        got = col(x)
        sl = tp.shard_range(N, world, rank)
        ok_col = torch.equal(got, want[:, sl])
        # row parallel: x is split along K like the output of a column-parallel predecessor
        wt, sc, sm, bs = tp.shard_w8a8(w, w_scale, smooth, bias, "row", world, rank)
        row = tp.W8A8Linear(wt, sc, sm, bs, mode="row", quant_fn=_oracle_quant, gemm_fn=_oracle_gemm)
        ks = tp.shard_range(K, world, rank)
        codes, scale = row.quantise(x[:, ks].contiguous())
        ok_codes = torch.equal(codes, want_codes[:, ks]) and torch.equal(scale, want_scale)
        got = row(x[:, ks].contiguous())
        err = (got.float() - want.float()).abs().max().item()
        tol = 4 * 2.0**-8 * want.float().abs().max().item()
        bias_ok = (bs is None) == (rank != 0)
        q.put((rank, ok_col, ok_codes, err <= tol, bias_ok, err, tol))
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_col, ok_codes, ok_out, bias_ok, err, tol in results:
        assert ok_col, f"rank {rank}: column-parallel slice differs"
        assert ok_codes, f"rank {rank}: row-parallel codes / scales differ from the unsharded layer"
        assert ok_out, f"rank {rank}: row-parallel output error {err} > {tol}"
        assert bias_ok


def test_shard_range_rejects_uneven_splits():
    from fms_model_optimizer_b200 import tp

    assert tp.shard_range(32, 4, 3) == slice(24, 32)
    with pytest.raises(ValueError):
        tp.shard_range(10, 4, 0)
