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


def _worker_token_split(rank, world, port, q):
    """The exchange scheme of the sharded prefill with the residual stream split by tokens, emulated with gloo
    collectives standing in for the kernels' peer stores: partial outputs of a row-parallel Linear go to the owner
    of each token block, the owner sums them in fp32 in rank order, adds them to its slice of the stream, normalises,
    quantises for the next column-parallel Linear and hands its codes and scales to every rank."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torch.nn.functional as F

        from fms_model_optimizer_b200 import tp

        torch.manual_seed(1)
        T, K, H, N = 16, 64, 32, 48  # tokens, row-parallel in-features, hidden, column-parallel out-features
        Ts = T // world
        stream = torch.randn(T, H).bfloat16()
        a = torch.randn(T, K).bfloat16()
        w_o = torch.randint(-127, 128, (H, K), dtype=torch.int8)
        w_c = torch.randint(-127, 128, (N, H), dtype=torch.int8)
        s_o, s_c = torch.rand(H) * 1e-3 + 1e-4, torch.rand(N) * 1e-3 + 1e-4
        sm_o, sm_c = (torch.rand(K) * 2 + 0.5).bfloat16().float(), (torch.rand(H) * 2 + 0.5).bfloat16().float()
        norm_w = torch.ones(H).bfloat16()
        kw = dict(quant_fn=_oracle_quant, gemm_fn=_oracle_gemm)
        row = tp.W8A8Linear(*tp.shard_w8a8(w_o, s_o, sm_o, None, "row", world, rank), mode="row", **kw)
        col = tp.W8A8Linear(*tp.shard_w8a8(w_c, s_c, sm_c, None, "column", world, rank), mode="column", **kw)
        ks = tp.shard_range(K, world, rank)
        # every shard's partial output for all tokens (scales max-reduced across the shards, no sum)
        partial = row(a[:, ks].contiguous(), reduce=False)
        # "peer stores": token block i of every shard's partial goes to rank i (gloo has no all-to-all: gather, then pick)
        parts = [torch.empty_like(partial) for _ in range(world)]
        dist.all_gather(parts, partial)
        recv = [p_[rank * Ts : (rank + 1) * Ts] for p_ in parts]
        acc = recv[0].float()
        for r in range(1, world):
            acc = acc + recv[r].float()
        mine = slice(rank * Ts, (rank + 1) * Ts)
        x_new = stream[mine] + acc.bfloat16()
        h = F.rms_norm(x_new.float(), (H,), norm_w.float(), 1e-5).bfloat16()
        codes, scale = col.quantise(h)
        all_codes = [torch.empty_like(codes) for _ in range(world)]
        all_scale = [torch.empty_like(scale) for _ in range(world)]
        dist.all_gather(all_codes, codes)
        dist.all_gather(all_scale, scale)
        got = col(None, (torch.cat(all_codes), torch.cat(all_scale)), torch.bfloat16)
        # the same block on whole tensors
        acc_full = parts[0].float()
        for r in range(1, world):
            acc_full = acc_full + parts[r].float()
        h_full = F.rms_norm((stream + acc_full.bfloat16()).float(), (H,), norm_w.float(), 1e-5).bfloat16()
        want = col(h_full)
        # and the all-reduce scheme agrees to the rounding of the partial sums
        y = row(a[:, ks].contiguous())
        h_ar = F.rms_norm((stream + y).float(), (H,), norm_w.float(), 1e-5).bfloat16()
        close = (h_ar.float() - h_full.float()).abs().max().item() <= 4 * 2.0**-8 * h_full.float().abs().max().item()
        q.put((rank, torch.equal(got, want), close))
    finally:
        dist.destroy_process_group()


def test_token_split_exchange_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_token_split, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, exact, close in results:
        assert exact, f"rank {rank}: token-split exchange differs from the whole-tensor computation"
        assert close, f"rank {rank}: token-split and all-reduce schemes disagree beyond the rounding of the partial sums"
