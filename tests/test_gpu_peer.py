"""Two processes on two GPUs: arena exchange over CUDA IPC, the flag barrier, a GEMM whose epilogue stores half of
its rows into the other GPU's buffer, and the fused quantiser writing its codes to both GPUs."""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, fail_q):
    try:
        sys.path.insert(0, ROOT)
        import torch.distributed as dist

        from fms_model_optimizer_b200 import _lib as L
        from fms_model_optimizer_b200 import ops
        from fms_model_optimizer_b200.peer import PeerArena, PeerBarrier

        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        M, K, N = 256 * world, 256, 256
        rows = M // world
        arena = PeerArena(world * rows * N * 2 + 2 * (M * K + 4 * M) + 4096, dev)
        bar = PeerBarrier(arena)
        part_off, part = arena.alloc(world * rows * N * 2)
        codes_off, codes = arena.alloc(M * K)
        scale_off, scales = arena.alloc(4 * M)
        g = torch.Generator().manual_seed(100)  # same operands on every rank, shard the K dimension
        a = torch.randint(-127, 128, (M, K * world), generator=g, dtype=torch.int8)
        b = torch.randint(-127, 128, (N, K * world), generator=g, dtype=torch.int8)
        a_r, b_r = a[:, rank * K : (rank + 1) * K].contiguous().to(dev), b[:, rank * K : (rank + 1) * K].contiguous().to(dev)
        rs = torch.full((M,), 2.0**-12, device=dev)
        for it in range(3):
            # reduce-scatter by remote stores: my partial rows of block o go to rank o, slot `rank`
            ops.gemm(a_r, b_r, epilogue=L.EPI_SCALE_PROD, row_scale=rs, out_dtype=torch.bfloat16,
                     scatter=([arena.addr(o, part_off) for o in range(world)], rows, rank * rows))
            bar.wait()
            mine = part.view(torch.bfloat16).view(world, rows, N)
            full = (a.double() @ b.double().t())
            want_parts = [((a[:, s * K : (s + 1) * K].double() @ b[:, s * K : (s + 1) * K].double().t()) * 2.0**-12).float().bfloat16()
                          for s in range(world)]
            for s in range(world):
                assert torch.equal(mine[s].cpu(), want_parts[s][rank * rows : (rank + 1) * rows]), (it, rank, s)
            # sum the parts, quantise, write the codes of my rows to every rank
            x = torch.zeros(rows, N, dtype=torch.bfloat16, device=dev)
            ops.block_quant(x, prologue=L.BLOCK_NORM, r=mine[0], r_parts=world, r_part_stride=rows * N,
                            norm_w=torch.ones(N, dtype=torch.bfloat16, device=dev), smooth_rcps=[None], sum_into=x,
                            dst=([arena.addr(o, 0) for o in range(world)], [codes_off], [scale_off], rank * rows))
            bar.wait()
            allc = codes[: M * N].view(torch.int8).view(M, N).cpu()
            ops.check_status(dev)
            acc = want_parts[0].float()
            for s in range(1, world):
                acc = acc + want_parts[s].float()
            xs = acc.bfloat16()
            h = torch.nn.functional.rms_norm(xs.float(), (N,), None, 1e-5).bfloat16()
            want_c = torch.round(h / (h.abs().amax(-1, keepdim=True).clamp(min=1e-5) / 127)).to(torch.int8)
            # the normalised row may differ from PyTorch's in the last place; compare where it agrees exactly
            agree = (allc == want_c).float().mean().item()
            assert agree > 0.98, (it, rank, agree)
            del full
            bar.wait()  # nobody overwrites the buffers before everyone has checked them
        arena.close()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        import traceback

        fail_q.put((rank, "".join(traceback.format_exception(e))))
        raise


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_remote_scatter_and_replicated_codes_two_gpus():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, port = 2, 29631
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    errs = []
    while not q.empty():
        errs.append(q.get())
    assert not errs, errs
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
