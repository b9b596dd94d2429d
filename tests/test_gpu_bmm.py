"""GPU parity of the quantized batched matmul (QBmm, QBmmINT8Deploy, ops.bmm_i8) against outputs of the reference itself
(tests/golden/bmm.pt) and against exact integer arithmetic."""

import pytest
import torch

from conftest import load_golden
from fms_model_optimizer_b200 import ops
from fms_model_optimizer_b200.modules import QBmm, QBmmINT8Deploy
from oracle import bmm as OB

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,M,N,K", [(3, 1, 40, 96), (2, 100, 70, 33), (5, 128, 256, 128), (4, 300, 130, 64), (6, 512, 512, 128), (2, 2048, 128, 2048)])
def test_bmm_i8_is_exact(cuda_dev, B, M, N, K):
    g = torch.Generator().manual_seed(B * 1000 + M)
    a = torch.randint(-128, 128, (B, M, K), dtype=torch.int8, generator=g)
    b = torch.randint(-128, 128, (B, N, K), dtype=torch.int8, generator=g)
    want = torch.matmul(a.double(), b.double().transpose(1, 2)).to(torch.int32)
    got = ops.bmm_i8(a.to(cuda_dev), b.to(cuda_dev))
    ops.check_status(cuda_dev)
    assert got.dtype == torch.int32 and torch.equal(got.cpu(), want)


def _build(c, dev):
    q = QBmm(qcfg=dict(c["qcfg"]), **c["kw"]).to(c["dtype"]).to(dev)
    return q


def test_qbmm_fake_quant_matches_reference(cuda_dev):
    """Operands quantised by the CUDA kernels equal the reference's quantised operands bit for bit (checked through the
    oracle, itself pinned to the fixture); the product is a library matmul as in the reference, compared within the
    summation-order tolerance of its dtype; gradients of both operands and of the clip values follow the fixture."""
    for c in load_golden("bmm.pt")["cases"]:
        kw, (nb1, nb2), dt = c["kw"], c["num_bits"], c["dtype"]
        q = _build(c, cuda_dev)
        assert (q.num_bits_m1, q.num_bits_m2) == (nb1, nb2)
        m1 = c["m1"].to(cuda_dev).requires_grad_(True)
        m2 = c["m2"].to(cuda_dev).requires_grad_(True)
        cv1 = torch.tensor([kw["m1_clip_init_val"]]).to(dt)
        cvn1 = torch.tensor([kw["m1_clip_init_valn"]]).to(dt)
        cv2 = torch.tensor([kw["m2_clip_init_val"]]).to(dt)
        want1 = OB.fake_quant_operand(c["m1"], kw["qm1_mode"], nb1, cv1, cvn1, kw["m1_unidirectional"])
        want2 = OB.fake_quant_operand(c["m2"], kw["qm2_mode"], nb2, cv2, None, False)
        assert torch.equal(q.quantize_m1(m1).detach().cpu(), want1), c["name"]
        assert torch.equal(q.quantize_m2(m2).detach().cpu(), want2), c["name"]
        y = q(m1, m2)
        tol = 2e-5 if dt == torch.float32 else 2.0**-7
        assert y.dtype == dt and y.shape == c["y"].shape
        err = (y.detach().cpu().float() - c["y"].float()).abs().max().item()
        assert err <= tol * c["y"].float().abs().max().item(), (c["name"], err)
        y.backward(c["grad_out"].to(cuda_dev))
        for got, want in ((m1.grad, c["grad_m1"]), (m2.grad, c["grad_m2"])):
            e = (got.cpu().float() - want.float()).norm() / want.float().norm()
            assert e < (1e-5 if dt == torch.float32 else 2e-2), (c["name"], e.item())
        if dt == torch.float32:
            for n, p in q.named_parameters():
                want = c["clip_grads"][n].float()
                assert torch.allclose(p.grad.cpu().float(), want, rtol=1e-3, atol=1e-3 * want.abs().max().item() + 1e-6), (c["name"], n)
        assert int(q.num_module_called) == 1


def test_qbmm_int8_deploy_matches_reference(cuda_dev):
    """Buffers and outputs of QBmmINT8Deploy equal the reference's own bit for bit -- including the infinities its fp16
    stage produces for large sums and the correction term as the reference evaluates it -- with the product of the codes
    computed by the integer tcgen05 GEMM."""
    for c in load_golden("bmm.pt")["cases"]:
        # converted from a module on the CPU (as the fixture was), the buffers are the reference's bit for bit; converted
        # on the GPU, PyTorch divides by a constant through its reciprocal there and a scale may differ in its last place
        q_cpu = QBmm(qcfg=dict(c["qcfg"]), **c["kw"]).to(c["dtype"])
        d = QBmmINT8Deploy.from_fms_mo(q_cpu, target_device=cuda_dev)
        for k, v in c["deploy_buffers"].items():
            got = getattr(d, k)
            assert got.dtype == v.dtype and got.device.type == "cuda" and torch.equal(got.cpu(), v), (c["name"], k)
        d_gpu = QBmmINT8Deploy.from_fms_mo(_build(c, cuda_dev))
        for k, v in c["deploy_buffers"].items():
            got = getattr(d_gpu, k).cpu()
            assert got.dtype == v.dtype and torch.allclose(got.float(), v.float(), rtol=2.0**-7 if v.dtype != torch.float32 else 2e-7, atol=0), (c["name"], k)
        y = d(c["m1"].to(cuda_dev), c["m2"].to(cuda_dev))
        ops.check_status(cuda_dev)
        want = c["y_deploy"]
        assert y.dtype == want.dtype
        a, b = torch.nan_to_num(y.cpu().float(), nan=12345.0), torch.nan_to_num(want.float(), nan=12345.0)
        assert torch.equal(a, b), (c["name"], (a - b).abs().max().item())


def test_qbmm_int8_deploy_attention_shapes(cuda_dev):
    """q @ k^T (m2 is the transposed view of k) and p @ v at attention sizes where the reference cannot run (its
    correction term does not broadcast): symmetric operands, against the oracle's exact integer restatement."""
    qcfg = {"use_PT_native_Qfunc": False, "sym_7bits_bmm": False}
    g = torch.Generator().manual_seed(9)
    B, H, S, D = 2, 4, 256, 64
    qh, kh, vh = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
    mod = QBmm(num_bits_m1=8, qm1_mode="pactsym+", num_bits_m2=8, qm2_mode="pactsym+", qcfg=qcfg, m1_clip_init_val=0.75, m2_clip_init_val=0.75)
    dep = QBmmINT8Deploy.from_fms_mo(mod, target_device=cuda_dev)  # clip value 0.75: round(0.75 / (1.5 / 255)) is 128 in fp32 (0.5 or 1.0 give 127)
    buf = {k: v.cpu() for k, v in dep.named_buffers()}
    assert int(buf["m1_zp"]) == 128
    for m1, m2 in ((qh * 0.1, (kh * 0.1).transpose(-1, -2)), (torch.softmax(qh @ kh.transpose(-1, -2), -1) - 0.004, vh * 0.1)):
        y = dep(m1.to(cuda_dev), m2.to(cuda_dev))
        m1_i8 = OB.qfunc_raw(m1, buf["m1_scale"], buf["m1_zp"] - 128)
        m2_i8 = OB.qfunc_raw(m2, buf["m2_scale"], buf["m2_zp"])
        want = (torch.matmul(m1_i8.double(), m2_i8.double()).to(torch.float16) * buf["m1_scale"] * buf["m2_scale"]).to(m1.dtype)
        assert torch.equal(torch.nan_to_num(y.cpu()), torch.nan_to_num(want))
        assert torch.isfinite(want).all()
