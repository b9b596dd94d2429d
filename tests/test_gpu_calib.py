"""Calibration statistics on the GPU against the reference's formula (activation_stats, fms_mo/quant/ptq.py:2586-2596):
``tensor.view(-1, hidden).abs().max(dim=0)`` maximised over batches.  A maximum has no rounding, so parity is exact."""

import pytest
import torch

from fms_model_optimizer_b200 import calib, ops

pytestmark = pytest.mark.gpu


def _ref_stats(batches):
    """activation_stats as the reference writes it, on CPU."""
    acc = None
    for t in batches:
        coming = torch.max(t.view(-1, t.shape[-1]).abs().detach(), dim=0)[0].float().cpu()
        acc = coming if acc is None else torch.max(acc, coming)
    return acc


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 16), (3, 7, 100), (5000, 4096), (2, 129, 1000), (40, 14336)])
def test_col_absmax_equals_reference_formula(cuda_dev, dtype, shape):
    g = torch.Generator().manual_seed(sum(shape))
    batches = [(torch.randn(shape, generator=g) * (1 + i)).to(dtype) for i in range(3)]
    want = _ref_stats(batches)
    running = None
    for t in batches:
        running = ops.col_absmax(t.to(cuda_dev), running=running) if running is not None else ops.col_absmax(t.to(cuda_dev))
    assert torch.equal(running.cpu(), want)
    # a strided view (rows with a pitch) and an offset that breaks the 16-byte alignment
    wide = torch.randn(shape[-2] if len(shape) > 1 else 1, shape[-1] + 9, generator=g).to(dtype).to(cuda_dev)
    view = wide[:, 1 : 1 + shape[-1]]
    assert torch.equal(ops.col_absmax(view).cpu(), view.cpu().abs().float().amax(0))


def test_col_absmax_propagates_nan_and_handles_empty(cuda_dev):
    x = torch.randn(64, 48, device=cuda_dev)
    x[7, 5] = float("nan")
    got = ops.col_absmax(x).cpu()
    want = torch.max(x.cpu().abs(), dim=0)[0]
    assert torch.isnan(got[5]) and torch.equal(got.nan_to_num(-1.0), want.nan_to_num(-1.0))
    assert ops.col_absmax(torch.zeros(0, 32, device=cuda_dev)).cpu().tolist() == [0.0] * 32


def test_get_act_scales_hooks_every_linear(cuda_dev):
    """The collector against the reference's collector logic on a toy model: two Linears, two batches."""
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.GELU(), torch.nn.Linear(96, 32)).to(cuda_dev).bfloat16()
    batches = [torch.randn(4, 10, 64).bfloat16() * (i + 1) for i in range(2)]
    got = calib.get_act_scales(model, batches, device=cuda_dev, to_cpu=True)
    assert set(got) == {"0", "2"}
    ins = {"0": [], "2": []}
    hooks = [model[i].register_forward_hook(lambda m, x, y, k=str(i): ins[k].append(x[0].detach().cpu())) for i in (0, 2)]
    with torch.no_grad():
        for b in batches:
            model(b.to(cuda_dev))
    for h in hooks:
        h.remove()
    for k in ins:
        assert torch.equal(got[k], _ref_stats(ins[k])), k
