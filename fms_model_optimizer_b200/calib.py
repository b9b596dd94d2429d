"""SmoothQuant calibration on the GPU: the activation statistics the quantized Linears are built from.

Mirrors ``get_act_scales`` / ``activation_stats`` / ``input_stats_hook`` of the reference
(fms_mo/quant/ptq.py:2586-2657): forward hooks on every Linear record the per-input-channel absolute maximum of the
layer's input, maximised over the calibration batches.  The reference computes ``abs().max(dim=0)`` with ATen and
copies every batch's vector to the host; here one kernel (``qlin_col_absmax``) folds each batch into a running vector
that stays on the device, and nothing is synchronised until the caller reads the result.
"""

from __future__ import annotations

from functools import partial
from typing import Dict, Iterable, Optional

import torch
from torch import nn

from . import ops


@torch.no_grad()
def activation_stats(name: str, tensor: torch.Tensor, act_scales: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """fms_mo/quant/ptq.py:2586-2596 with the running maximum kept on the device (fp32 ``[hidden]``)."""
    if name in act_scales:
        ops.col_absmax(tensor.detach(), running=act_scales[name])
    else:
        act_scales[name] = ops.col_absmax(tensor.detach())
    return act_scales


@torch.no_grad()
def input_stats_hook(m, x, _y, name, act_scales):
    """fms_mo/quant/ptq.py:2599-2606 (the QBmm branch of the reference takes the second input; this package has no
    QBmm, so a tuple input means its first element)."""
    if isinstance(x, tuple):
        x = x[0]
    activation_stats(name, x, act_scales)


@torch.no_grad()
def get_act_scales(model: nn.Module, dloader: Iterable, qcfg: Optional[dict] = None, device=None, n_samples: int = 100,
                   to_cpu: bool = False) -> Dict[str, torch.Tensor]:
    """Per-channel activation maxima of every Linear-like module of ``model`` over up to ``n_samples`` batches of
    ``dloader`` (dicts are passed as keyword arguments, anything else positionally), as the reference's
    ``get_act_scales`` (fms_mo/quant/ptq.py:2609-2657).  Modules are matched by type (``nn.Linear`` and subclasses, which
    covers this package's ``QLinear``) or by the class name ``QLinear`` so that the reference's own modules qualify too.
    The vectors stay on the device unless ``to_cpu``."""
    model.eval()
    if device is not None:
        model.to(device)
    act_scales: Dict[str, torch.Tensor] = {}
    if qcfg is not None:
        qcfg["sample_id"] = 0
    hooks = []
    for name, m in model.named_modules():
        if isinstance(m, nn.Linear) or type(m).__name__ == "QLinear":
            hooks.append(m.register_forward_hook(partial(input_stats_hook, name=name, act_scales=act_scales)))
    try:
        for data_mb, _ in zip(dloader, range(n_samples)):
            if qcfg is not None:
                qcfg["sample_id"] += 1
            if isinstance(data_mb, dict):
                model(**{k: (v.to(device) if (device is not None and torch.is_tensor(v)) else v) for k, v in data_mb.items()})
            else:
                model(data_mb.to(device) if (device is not None and torch.is_tensor(data_mb)) else data_mb)
    finally:
        for h in hooks:
            h.remove()
    if to_cpu:
        return {k: v.cpu() for k, v in act_scales.items()}
    return act_scales
