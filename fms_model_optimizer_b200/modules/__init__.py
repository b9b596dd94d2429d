"""Quantized Linear and batched-matmul modules (mirror of fms_mo/modules/linear.py and fms_mo/modules/bmm.py for the B200 path)."""

from .bmm import QBmm, QBmmINT8Deploy
from .linear import (
    LinearFPxAcc,
    QLinear,
    QLinearCublasI8I32NT,
    QLinearCutlassI8I32NT,
    QLinearINT8Deploy,
    QLinearINT8Train,
    lower_qmodel_b200,
)

__all__ = ["QLinear", "QLinearINT8Deploy", "QLinearINT8Train", "QLinearCublasI8I32NT", "QLinearCutlassI8I32NT", "LinearFPxAcc", "lower_qmodel_b200",
           "QBmm", "QBmmINT8Deploy"]  # fmt: skip
