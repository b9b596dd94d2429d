"""Quantized Linear modules (mirror of fms_mo/modules/linear.py for the B200 path)."""

from .linear import (
    LinearFPxAcc,
    QLinear,
    QLinearCublasI8I32NT,
    QLinearCutlassI8I32NT,
    QLinearINT8Deploy,
    QLinearINT8Train,
    lower_qmodel_b200,
)

__all__ = ["QLinear", "QLinearINT8Deploy", "QLinearINT8Train", "QLinearCublasI8I32NT", "QLinearCutlassI8I32NT", "LinearFPxAcc", "lower_qmodel_b200"]
