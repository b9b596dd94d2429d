"""Quantized Linear modules (mirror of fms_mo/modules/linear.py for the B200 path)."""

from .linear import LinearFPxAcc, QLinear, QLinearINT8Deploy, QLinearINT8Train

__all__ = ["QLinear", "QLinearINT8Deploy", "QLinearINT8Train", "LinearFPxAcc"]
