"""rzlinear_b200: the RzLinear (ROBE-Z compressed linear layer) hot path on NVIDIA B200.

Same public names as the reference's `rz_linear` package:
    from rzlinear_b200 import RzLinear, RzLinearFunction, controls
"""
from .RzLinearFunction import RzLinearFunction, RzConfig, controls  # noqa: F401
from .RzLinear import RzLinear  # noqa: F401

__all__ = ["RzLinear", "RzLinearFunction", "RzConfig", "controls"]
