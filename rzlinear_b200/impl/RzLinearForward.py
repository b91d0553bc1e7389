"""Same import path as the reference's python/rz_linear/impl/RzLinearForward.py."""
from .launchers import rz_linear_forward_tl  # noqa: F401
