"""Same import path as the reference's python/rz_linear/impl/RzLinearIdx.py."""
from .launchers import rz_linear_idx_tl  # noqa: F401
