"""Same import path as the reference's python/rz_linear/impl/RzLinearBackward.py."""
from .launchers import (rz_linear_backward_tl, rz_linear_backward_input_grad_tl,  # noqa: F401
                        rz_linear_backward_weight_grad_tl)
