"""Mirror of ``lucid_kernels.cute`` (lucid_kernels/cute/__init__.py:1-13): re-exports the operator
interface."""
from .forward_sub_interface import (
    _forward_sub_fwd,
    _forward_sub_bwd,
    _forward_sub_bwd_dv,
    _forward_sub_bwd_combined,
)

__all__ = [
    "_forward_sub_fwd",
    "_forward_sub_bwd",
    "_forward_sub_bwd_dv",
    "_forward_sub_bwd_combined",
]
