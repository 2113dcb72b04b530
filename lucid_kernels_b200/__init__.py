"""B200 (sm_100a) implementation of LUCID's block-triangular forward substitution and its backward,
behind the operator interface of saisuryadv/lucid-kernels (``lucid_kernels.cute``)."""
from .cute import _forward_sub_fwd, _forward_sub_bwd, _forward_sub_bwd_dv, _forward_sub_bwd_combined
from .autograd import LUCIDForwardSub, lucid_forward_sub

__all__ = [
    "_forward_sub_fwd",
    "_forward_sub_bwd",
    "_forward_sub_bwd_dv",
    "_forward_sub_bwd_combined",
    "LUCIDForwardSub",
    "lucid_forward_sub",
]
