"""Autograd wrapper of the LUCID solve.

Mirrors ``LUCIDForwardSub`` of the reference's benchmark scripts (bench_lucid_model.py:34-51,
bench_lucid_e2e.py:34-49): forward saves ``(k, v_prime)``, backward returns ``(dk, dv)`` in the order of
the inputs ``(k, v)``.  The backward reuses the diagonal-block inverses the forward left in the workspace
when they are still there: autograd refuses to run a backward whose saved ``k`` was modified in place, so
between the two calls of one node ``k`` is known to be unchanged.
"""
from __future__ import annotations

import torch

from .cute.forward_sub_interface import _forward_sub_fwd, _forward_sub_bwd


class LUCIDForwardSub(torch.autograd.Function):
    """``v_prime = LUCIDForwardSub.apply(k, v)`` with k, v in BSHD layout."""

    @staticmethod
    def forward(ctx, k, v, block_size=128, k_scale=1.0):
        v_prime = _forward_sub_fwd(k, v, block_size=block_size, use_diag_solve=True, k_scale=k_scale)
        ctx.save_for_backward(k, v_prime)
        ctx.block_size = block_size
        ctx.k_scale = k_scale
        return v_prime

    @staticmethod
    def backward(ctx, dv_prime):
        k, v_prime = ctx.saved_tensors
        dv, dk = _forward_sub_bwd(k, v_prime, dv_prime, block_size=ctx.block_size, use_diag_solve=True,
                                  use_combined_kernel=True, k_scale=ctx.k_scale, reuse_diag=True)
        return dk, dv, None, None


def lucid_forward_sub(k: torch.Tensor, v: torch.Tensor, k_scale: float = 1.0) -> torch.Tensor:
    """``k_scale``: the solve acts on ``k_scale * k`` (folded into the kernels); gradients are with respect
    to ``k`` and ``v`` as passed."""
    return LUCIDForwardSub.apply(k, v, 128, k_scale)
