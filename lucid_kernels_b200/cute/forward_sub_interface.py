"""Operator interface of the LUCID forward substitution, B200 build.

Same names, arguments and error behaviour as the reference's
``lucid_kernels/cute/forward_sub_interface.py`` (``_forward_sub_fwd`` :56-165, ``_forward_sub_bwd_dv``
:196-268, ``_forward_sub_bwd_combined`` :271-354, ``_forward_sub_bwd`` :357-378), so that

    from lucid_kernels_b200.cute import _forward_sub_fwd, _forward_sub_bwd

is a drop-in for ``from lucid_kernels.cute import ...``.  Differences, all behind the same signatures:

* no JIT: the kernels are ahead-of-time compiled sm_100a CUDA reached through a C ABI;
* the diagonal-block inverses are formed on the device (no ``_compute_diag_inv`` ATen pass) and the
  diagonal dK term is part of the dK kernel (no ``_add_diagonal_dk_correction`` on the host);
* ``_forward_sub_bwd_combined`` returns the FULL dK (off-diagonal and diagonal terms);
* ``use_combined_kernel=False`` still returns the full dK: the dense host formula the reference uses
  there (``_backward_dk_reference``, O(T^2) fp32 temporaries) is an oracle, not a product path;
* every call recomputes the diagonal-block inverses, as the reference does (:116, :230, :311), unless the
  caller passes ``reuse_diag=True``: then a call whose k is the very tensor of the previous call on the
  same stream (same object, unchanged version counter), such as the backward after the forward, reuses
  the inverses still in the workspace.  The autograd wrapper asks for it; ``LUCID_B200_REUSE_DIAG=1``
  makes it the default for bare calls too (only safe when nothing writes k behind torch's back);
* ``window_size=None`` is full causality, ``window_size=0`` subtracts no earlier block at all, as in the
  reference (``min(m_block, window_size)``, forward_sub_fwd.py:518-519);
* inter-block waits are bounded: with ``check=True`` (or ``LUCID_B200_CHECK=1``) the call
  synchronises and raises if a wait ran out instead of hanging.

Inputs: BSHD ``(batch, seqlen, heads_kv, head_dim)``, fp16 or bf16, head_dim == 128,
seqlen % block_size == 0, block_size == 128.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _cabi

__all__ = ["_forward_sub_fwd", "_forward_sub_bwd", "_forward_sub_bwd_dv", "_forward_sub_bwd_combined"]

_CHECK_DEFAULT = os.environ.get("LUCID_B200_CHECK", "0") not in ("0", "", "false")
_GROUP_DEFAULT = int(os.environ.get("LUCID_B200_CHAIN_GROUP", "0"))
# Default of ``reuse_diag`` for bare calls: off, i.e. every call recomputes the diagonal-block inverses as the
# reference does.  (The version counter torch keeps cannot see writes made through raw pointers.)
_REUSE_DIAG = os.environ.get("LUCID_B200_REUSE_DIAG", "0") not in ("0", "", "false")


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """TMA needs a 16-byte aligned base and strides that are multiples of 16 bytes; a tensor expanded
    along a dimension (stride 0, extent > 1) has no tensor map and is materialised."""
    if t.data_ptr() % 16 or any(s % 8 for s in t.stride()[:3]) or \
            any(s == 0 and n > 1 for s, n in zip(t.stride()[:3], t.shape[:3])):
        return t.contiguous()
    return t


def _common_asserts(k, others, block_size):
    batch_size, seqlen, num_head_kv, head_dim = k.shape
    for t in others:
        assert t.shape == (batch_size, seqlen, num_head_kv, head_dim), "all tensors must share k's shape"
    assert seqlen % block_size == 0, f"seqlen ({seqlen}) must be divisible by block_size ({block_size})"
    assert k.dtype in [torch.float16, torch.bfloat16], "inputs must be float16 or bfloat16"
    assert all(t.dtype == k.dtype for t in others), "all tensors must have the same dtype"
    assert all(t.is_cuda for t in (k, *others)), "inputs must be on CUDA device"
    assert block_size == 128 and head_dim == 128, (
        f"this build supports block_size == head_dim == 128, got {block_size} and {head_dim}")
    return batch_size, seqlen, num_head_kv, head_dim


def _timestamps_view(ws: torch.Tensor, B: int, N: int, H: int) -> torch.Tensor:
    off = _cabi.load().lucid_workspace_timestamps_offset(B, N, H)
    T = N // 128
    return ws[off:off + B * H * T * 64].view(torch.int64).view(B * H, T, 8)


def _forward_sub_fwd(
    k: torch.Tensor,
    v: torch.Tensor,
    block_size: int = 128,
    window_size: Optional[int] = None,
    no_sync: bool = False,
    instrument: bool = False,
    use_diag_solve: bool = True,
    *,
    check: Optional[bool] = None,
    chain_group: Optional[int] = None,
    k_scale: float = 1.0,
    reuse_diag: Optional[bool] = None,
) -> torch.Tensor:
    """V'_i = inv(tril(exp(K_i K_i^T))) (V_i - sum_{j<i} exp(K_i K_j^T) V'_j)   (diagonal factor only
    with ``use_diag_solve``; with ``window_size=W`` only the last W blocks are subtracted, none for W = 0).

    ``k_scale`` (extension): the operator acts on ``k_scale * k`` without the caller having to form that
    tensor (the reference's call site scales by ``d ** -0.25``, bench_lucid_model.py:164-170); the factor is
    folded into the multiplier of the exponentials.

    Returns ``v_prime`` (same shape and dtype as ``v``), or ``(v_prime, timestamps)`` with
    ``instrument``; timestamps are int64 ``(batch*heads, T, 8)`` =
    {start ns, loop end ns, published ns, ns spent waiting on flags, CTA, tiles, SM cycles, 0}.
    """
    k, v = [maybe_contiguous(t) for t in (k, v)]
    B, N, H, D = _common_asserts(k, (v,), block_size)
    k_in = k
    k, v = _aligned(k.detach()), _aligned(v.detach())
    lib = _cabi.load()
    v_prime = torch.empty_like(v, memory_format=torch.contiguous_format)
    stream = torch.cuda.current_stream(k.device).cuda_stream
    with torch.cuda.device(k.device):
        ws = _cabi.workspace(k.device, stream, B, N, H, full=False)
        flags = ((_cabi.FLAG_DIAG_SOLVE if use_diag_solve else 0) | (_cabi.FLAG_NO_SYNC if no_sync else 0) |
                 (_cabi.FLAG_INSTRUMENT if instrument else 0))
        if window_size is not None:
            assert int(window_size) >= 0, "window_size must be None or a non-negative number of blocks"
        if use_diag_solve and (_REUSE_DIAG if reuse_diag is None else reuse_diag) and \
                _cabi.diag_is_cached(k.device, stream, k_in, k_scale):
            flags |= _cabi.FLAG_REUSE_DIAG
        rc = lib.lucid_fwd_sub_scaled(k.data_ptr(), v.data_ptr(), v_prime.data_ptr(), _cabi.strides3(k),
                                      _cabi.strides3(v), _cabi.strides3(v_prime), B, N, H, D,
                                      _cabi.dtype_code(k.dtype), flags,
                                      -1 if window_size is None else int(window_size),
                                      _GROUP_DEFAULT if chain_group is None else int(chain_group),
                                      float(k_scale), ws.data_ptr(), ws.numel(), stream)
        _cabi.check_rc(rc, "lucid_fwd_sub")
        # the inverses now in the workspace belong to k_in, provided the kernels read k_in's own storage
        _cabi.diag_remember(k.device, stream, k_in, use_diag_solve and k.data_ptr() == k_in.data_ptr(), k_scale)
        if _CHECK_DEFAULT if check is None else check:
            _cabi.raise_on_device_error(ws, stream, "_forward_sub_fwd")
    if instrument:
        return v_prime, _timestamps_view(ws, B, N, H).clone()
    return v_prime


def _bwd_call(k, v_prime, dv_prime, mode, use_diag_solve, instrument, check, chain_group, what, k_in=None,
              k_scale=1.0, reuse_diag=None):
    B, N, H, D = k.shape
    k_in = k if k_in is None else k_in
    lib = _cabi.load()
    dv = torch.empty_like(dv_prime, memory_format=torch.contiguous_format)
    dk = torch.empty_like(k, memory_format=torch.contiguous_format) if mode == _cabi.BWD_COMBINED else None
    stream = torch.cuda.current_stream(k.device).cuda_stream
    with torch.cuda.device(k.device):
        ws = _cabi.workspace(k.device, stream, B, N, H, full=mode == _cabi.BWD_COMBINED)
        flags = (_cabi.FLAG_DIAG_SOLVE if use_diag_solve else 0) | (_cabi.FLAG_INSTRUMENT if instrument else 0)
        if use_diag_solve and (_REUSE_DIAG if reuse_diag is None else reuse_diag) and \
                _cabi.diag_is_cached(k.device, stream, k_in, k_scale):
            flags |= _cabi.FLAG_REUSE_DIAG
        vp_ptr = v_prime.data_ptr() if v_prime is not None else None
        vp_str = _cabi.strides3(v_prime) if v_prime is not None else _cabi.strides3(k)
        rc = lib.lucid_bwd_sub_scaled(k.data_ptr(), vp_ptr, dv_prime.data_ptr(), dv.data_ptr(),
                                      dk.data_ptr() if dk is not None else None,
                                      _cabi.strides3(k), vp_str, _cabi.strides3(dv_prime), _cabi.strides3(dv),
                                      _cabi.strides3(dk) if dk is not None else _cabi.strides3(dv),
                                      B, N, H, D, _cabi.dtype_code(k.dtype), flags, mode,
                                      _GROUP_DEFAULT if chain_group is None else int(chain_group),
                                      float(k_scale), ws.data_ptr(), ws.numel(), stream)
        _cabi.check_rc(rc, what)
        _cabi.diag_remember(k.device, stream, k_in, use_diag_solve and k.data_ptr() == k_in.data_ptr(), k_scale)
        if _CHECK_DEFAULT if check is None else check:
            _cabi.raise_on_device_error(ws, stream, what)
    ts = _timestamps_view(ws, B, N, H).clone() if instrument else None
    return dv, dk, ts


def _forward_sub_bwd_dv(
    k: torch.Tensor,
    dv_prime: torch.Tensor,
    block_size: int = 128,
    use_diag_solve: bool = True,
    instrument: bool = False,
    *,
    check: Optional[bool] = None,
    chain_group: Optional[int] = None,
    k_scale: float = 1.0,
    reuse_diag: Optional[bool] = None,
) -> torch.Tensor:
    """dV_i = inv(tril(exp(K_i K_i^T)))^T (dV'_i - sum_{j>i} exp(K_i K_j^T) dV_j), solved from the last
    block to the first."""
    k, dv_prime = [maybe_contiguous(t) for t in (k, dv_prime)]
    _common_asserts(k, (dv_prime,), block_size)
    k_in = k
    k, dv_prime = _aligned(k.detach()), _aligned(dv_prime.detach())
    dv, _, ts = _bwd_call(k, None, dv_prime, _cabi.BWD_DV_ONLY, use_diag_solve, instrument, check, chain_group,
                          "_forward_sub_bwd_dv", k_in=k_in, k_scale=k_scale, reuse_diag=reuse_diag)
    if instrument:
        return dv, ts
    return dv


def _forward_sub_bwd_combined(
    k: torch.Tensor,
    v_prime: torch.Tensor,
    dv_prime: torch.Tensor,
    block_size: int = 128,
    use_diag_solve: bool = True,
    instrument: bool = False,
    *,
    check: Optional[bool] = None,
    chain_group: Optional[int] = None,
    k_scale: float = 1.0,
    reuse_diag: Optional[bool] = None,
) -> tuple:
    """(dv, dk).  Unlike the reference, ``dk`` already contains the diagonal-block term.  With ``k_scale``
    the operator acts on ``k_scale * k`` and ``dk`` is the gradient with respect to ``k`` itself."""
    k, v_prime, dv_prime = [maybe_contiguous(t) for t in (k, v_prime, dv_prime)]
    _common_asserts(k, (v_prime, dv_prime), block_size)
    k_in = k
    k, v_prime, dv_prime = [_aligned(t.detach()) for t in (k, v_prime, dv_prime)]
    dv, dk, ts = _bwd_call(k, v_prime, dv_prime, _cabi.BWD_COMBINED, use_diag_solve, instrument, check,
                           chain_group, "_forward_sub_bwd_combined", k_in=k_in, k_scale=k_scale, reuse_diag=reuse_diag)
    if instrument:
        return dv, dk, ts
    return dv, dk


def _forward_sub_bwd(
    k: torch.Tensor,
    v_prime: torch.Tensor,
    dv_prime: torch.Tensor,
    block_size: int = 128,
    use_diag_solve: bool = True,
    use_combined_kernel: bool = False,
    *,
    check: Optional[bool] = None,
    chain_group: Optional[int] = None,
    k_scale: float = 1.0,
    reuse_diag: Optional[bool] = None,
) -> tuple:
    """Full backward pass: returns ``(dv, dk)``, gradients w.r.t. V and K.  Both settings of
    ``use_combined_kernel`` run the same device kernels here."""
    del use_combined_kernel
    return _forward_sub_bwd_combined(k, v_prime, dv_prime, block_size=block_size,
                                     use_diag_solve=use_diag_solve, check=check, chain_group=chain_group,
                                     k_scale=k_scale, reuse_diag=reuse_diag)
