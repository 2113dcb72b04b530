"""CPU oracle for LUCID block-triangular forward substitution and its backward.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is the checker
used by the tests, by the smoke entry point and by the CPU-baseline leg of the benchmark.  It is a
restatement, in plain torch on the CPU, of the reference's own pure-torch definitions:

* ``build_L`` / ``forward_sub_dense``      <- test_correctness.py:12-40 (``build_L``,
  ``forward_sub_autograd``): the dense N x N lower-triangular operator and the dense solve.  This is
  THE definition of the forward result; with ``requires_grad`` inputs it is also the autograd
  definition of (dV, dK).
* ``forward_sub_blockwise``                <- bench_lucid_model.py:54-78 (``NaiveLUCIDSolve.forward``):
  the block recurrence V'_i = tril(E_ii)^-1 (V_i - sum_{j<i} E_ij V'_j), E_ij = exp(K_i K_j^T).
  Extended with the interface's ``use_diag_solve=False`` (identity diagonal blocks) and
  ``window_size`` semantics (forward_sub_interface.py:56-75).
* ``diag_inv`` / ``diag_inv_transpose``    <- forward_sub_interface.py:30-53, 177-193.
* ``backward_blockwise``                   <- forward_sub_bwd.py:3-8 (recurrence for dV) and
  forward_sub_interface.py:381-432 (``_add_diagonal_dk_correction`` / ``_backward_dk_reference``:
  dK = (dS + dS^T) K with dS = blockmask(-dV V'^T * exp(K K^T))), evaluated block by block so that no
  N x N matrix is needed.

Parity of this restatement is pinned in tests/test_oracle_golden.py against vectors produced by the
reference's own functions (tests/golden/make_golden.py extracts and executes them).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

BLOCK = 128


# --------------------------------------------------------------------------------------------
# seeded inputs (the distributions the benchmark configurations name)
# --------------------------------------------------------------------------------------------
def make_inputs(B: int, N: int, H: int, D: int = 128, *, seed: int = 0, dist: str = "baseline",
                dtype: torch.dtype = torch.bfloat16, device: str = "cpu",
                hb_slice: Optional[Tuple[int, int]] = None):
    """K, V, dV' with K ~ N(0,1) * D^-1/4 ("baseline") or N(0,1) * 0.1 ("reftest", the scale used by
    test_correctness.py:61).  Generated in fp32 from a CPU generator, then cast.

    ``hb_slice=(lo, hi)`` returns only the (batch, head) systems lo..hi-1 of the flattened index
    hb = b*H + h, as a (1, N, hi-lo, D) tensor: each system is generated from its own seed so that a
    rank holding a shard sees exactly the values the unsharded tensor has.
    """
    scale = D ** -0.25 if dist == "baseline" else 0.1
    lo, hi = (0, B * H) if hb_slice is None else hb_slice
    ks, vs, gs = [], [], []
    for hb in range(lo, hi):
        g = torch.Generator(device="cpu")
        g.manual_seed(seed * 1000003 + hb)
        ks.append(torch.randn(N, D, generator=g) * scale)
        vs.append(torch.randn(N, D, generator=g))
        gs.append(torch.randn(N, D, generator=g))

    def pack(lst):
        t = torch.stack(lst, 0)  # (nsys, N, D)
        if hb_slice is None:
            t = t.reshape(B, H, N, D).permute(0, 2, 1, 3).contiguous()
        else:
            t = t.permute(1, 0, 2).unsqueeze(0).contiguous()
        return t.to(dtype).to(device)

    return pack(ks), pack(vs), pack(gs)


# --------------------------------------------------------------------------------------------
# dense definition (small N only)
# --------------------------------------------------------------------------------------------
def build_L(K: torch.Tensor, block_size: int = BLOCK) -> torch.Tensor:
    """(B, H, N, N) block-lower-triangular operator: full exp(K_i K_j^T) blocks below the block
    diagonal, tril(exp(K_i K_i^T)) on it, zero above."""
    B, N, H, D = K.shape
    Kh = K.permute(0, 2, 1, 3)  # (B, H, N, D)
    E = torch.exp(Kh @ Kh.transpose(-1, -2))
    r = torch.arange(N, device=K.device)
    bi = (r // block_size)[:, None]
    bj = (r // block_size)[None, :]
    keep = (bj < bi) | ((bj == bi) & (r[None, :] <= r[:, None]))
    return E * keep.to(E.dtype)


def forward_sub_dense(K: torch.Tensor, V: torch.Tensor, block_size: int = BLOCK) -> torch.Tensor:
    """V' = L^-1 V through one dense triangular solve; differentiable."""
    L = build_L(K, block_size)
    Vp = torch.linalg.solve_triangular(L, V.permute(0, 2, 1, 3), upper=False)
    return Vp.permute(0, 2, 1, 3)


def dense_fwd_bwd(K: torch.Tensor, V: torch.Tensor, dVp: torch.Tensor, block_size: int = BLOCK,
                  dtype: torch.dtype = torch.float64):
    """(V', dV, dK) from the dense solve and autograd with loss = sum(V' * dV')."""
    Kd = K.detach().to(dtype).requires_grad_(True)
    Vd = V.detach().to(dtype).requires_grad_(True)
    Vp = forward_sub_dense(Kd, Vd, block_size)
    (Vp * dVp.to(dtype)).sum().backward()
    return Vp.detach(), Vd.grad.detach(), Kd.grad.detach()


# --------------------------------------------------------------------------------------------
# blockwise forms (any N)
# --------------------------------------------------------------------------------------------
def _blocks(x: torch.Tensor, bs: int) -> torch.Tensor:
    B, N, H, D = x.shape
    return x.reshape(B, N // bs, bs, H, D).permute(0, 3, 1, 2, 4)  # (B, H, T, bs, D)


def _unblocks(xb: torch.Tensor) -> torch.Tensor:
    B, H, T, bs, D = xb.shape
    return xb.permute(0, 2, 3, 1, 4).reshape(B, T * bs, H, D)


def forward_sub_blockwise(K: torch.Tensor, V: torch.Tensor, block_size: int = BLOCK, *,
                          use_diag_solve: bool = True, window_size: Optional[int] = None,
                          dtype: torch.dtype = torch.float64) -> torch.Tensor:
    Kb = _blocks(K.to(dtype), block_size)
    Vb = _blocks(V.to(dtype), block_size)
    T = Kb.shape[2]
    out = torch.zeros_like(Vb)
    for i in range(T):
        rhs = Vb[:, :, i].clone()
        j0 = 0 if window_size is None else max(0, i - window_size)
        if i > j0:
            # one batched product over all j in the window
            Kj = Kb[:, :, j0:i].reshape(Kb.shape[0], Kb.shape[1], -1, Kb.shape[-1])
            Vj = out[:, :, j0:i].reshape(Kb.shape[0], Kb.shape[1], -1, Kb.shape[-1])
            rhs -= torch.exp(Kb[:, :, i] @ Kj.transpose(-1, -2)) @ Vj
        if use_diag_solve:
            M = torch.tril(torch.exp(Kb[:, :, i] @ Kb[:, :, i].transpose(-1, -2)))
            out[:, :, i] = torch.linalg.solve_triangular(M, rhs, upper=False)
        else:
            out[:, :, i] = rhs
    return _unblocks(out)


def diag_inv(K: torch.Tensor, block_size: int = BLOCK, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """inv(tril(exp(K_i K_i^T))) per block, packed (B, T*bs, H, bs): row r of block i at sequence
    position i*bs + r."""
    Kb = _blocks(K.to(dtype), block_size)
    M = torch.tril(torch.exp(Kb @ Kb.transpose(-1, -2)))
    eye = torch.eye(block_size, dtype=dtype).expand_as(M)
    return _unblocks(torch.linalg.solve_triangular(M, eye, upper=False))


def diag_inv_transpose(K: torch.Tensor, block_size: int = BLOCK, dtype: torch.dtype = torch.float32):
    B, N, H, D = K.shape
    Db = _blocks(diag_inv(K, block_size, dtype), block_size)
    return _unblocks(Db.transpose(-1, -2).contiguous())


def backward_blockwise(K: torch.Tensor, Vp: torch.Tensor, dVp: torch.Tensor, block_size: int = BLOCK, *,
                       use_diag_solve: bool = True, dtype: torch.dtype = torch.float64):
    """(dV, dK) by the closed form.

    dV_i = tril(E_ii)^-T (dV'_i - sum_{j>i} E_ji^T dV_j), E_ji = exp(K_j K_i^T);
    dS_ij = -(dV_i V'_j^T) * E_ij for j < i, dS_ii = tril(-(dV_i V'_i^T) * E_ii) (zero when the diagonal
    blocks are the identity); dK_i = sum_j dS_ij K_j + sum_j dS_ji^T K_j.
    """
    Kb = _blocks(K.to(dtype), block_size)
    Vpb = _blocks(Vp.to(dtype), block_size)
    Gb = _blocks(dVp.to(dtype), block_size)
    B, H, T, bs, D = Kb.shape
    dV = torch.zeros_like(Gb)
    for i in range(T - 1, -1, -1):
        rhs = Gb[:, :, i].clone()
        if i + 1 < T:
            Kj = Kb[:, :, i + 1:].reshape(B, H, -1, D)
            dVj = dV[:, :, i + 1:].reshape(B, H, -1, D)
            rhs -= torch.exp(Kb[:, :, i] @ Kj.transpose(-1, -2)) @ dVj
        if use_diag_solve:
            M = torch.tril(torch.exp(Kb[:, :, i] @ Kb[:, :, i].transpose(-1, -2)))
            dV[:, :, i] = torch.linalg.solve_triangular(M.transpose(-1, -2), rhs, upper=True)
        else:
            dV[:, :, i] = rhs
    dK = torch.zeros_like(Kb)
    for i in range(T):
        # strictly-lower blocks of row i: dS_ij, j < i
        if i > 0:
            Kj = Kb[:, :, :i].reshape(B, H, -1, D)
            Vj = Vpb[:, :, :i].reshape(B, H, -1, D)
            dS = -(dV[:, :, i] @ Vj.transpose(-1, -2)) * torch.exp(Kb[:, :, i] @ Kj.transpose(-1, -2))
            dK[:, :, i] += dS @ Kj
            # the same tiles transposed feed dK_j for every j < i
            dK[:, :, :i] += (dS.transpose(-1, -2) @ Kb[:, :, i]).reshape(B, H, i, bs, D)
        if use_diag_solve:
            E = torch.exp(Kb[:, :, i] @ Kb[:, :, i].transpose(-1, -2))
            dSd = torch.tril(-(dV[:, :, i] @ Vpb[:, :, i].transpose(-1, -2)) * E)
            dK[:, :, i] += (dSd + dSd.transpose(-1, -2)) @ Kb[:, :, i]
    return _unblocks(dV), _unblocks(dK)


# --------------------------------------------------------------------------------------------
# the reference's naive CPU path (what the CPU baseline times)
# --------------------------------------------------------------------------------------------
def naive_cpu_fwd_bwd(K32: torch.Tensor, V32: torch.Tensor, dVp32: torch.Tensor, block_size: int = BLOCK):
    """fp32 dense L + torch.linalg.solve_triangular + autograd: the reference's naive path
    (test_correctness.py:34-40 with loss = (V' * dV').sum(), :66-67)."""
    return dense_fwd_bwd(K32, V32, dVp32, block_size, dtype=torch.float32)


def naive_cpu_fwd_blockwise(K: torch.Tensor, V: torch.Tensor, block_size: int = BLOCK) -> torch.Tensor:
    """fp32 blockwise loop with a 128x128 solve_triangular per block (bench_lucid_model.py:54-78)."""
    return forward_sub_blockwise(K, V, block_size, dtype=torch.float32)


# --------------------------------------------------------------------------------------------
# accounting
# --------------------------------------------------------------------------------------------
def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative Frobenius error, the metric of test_correctness.py:82-83."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def algorithmic_flops(B: int, N: int, H: int, block_size: int = BLOCK) -> Tuple[float, float]:
    """(forward, backward) algorithmic flops: per (b,h) fwd = pairs*2g + T*1.5g, bwd = pairs*5g + T*3.5g
    with g = 2*128^3 and pairs = T(T-1)/2."""
    T = N // block_size
    g = 2.0 * block_size ** 3
    pairs = T * (T - 1) / 2
    return B * H * (pairs * 2 * g + T * 1.5 * g), B * H * (pairs * 5 * g + T * 3.5 * g)
