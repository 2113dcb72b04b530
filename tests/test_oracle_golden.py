"""Pin the CPU oracle against vectors produced by the reference's own functions.

tests/golden/*.npz were written by tests/golden/make_golden.py, which executes the reference's
``build_L`` / ``forward_sub_autograd`` (test_correctness.py:12-40), ``_compute_diag_inv``,
``_compute_diag_inv_transpose``, ``_add_diagonal_dk_correction``, ``_backward_dk_reference``
(forward_sub_interface.py:30-53,177-193,381-432) and ``NaiveLUCIDSolve.forward``
(bench_lucid_model.py:54-78) on seeded inputs.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = sorted(glob.glob(os.path.join(GOLD, "t*.npz")))


def _load(path):
    z = np.load(path)
    return {k: torch.from_numpy(z[k]) for k in z.files}


def test_fixtures_present():
    assert len(CASES) == 3
    assert os.path.exists(os.path.join(GOLD, "c1_fp32_seed0.npz"))


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_dense_oracle_matches_reference_autograd(path):
    g = _load(path)
    Vp, dV, dK = orc.dense_fwd_bwd(g["K"], g["V"], g["dVp"])
    # same algorithm, same fp64 arithmetic: agreement to rounding
    assert orc.rel_err(Vp, g["Vp"]) < 1e-12
    assert orc.rel_err(dV, g["dV"]) < 1e-12
    assert orc.rel_err(dK, g["dK"]) < 1e-11
    L = orc.build_L(g["K"].double())
    N = L.shape[-1]
    assert abs(float(L.sum()) - float(g["L_checksum"][0])) <= 1e-9 * abs(float(g["L_checksum"][0]))
    assert float((L != 0).sum()) == float(g["L_checksum"][2])
    assert torch.allclose(L[0, 0, N - 1], g["L_row"], rtol=1e-13, atol=0)


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_blockwise_forms_match_reference(path):
    g = _load(path)
    Vp = orc.forward_sub_blockwise(g["K"], g["V"])
    assert orc.rel_err(Vp, g["Vp"]) < 1e-10
    dV, dK = orc.backward_blockwise(g["K"], g["Vp"], g["dVp"])
    assert orc.rel_err(dV, g["dV"]) < 1e-10
    assert orc.rel_err(dK, g["dK"]) < 1e-9
    # fp32 host pieces of the reference interface
    assert orc.rel_err(orc.diag_inv(g["K"]), g["diag_inv"]) < 1e-5
    assert orc.rel_err(orc.diag_inv_transpose(g["K"]), g["diag_inv_t"]) < 1e-5
    assert orc.rel_err(orc.naive_cpu_fwd_blockwise(g["K"], g["V"]), g["naive_fwd_fp32"]) < 1e-5
    # the reference's closed-form fp32 dK agrees with its own autograd result, and so does ours
    assert orc.rel_err(g["dK_reference_fp32"], g["dK"]) < 1e-4
    _, dK32 = orc.backward_blockwise(g["K"], g["Vp"], g["dVp"], dtype=torch.float32)
    assert orc.rel_err(dK32, g["dK_reference_fp32"]) < 1e-4


def test_c1_configuration_fp32():
    """B=1, N=512, H=4, d=128, fp32, seed 0: the reference's CPU-runnable configuration."""
    g = _load(os.path.join(GOLD, "c1_fp32_seed0.npz"))
    Vp, dV, dK = orc.naive_cpu_fwd_bwd(g["K"], g["V"], g["dVp"])
    H = 4
    for name, t in (("Vp", Vp), ("dV", dV), ("dK", dK)):
        norms = t.permute(2, 0, 1, 3).reshape(H, -1).norm(dim=1)
        assert torch.allclose(norms, g[f"{name}_head_norms"], rtol=1e-4), name
        assert orc.rel_err(t[:, :, 0], g[f"{name}_head0"]) < 1e-4, name


def test_oracle_edge_semantics():
    K, V, G = orc.make_inputs(1, 384, 2, dtype=torch.float64)
    # identity diagonal blocks and window truncation
    full = orc.forward_sub_blockwise(K, V, use_diag_solve=False)
    w_all = orc.forward_sub_blockwise(K, V, use_diag_solve=False, window_size=99)
    assert torch.equal(full, w_all)
    w1 = orc.forward_sub_blockwise(K, V, use_diag_solve=False, window_size=1)
    assert torch.equal(w1[:, :256], full[:, :256]) and not torch.equal(w1[:, 256:], full[:, 256:])
    # T = 1: a single diagonal block
    K1, V1, G1 = orc.make_inputs(2, 128, 3, dtype=torch.float64)
    Vp, dV, dK = orc.dense_fwd_bwd(K1, V1, G1)
    assert orc.rel_err(orc.forward_sub_blockwise(K1, V1), Vp) < 1e-12
    dV2, dK2 = orc.backward_blockwise(K1, Vp, G1)
    assert orc.rel_err(dV2, dV) < 1e-12 and orc.rel_err(dK2, dK) < 1e-11


def test_sharded_inputs_equal_unsharded():
    K, V, G = orc.make_inputs(2, 256, 4, dtype=torch.float32)
    for lo, hi in ((0, 2), (2, 8), (5, 6)):
        Ks, Vs, Gs = orc.make_inputs(2, 256, 4, dtype=torch.float32, hb_slice=(lo, hi))
        ref = K.permute(0, 2, 1, 3).reshape(8, 256, 128)[lo:hi].permute(1, 0, 2).unsqueeze(0)
        assert torch.equal(Ks, ref)


def test_flop_accounting():
    f, b = orc.algorithmic_flops(2, 32768, 8)
    assert abs(f / 1e12 - 4.407) < 0.01 and abs(b / 1e12 - 11.01) < 0.01
    f, _ = orc.algorithmic_flops(1, 8192, 8)
    assert abs(f / 1e12 - 0.1385) < 0.001
