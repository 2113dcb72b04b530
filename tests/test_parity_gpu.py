"""Parity of the CUDA path against the CPU oracle, through the operator interface / C ABI.

Gates (relative Frobenius error against the fp64 oracle evaluated on the same 16-bit input values):
V' <= 1 %, dV <= 1 %, dK <= 2 % on the benchmark distribution K ~ N(0,1) * d^-1/4.  On the
reference's own test distribution (K ~ N(0,1) * 0.1, test_correctness.py:61) the reference gates dV
and dK at 5 % for T <= 8 (test_correctness.py:84-85); the same gate is used here.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ops():
    from lucid_kernels_b200 import _cabi
    from lucid_kernels_b200 import cute

    _cabi.load()  # raises if the library is missing: there is no fallback to test
    return cute


def _gates(dist):
    return (0.01, 0.01, 0.02) if dist == "baseline" else (0.05, 0.05, 0.05)


def _run_all(ops, K, V, G, diag=True):
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, use_diag_solve=diag, check=True)
    dv, dk = ops._forward_sub_bwd(Kc, vp, Gc, use_diag_solve=diag, use_combined_kernel=True, check=True)
    return vp, dv, dk


@pytest.mark.parametrize("B,N,H", [(1, 128, 1), (1, 256, 1), (1, 384, 1), (1, 512, 4), (1, 1024, 1),
                                   (2, 512, 3), (2, 2048, 8)])
@pytest.mark.parametrize("dist", ["baseline", "reftest"])
def test_fwd_bwd_vs_dense_oracle(ops, B, N, H, dist):
    K, V, G = orc.make_inputs(B, N, H, dist=dist, dtype=torch.bfloat16, seed=N + H)
    vp, dv, dk = _run_all(ops, K, V, G)
    rvp, rdv, rdk = orc.dense_fwd_bwd(K, V, G)
    g = _gates(dist)
    assert orc.rel_err(vp, rvp) < g[0]
    # the backward is given the kernel's own V' (as the autograd wrapper does)
    assert orc.rel_err(dv, rdv) < g[1]
    assert orc.rel_err(dk, rdk) < g[2]
    assert not torch.isnan(vp.float()).any() and not torch.isnan(dk.float()).any()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "t*.npz"))),
                         ids=lambda p: os.path.basename(p)[:-4])
def test_against_reference_golden_vectors(ops, path):
    """Inputs and fp64 results stored by the reference's own functions (tests/golden/make_golden.py)."""
    z = np.load(path)
    K, V, G = [torch.from_numpy(z[n]).bfloat16() for n in ("K", "V", "dVp")]
    assert torch.equal(K.float(), torch.from_numpy(z["K"]))  # stored values are bf16-representable
    vp, dv, dk = _run_all(ops, K, V, G)
    g = _gates("reftest" if "reftest" in path else "baseline")
    assert orc.rel_err(vp, torch.from_numpy(z["Vp"])) < g[0]
    assert orc.rel_err(dv, torch.from_numpy(z["dV"])) < g[1]
    assert orc.rel_err(dk, torch.from_numpy(z["dK"])) < g[2]


def test_c1_configuration(ops):
    """B=1, N=512, H=4 (the reference's CPU-runnable configuration); golden values are fp32 results of
    the reference's naive path on unquantised fp32 inputs, so the gate includes bf16 input rounding."""
    z = np.load(os.path.join(GOLD, "c1_fp32_seed0.npz"))
    K, V, G = [torch.from_numpy(z[n]).bfloat16() for n in ("K", "V", "dVp")]
    vp, dv, dk = _run_all(ops, K, V, G)
    assert orc.rel_err(vp[:, :, 0], torch.from_numpy(z["Vp_head0"])) < 0.02
    assert orc.rel_err(dv[:, :, 0], torch.from_numpy(z["dV_head0"])) < 0.02
    assert orc.rel_err(dk[:, :, 0], torch.from_numpy(z["dK_head0"])) < 0.03


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fp16_and_bf16(ops, dtype):
    K, V, G = orc.make_inputs(1, 1024, 2, dist="reftest", dtype=dtype)
    vp, dv, dk = _run_all(ops, K, V, G)
    rvp, rdv, rdk = orc.dense_fwd_bwd(K, V, G)
    gate = 0.01 if dtype == torch.float16 else 0.05
    assert orc.rel_err(vp, rvp) < gate and orc.rel_err(dv, rdv) < gate and orc.rel_err(dk, rdk) < gate


def test_identity_diagonal_and_window(ops):
    K, V, G = orc.make_inputs(2, 1024, 2, dtype=torch.bfloat16)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    out = ops._forward_sub_fwd(Kc, Vc, use_diag_solve=False, check=True)
    assert orc.rel_err(out, orc.forward_sub_blockwise(K, V, use_diag_solve=False)) < 0.01
    # window 0 subtracts no earlier block (only the diagonal-block solve), as in the reference
    # (min(m_block, window_size), forward_sub_fwd.py:518-519); None is full causality
    for w in (0, 1, 3):
        out = ops._forward_sub_fwd(Kc, Vc, use_diag_solve=True, window_size=w, check=True)
        assert orc.rel_err(out, orc.forward_sub_blockwise(K, V, window_size=w)) < 0.01
    full = ops._forward_sub_fwd(Kc, Vc, use_diag_solve=True, window_size=None, check=True)
    assert orc.rel_err(full, orc.forward_sub_blockwise(K, V)) < 0.01
    with pytest.raises(AssertionError):
        ops._forward_sub_fwd(Kc, Vc, window_size=-2)
    vp = orc.forward_sub_blockwise(K, V, use_diag_solve=False).bfloat16()
    dv, dk = ops._forward_sub_bwd(Kc, vp.cuda(), Gc, use_diag_solve=False, use_combined_kernel=True, check=True)
    rdv, rdk = orc.backward_blockwise(K, vp, G, use_diag_solve=False)
    assert orc.rel_err(dv, rdv) < 0.01 and orc.rel_err(dk, rdk) < 0.02
    dv_only = ops._forward_sub_bwd_dv(Kc, Gc, use_diag_solve=False, check=True)
    assert torch.equal(dv_only, dv)


def test_strided_views_and_repeated_calls(ops):
    """Head-sliced and BHSD-transposed views (non-contiguous BSHD), poison-filled outputs are fully
    overwritten, and a workspace reused by back-to-back calls gives identical results."""
    K, V, G = orc.make_inputs(2, 512, 4, dtype=torch.bfloat16)
    Kc, Vc = K.cuda(), V.cuda()
    full = ops._forward_sub_fwd(Kc, Vc, check=True)
    again = ops._forward_sub_fwd(Kc, Vc, check=True)
    assert torch.equal(full, again)
    sl = ops._forward_sub_fwd(Kc[:, :, 1:3], Vc[:, :, 1:3], check=True)
    assert torch.equal(sl, full[:, :, 1:3])
    k_bhsd = Kc.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)   # BSHD view of BHSD storage
    v_bhsd = Vc.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert not k_bhsd.is_contiguous()
    tr = ops._forward_sub_fwd(k_bhsd, v_bhsd, check=True)
    assert torch.equal(tr, full)


def test_autograd_wrapper_order(ops):
    from lucid_kernels_b200 import LUCIDForwardSub

    K, V, G = orc.make_inputs(1, 512, 2, dtype=torch.bfloat16)
    k = K.cuda().requires_grad_(True)
    v = V.cuda().requires_grad_(True)
    vp = LUCIDForwardSub.apply(k, v)
    vp.backward(G.cuda())
    rvp, rdv, rdk = orc.dense_fwd_bwd(K, V, G)
    assert orc.rel_err(k.grad, rdk) < 0.02 and orc.rel_err(v.grad, rdv) < 0.01


def test_two_streams_concurrently(ops):
    K, V, G = orc.make_inputs(1, 2048, 4, dtype=torch.bfloat16)
    Kc, Vc = K.cuda(), V.cuda()
    ref = ops._forward_sub_fwd(Kc, Vc, check=True)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(s1):
        a = ops._forward_sub_fwd(Kc, Vc)
    with torch.cuda.stream(s2):
        b = ops._forward_sub_fwd(Kc, Vc)
    torch.cuda.synchronize()
    assert torch.equal(a, ref) and torch.equal(b, ref)


def test_large_sizes_by_properties(ops):
    """N = 32768 (T = 256): too large for the dense oracle.  Checked through (i) the blockwise fp64 oracle
    on one (batch, head) system and (ii) linearity in V: solve(K, a V1 + b V2) = a solve(K, V1) + b solve(K, V2)."""
    B, N, H = 1, 32768, 2
    K, V, G = orc.make_inputs(B, N, H, dtype=torch.bfloat16)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, check=True)
    dv, dk = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
    # (i) one system against the blockwise oracle, computed on the GPU in fp64
    k1, v1, g1 = [t[:, :, :1].cuda().double() for t in (K, V, G)]
    rvp = orc.forward_sub_blockwise(k1, v1)
    assert orc.rel_err(vp[:, :, :1], rvp) < 0.01
    rdv, rdk = orc.backward_blockwise(k1, vp[:, :, :1].double(), g1)
    assert orc.rel_err(dv[:, :, :1], rdv) < 0.01
    assert orc.rel_err(dk[:, :, :1], rdk) < 0.02
    # (ii) linearity
    V2 = torch.flip(Vc, dims=[1])
    vp2 = ops._forward_sub_fwd(Kc, V2, check=True)
    comb = ops._forward_sub_fwd(Kc, (0.5 * Vc.float() + 2.0 * V2.float()).bfloat16(), check=True)
    assert orc.rel_err(comb, 0.5 * vp.float() + 2.0 * vp2.float()) < 0.01


@pytest.mark.parametrize("dtype,H", [(torch.bfloat16, 2), (torch.float16, 1)])
def test_backward_in_one_launch_matches_separate_launches(ops, dtype, H):
    """With one or two systems per GPU the combined backward runs the reverse solve and the dK program in one
    launch (the dK CTAs follow the solve's flags).  With whole row-blocks as dK work items: same arithmetic in
    the same order, bit-identical.  With a row-block's tiles dealt out as two items (the default there) the two
    fp32 partial sums are added at the end instead of one running sum: dV bit-identical, dK equal to rounding."""
    from lucid_kernels_b200 import _cabi

    lib = _cabi.load()
    K, V, G = orc.make_inputs(1, 32768, H, dtype=dtype, seed=11)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, check=True)
    try:
        lib.lucid_set_fused_backward(0, 0)                      # separate launches: reverse solve, then dK over all tiles
        lib.lucid_set_upper_in_solve(0)
        dv0, dk0 = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
        for solve_ctas in (0, 20, 120):                         # automatic share, a small and a large one
            lib.lucid_set_fused_backward(2, solve_ctas)
            lib.lucid_set_dk_split(0)
            dv1, dk1 = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
            assert torch.equal(dv0, dv1) and torch.equal(dk0, dk1), solve_ctas
            lib.lucid_set_dk_split(1)
            dv2, dk2 = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
            assert torch.equal(dv0, dv2), solve_ctas
            rel = float((dk2.float() - dk0.float()).norm() / dk0.float().norm())
            assert rel < 1e-3, (solve_ctas, rel)                # bf16/fp16 rounding of a differently ordered sum
    finally:
        lib.lucid_set_fused_backward(2, 0)                      # library defaults
        lib.lucid_set_dk_split(1)
        lib.lucid_set_upper_in_solve(1)
    assert bool(torch.isfinite(dk0.float()).all())


def test_pair_mode_matches_single_row_blocks(ops):
    """With few chains the stand-alone solve kernels run as clusters of two CTAs that solve pairs of
    row-blocks and hand the first result to the second through shared memory.  Same arithmetic in the same
    order as single row-blocks: bit-identical, forward and reverse, bf16 and fp16."""
    from lucid_kernels_b200 import _cabi

    lib = _cabi.load()
    for dtype, (B, N, H) in ((torch.bfloat16, (1, 8192, 8)), (torch.float16, (1, 4096, 3)), (torch.bfloat16, (2, 256, 1))):
        K, V, G = orc.make_inputs(B, N, H, dtype=dtype, seed=31)
        Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
        try:
            lib.lucid_set_pair_solve(0)
            lib.lucid_set_fused_backward(0, 0)
            vp0 = ops._forward_sub_fwd(Kc, Vc, check=True)
            dv0 = ops._forward_sub_bwd_dv(Kc, Gc, check=True)
            lib.lucid_set_pair_solve(8)
            vp1 = ops._forward_sub_fwd(Kc, Vc, check=True)
            dv1 = ops._forward_sub_bwd_dv(Kc, Gc, check=True)
        finally:
            lib.lucid_set_pair_solve(8)
            lib.lucid_set_fused_backward(2, 0)
        assert torch.equal(vp0, vp1) and torch.equal(dv0, dv1), (dtype, B, N, H)


def test_group_overlap_only_reorders_the_work(ops):
    """Scheduler knob: the start of a group of chains dealt out alternately with the end of the group before.
    Every row-block is still solved by one CTA from the same inputs: bit-identical results, forward and
    reverse, for an overlap shorter than, equal to and (clamped) longer than half the row-blocks."""
    from lucid_kernels_b200 import _cabi

    lib = _cabi.load()
    K, V, G = orc.make_inputs(2, 2048, 3, dtype=torch.bfloat16, seed=37)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    try:
        lib.lucid_set_pair_solve(0)
        lib.lucid_set_group_overlap(0)
        vp0 = ops._forward_sub_fwd(Kc, Vc, check=True, chain_group=2)
        dv0 = ops._forward_sub_bwd_dv(Kc, Gc, check=True, chain_group=2)
        for steps in (3, 8, 100):
            lib.lucid_set_group_overlap(steps)
            vp1 = ops._forward_sub_fwd(Kc, Vc, check=True, chain_group=2)
            dv1 = ops._forward_sub_bwd_dv(Kc, Gc, check=True, chain_group=2)
            assert torch.equal(vp0, vp1) and torch.equal(dv0, dv1), steps
    finally:
        lib.lucid_set_pair_solve(8)
        lib.lucid_set_group_overlap(-1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_key_scale_folded_into_the_kernels(ops, dtype):
    """k_scale: the operator acts on k_scale * k while the kernels read k itself.  Checked against the fp64
    oracle on k_scale * k (same 16-bit k), with dK chained back to the unscaled k; and the autograd wrapper
    hands the same gradients out."""
    from lucid_kernels_b200 import lucid_forward_sub

    s = 128 ** -0.25
    Ks, V, G = orc.make_inputs(2, 1024, 2, dtype=torch.float32, seed=3)
    K = (Ks / s).to(dtype)                                    # unscaled keys, N(0, 1), rounded to 16 bits
    V, G = V.to(dtype), G.to(dtype)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, k_scale=s, check=True)
    dv, dk = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, k_scale=s, check=True)
    rvp, rdv, rdk_scaled = orc.dense_fwd_bwd(K.double() * s, V, G)
    assert orc.rel_err(vp, rvp) < 0.01
    assert orc.rel_err(dv, rdv) < 0.01
    assert orc.rel_err(dk, rdk_scaled * s) < 0.02
    # a different scale on the same k must not reuse the diagonal inverses of the first call
    vp2 = ops._forward_sub_fwd(Kc, Vc, k_scale=0.5 * s, check=True)
    rvp2 = orc.forward_sub_dense(K.double() * (0.5 * s), V.double())
    assert orc.rel_err(vp2, rvp2) < 0.01
    # autograd wrapper
    Kg, Vg = Kc.clone().requires_grad_(True), Vc.clone().requires_grad_(True)
    out = lucid_forward_sub(Kg, Vg, k_scale=s)
    (out.float() * Gc.float()).sum().backward()
    assert torch.equal(out.detach(), vp) and torch.equal(Vg.grad, dv) and torch.equal(Kg.grad, dk)


def test_calls_can_be_captured_in_a_cuda_graph(ops):
    """A forward + backward step issues only stream-ordered work (memsets, kernels), so it can be captured
    once and replayed; the replay must reproduce the eager results bit for bit, also after the inputs'
    contents change in place."""
    K, V, G = orc.make_inputs(1, 2048, 2, dtype=torch.bfloat16, seed=21)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()

    def step():
        vp = ops._forward_sub_fwd(Kc, Vc)
        dv, dk = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True)
        return vp, dv, dk

    ref = [t.clone() for t in step()]
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        out = step()
    g.replay()
    torch.cuda.synchronize()
    for a, b in zip(out, ref):
        assert torch.equal(a, b)
    # new values in the same buffers: the captured forward recomputes the diagonal inverses itself
    K2, V2, G2 = orc.make_inputs(1, 2048, 2, dtype=torch.bfloat16, seed=22)
    Kc.copy_(K2.cuda()); Vc.copy_(V2.cuda()); Gc.copy_(G2.cuda())
    g.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in out]
    ref2 = step()
    for a, b in zip(got, ref2):
        assert torch.equal(a, b)
    rvp, rdv, rdk = orc.dense_fwd_bwd(K2, V2, G2)
    assert orc.rel_err(got[0], rvp) < 0.01 and orc.rel_err(got[1], rdv) < 0.01 and orc.rel_err(got[2], rdk) < 0.02


def test_argument_errors(ops):
    K, V, _ = orc.make_inputs(1, 256, 1, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        ops._forward_sub_fwd(K.cuda()[:, :200], V.cuda()[:, :200])          # seqlen % 128 != 0
    with pytest.raises(AssertionError):
        ops._forward_sub_fwd(K.cuda().float(), V.cuda().float())            # dtype
    with pytest.raises(AssertionError):
        ops._forward_sub_fwd(K.cuda(), V.cuda().half())                     # mixed dtypes
    with pytest.raises(AssertionError):
        ops._forward_sub_fwd(K, V)                                          # not on CUDA


def test_diag_inverse_reuse_is_opt_in_and_safe(ops):
    """Bare calls recompute the diagonal-block inverses every time, like the reference.  With reuse_diag=True the
    backward after a forward on the same k object reuses those left in the workspace; a different k (even one
    that lands at the same address) or an in-place update must not."""
    from lucid_kernels_b200 import _cabi

    K, V, G = orc.make_inputs(1, 512, 2, dtype=torch.bfloat16, seed=5)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, check=True)
    stream = torch.cuda.current_stream().cuda_stream
    assert _cabi.diag_is_cached(Kc.device, stream, Kc)
    dv_cached, dk_cached = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True, reuse_diag=True)
    dv_fresh, dk_fresh = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)   # default: recompute
    assert torch.equal(dv_cached, dv_fresh) and torch.equal(dk_cached, dk_fresh)
    # a writer torch cannot see (raw pointer): the default path is still right, because it never trusts the cache
    K1, _, _ = orc.make_inputs(1, 512, 2, dtype=torch.bfloat16, seed=55)
    Kc.data.copy_(K1.cuda())           # (this one does bump the counter; the point is the default below)
    vp1 = ops._forward_sub_fwd(Kc, Vc, check=True)
    assert orc.rel_err(vp1, orc.forward_sub_blockwise(K1, V)) < 0.01
    # a new tensor of the same shape, possibly at the same address, is not a cache hit
    addr = Kc.data_ptr()
    del Kc
    K2, V2, _ = orc.make_inputs(1, 512, 2, dtype=torch.bfloat16, seed=6)
    K2c = K2.cuda()
    assert not _cabi.diag_is_cached(K2c.device, stream, K2c), (addr == K2c.data_ptr())
    vp2 = ops._forward_sub_fwd(K2c, V2.cuda(), check=True, reuse_diag=True)
    assert orc.rel_err(vp2, orc.forward_sub_blockwise(K2, V2)) < 0.01
    # an in-place update bumps the version counter
    K2c.mul_(0.5)
    assert not _cabi.diag_is_cached(K2c.device, stream, K2c)
    vp3 = ops._forward_sub_fwd(K2c, V2.cuda(), check=True, reuse_diag=True)
    assert orc.rel_err(vp3, orc.forward_sub_blockwise(K2c.cpu(), V2)) < 0.01


def test_dv_only_backward_with_the_diagonal_solve(ops):
    """_forward_sub_bwd_dv(use_diag_solve=True) against the oracle and against the combined path's dV."""
    K, V, G = orc.make_inputs(2, 1024, 3, dtype=torch.bfloat16, seed=9)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, check=True)
    dv_only = ops._forward_sub_bwd_dv(Kc, Gc, use_diag_solve=True, check=True)
    dv, _ = ops._forward_sub_bwd_combined(Kc, vp, Gc, use_diag_solve=True, check=True)
    assert torch.equal(dv_only, dv)
    rdv, _ = orc.backward_blockwise(K, vp.cpu(), G)
    assert orc.rel_err(dv_only, rdv) < 0.01


def test_expanded_inputs_are_materialised_not_misread(ops):
    """k expanded over the heads (stride 0, the GQA broadcast pattern) has no tensor map: the interface makes
    it contiguous, and the C ABI refuses such strides outright instead of reading neighbouring rows."""
    import ctypes
    from lucid_kernels_b200 import _cabi

    K, V, _ = orc.make_inputs(1, 512, 1, dtype=torch.bfloat16, seed=13)
    _, V4, _ = orc.make_inputs(1, 512, 4, dtype=torch.bfloat16, seed=14)
    Kc, V4c = K.cuda(), V4.cuda()
    k_exp = Kc.expand(1, 512, 4, 128)
    assert k_exp.stride(2) == 0
    out = ops._forward_sub_fwd(k_exp, V4c, check=True)
    ref = orc.forward_sub_blockwise(K.expand(1, 512, 4, 128), V4)
    assert orc.rel_err(out, ref) < 0.01
    lib = _cabi.load()
    ws = _cabi.workspace(Kc.device, torch.cuda.current_stream().cuda_stream, 1, 512, 4)
    res = torch.empty_like(V4c)
    rc = lib.lucid_fwd_sub(k_exp.data_ptr(), V4c.data_ptr(), res.data_ptr(), _cabi.strides3(k_exp),
                           _cabi.strides3(V4c), _cabi.strides3(res), 1, 512, 4, 128, 1, 1, -1, 0, ws.data_ptr(),
                           ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == -9 and b"stride" in lib.lucid_status_string(rc)


def test_step_captured_twice_replays_with_fresh_inverses(ops):
    """The usual static-input pattern: capture the step, later capture it again with the same K object, write
    new values into K, replay.  Each capture works in its own workspace and recomputes the diagonal inverses
    inside the graph, so neither replay can solve with inverses of earlier contents."""
    K, V, G = orc.make_inputs(1, 1024, 2, dtype=torch.bfloat16, seed=61)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()

    def step():
        vp = ops._forward_sub_fwd(Kc, Vc)
        dv, dk = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, reuse_diag=True)
        return vp, dv, dk

    s = torch.cuda.Stream()
    step()                                            # an eager call first, on the current stream
    torch.cuda.synchronize()
    graphs, outs = [], []
    for _ in range(2):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
            outs.append(step())
        graphs.append(g)
        with torch.cuda.stream(s):
            step()                                    # and an eager call on the capture stream in between
        torch.cuda.synchronize()
    K2, V2, G2 = orc.make_inputs(1, 1024, 2, dtype=torch.bfloat16, seed=62)
    Kc.copy_(K2.cuda()); Vc.copy_(V2.cuda()); Gc.copy_(G2.cuda())
    rvp, rdv, rdk = orc.dense_fwd_bwd(K2, V2, G2)
    for g, out in zip(graphs, outs):
        g.replay()
        torch.cuda.synchronize()
        assert orc.rel_err(out[0], rvp) < 0.01 and orc.rel_err(out[1], rdv) < 0.01 and orc.rel_err(out[2], rdk) < 0.02


def test_two_streams_with_pairs_of_row_blocks(ops):
    """Two forward solves of a pair-eligible shape (clusters of two CTAs) on two streams at once: neither launch
    has the GPU to itself, so pairs must be claimed by ticket by clusters that are actually running."""
    K, V, _ = orc.make_inputs(1, 8192, 8, dtype=torch.bfloat16, seed=71)
    Kc, Vc = K.cuda(), V.cuda()
    ref = ops._forward_sub_fwd(Kc, Vc, check=True)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = []
    for _ in range(3):
        with torch.cuda.stream(s1):
            outs.append(ops._forward_sub_fwd(Kc, Vc))
        with torch.cuda.stream(s2):
            outs.append(ops._forward_sub_fwd(Kc, Vc))
    with torch.cuda.stream(s1):
        a = ops._forward_sub_fwd(Kc, Vc, check=True)
    with torch.cuda.stream(s2):
        b = ops._forward_sub_fwd(Kc, Vc, check=True)
    torch.cuda.synchronize()
    assert all(torch.equal(o, ref) for o in outs) and torch.equal(a, ref) and torch.equal(b, ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_upper_dk_accumulated_by_the_reverse_solve(ops, dtype):
    """With more than two systems the reverse solve also accumulates the upper-triangle dK terms of the tiles it
    streams and the dK kernel runs the rest.  Against the plain pair of kernels (reverse solve, dK over all
    tiles): dV bit-identical (same products in the same order), dK equal to rounding (the same terms summed in
    two fp32 pieces), both within the gates of the oracle; T = 1, 2, 3 exercise the row-blocks without full tiles,
    and the last two shapes (32 systems of T = 4 and of T = 2) make every CTA take several such row-blocks in a row,
    the case in which the two issuing warps of the kernel are furthest apart."""
    from lucid_kernels_b200 import _cabi

    lib = _cabi.load()
    for B, N, H in ((1, 128, 3), (1, 256, 3), (1, 384, 3), (1, 1024, 3), (2, 2048, 8), (4, 512, 8), (2, 256, 16)):
        K, V, G = orc.make_inputs(B, N, H, dtype=dtype, seed=17)
        Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
        vp = ops._forward_sub_fwd(Kc, Vc, check=True)
        try:
            lib.lucid_set_upper_in_solve(0)
            dv0, dk0 = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
            lib.lucid_set_upper_in_solve(1)
            dv1, dk1 = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
            dv2, dk2 = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True)
        finally:
            lib.lucid_set_upper_in_solve(1)
        assert torch.equal(dv0, dv1), (B, N, H)
        assert torch.equal(dv1, dv2) and torch.equal(dk1, dk2), (B, N, H)
        assert float((dk1.float() - dk0.float()).norm() / dk0.float().norm()) < 3e-3, (B, N, H)
        rdv, rdk = orc.backward_blockwise(Kc.double(), vp.double(), Gc.double())
        assert orc.rel_err(dv1, rdv) < 0.01 and orc.rel_err(dk1, rdk) < 0.02, (B, N, H)


def _oracle_one_system(K, V, G, vp, dv, dk, s):
    """Errors of system s (index into the head dimension of (1, N, n, 128) tensors) against the fp64 block
    recurrence, evaluated on the GPU."""
    k1, v1, g1 = [t[:, :, s:s + 1].cuda().double() for t in (K, V, G)]
    rvp = orc.forward_sub_blockwise(k1, v1)
    e = [orc.rel_err(vp[:, :, s:s + 1], rvp)]
    if dv is not None:
        rdv, rdk = orc.backward_blockwise(k1, vp[:, :, s:s + 1].double(), g1)
        e += [orc.rel_err(dv[:, :, s:s + 1], rdv), orc.rel_err(dk[:, :, s:s + 1], rdk)]
    return e


def test_config_fwd_b1_n8192_h8_against_the_oracle(ops):
    """Forward-only configuration B=1, N=8192, H=8 (T = 64), with pairs of row-blocks (the default for this
    shape) and with single row-blocks: every system against the fp64 recurrence."""
    from lucid_kernels_b200 import _cabi

    lib = _cabi.load()
    K, V, _ = orc.make_inputs(1, 8192, 8, dtype=torch.bfloat16)
    Kc, Vc = K.cuda(), V.cuda()
    ref = orc.forward_sub_blockwise(Kc.double(), Vc.double())
    try:
        assert lib.lucid_query_pair_solve(1, 8192, 8) == 1
        vp_pair = ops._forward_sub_fwd(Kc, Vc, check=True)
        lib.lucid_set_pair_solve(0)
        assert lib.lucid_query_pair_solve(1, 8192, 8) == 0
        vp_single = ops._forward_sub_fwd(Kc, Vc, check=True)
    finally:
        lib.lucid_set_pair_limits(8, 0)
    for h in range(8):
        assert orc.rel_err(vp_pair[:, :, h], ref[:, :, h]) < 0.01, h
        assert orc.rel_err(vp_single[:, :, h], ref[:, :, h]) < 0.01, h


def test_benchmark_shape_b2_n32768_h8_against_the_oracle(ops):
    """The benchmarked configuration itself (B=2, N=32768, H=8: 16 systems, T = 256, scheduler groups of four,
    separate solve and dK launches): one system of every group against the fp64 recurrence on the GPU."""
    B, N, H = 2, 32768, 8
    K, V, G = orc.make_inputs(B, N, H, dtype=torch.bfloat16)
    Kc, Vc, Gc = K.cuda(), V.cuda(), G.cuda()
    vp = ops._forward_sub_fwd(Kc, Vc, check=True)
    dv, dk = ops._forward_sub_bwd(Kc, vp, Gc, use_combined_kernel=True, check=True, reuse_diag=True)
    for b, h in ((0, 0), (0, 5), (1, 2), (1, 7)):          # systems 0, 5, 10, 15: one of each group of four
        e = _oracle_one_system(K[b:b + 1], V[b:b + 1], G[b:b + 1], vp[b:b + 1], dv[b:b + 1], dk[b:b + 1], h)
        assert e[0] < 0.01 and e[1] < 0.01 and e[2] < 0.02, (b, h, e)


def test_config_fwd_b1_n131072_h8_against_the_oracle(ops):
    """Long-context forward B=1, N=131072, H=8 (T = 1024): one system against the fp64 recurrence on the GPU,
    and the instrumented call's timestamps describe every row-block."""
    K, V, _ = orc.make_inputs(1, 131072, 8, dtype=torch.bfloat16, hb_slice=(0, 8))
    Kc, Vc = K.cuda(), V.cuda()
    vp, ts = ops._forward_sub_fwd(Kc, Vc, instrument=True, check=True)
    assert ts.shape == (8, 1024, 8) and bool((ts[:, :, 2] > ts[:, :, 0]).all())
    e = _oracle_one_system(K, V, V, vp, None, None, 6)
    assert e[0] < 0.01, e


def test_tma_delivery_probe_reports_a_rate(ops):
    """The diagnostic that measures the operand-delivery ceiling: every SM reports a positive clock count and the
    rate lies in the range the SM's L2 port allows (a 64-byte port; 65.8 bytes per clock were measured, the clock
    of the port being a little above the SM's under load)."""
    from lucid_kernels_b200 import _cabi
    K = torch.randn(2, 8192, 8, 128, device="cuda").bfloat16()
    for slots in (1, 4):
        r = _cabi.tma_delivery_rate(K, slots=slots, boxes_per_sm=500)
        assert 2.0 < r["bytes_per_clk_per_sm"] < 80.0, r
        assert r["tb_per_s"] > 0.5, r
    with pytest.raises(_cabi.LucidKernelError):
        _cabi.tma_delivery_rate(K, slots=13)
