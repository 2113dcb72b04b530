"""CPU-only checks: the C-ABI library loads and exports every declared symbol, argument validation,
status strings, sharding index maths, and a world-size-2 gloo run of the shard/gather logic."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from lucid_kernels_b200 import build, _cabi

    build.build()
    return _cabi.load()


def test_library_exports_every_declared_symbol(lib):
    hdr = open(os.path.join(ROOT, "include", "lucid_b200.h")).read()
    declared = set(re.findall(r"\b(lucid_[a-z_0-9]+)\s*\(", hdr))
    assert {"lucid_fwd_sub", "lucid_bwd_sub", "lucid_workspace_bytes", "lucid_read_status"} <= declared
    from lucid_kernels_b200 import _cabi

    assert declared == set(_cabi.EXPORTS)
    for name in declared:
        assert getattr(lib, name) is not None


def test_workspace_size_and_status_strings(lib):
    assert lib.lucid_workspace_bytes(1, 100, 1) == 0
    small = lib.lucid_workspace_bytes(1, 128, 1)
    big = lib.lucid_workspace_bytes(2, 32768, 8)
    # per 128 rows: one tile of inverses, flags and row scales (the forward's share), plus one fp32 tile of dK
    # partial sums for the combined backward
    assert 32768 + 65536 < small < 65536 + 65536
    assert 32768 < lib.lucid_fwd_workspace_bytes(1, 128, 1) < 40000
    assert lib.lucid_fwd_workspace_bytes(1, 100, 1) == 0
    assert 128 * 2 ** 20 < lib.lucid_fwd_workspace_bytes(2, 32768, 8) < 140 * 2 ** 20
    assert big - lib.lucid_fwd_workspace_bytes(2, 32768, 8) >= 256 * 2 ** 20
    assert big < 400 * 2 ** 20
    assert lib.lucid_status_string(0) == b"ok"
    assert b"128" in lib.lucid_status_string(-1)
    assert b"published" in lib.lucid_status_string(2)


def test_scheduler_group_sizes(lib):
    """The automatic group size (chain_group = 0): K and V' of a group at about the size of the L2 in the forward,
    104 MiB but at least four systems in the combined backward, groups of equal size, never more than there are
    systems.  The shapes are those the rule was measured on."""
    q = lib.lucid_query_chain_group
    assert q(1, 100, 1, 0) == 0                                   # invalid shape
    assert (q(2, 32768, 8, 0), q(2, 32768, 8, 1)) == (8, 6)       # the benchmark: 16 systems of N = 32768
    assert (q(1, 65536, 8, 0), q(1, 65536, 8, 1)) == (4, 4)
    assert (q(1, 131072, 8, 0), q(1, 131072, 8, 1)) == (2, 4)
    assert (q(1, 65536, 4, 0), q(1, 65536, 4, 1)) == (4, 4)
    assert (q(2, 16384, 8, 0), q(2, 16384, 8, 1)) == (16, 8)
    assert (q(1, 32768, 2, 0), q(1, 32768, 2, 1)) == (2, 2)       # the 8-GPU share: all of its systems
    assert (q(1, 8192, 8, 0), q(1, 8192, 8, 1)) == (8, 8)
    for B, N, H in ((3, 32768, 5), (1, 1 << 20, 3), (7, 128, 1)):
        for bwd in (0, 1):
            g = q(B, N, H, bwd)
            assert 1 <= g <= B * H


def test_argument_validation_without_gpu(lib):
    I3 = ctypes.c_int64 * 3
    st = I3(128 * 4 * 512, 128 * 4, 128)
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 1023) // 1024 * 1024
    args = lambda N, D, dt, k=p, ws=p, wsb=1 << 40: (k, p, p, st, st, st, 1, N, 4, D, dt, 1, 0, 0, ws, wsb, None)
    assert lib.lucid_fwd_sub(*args(500, 128, 1)) == -1      # N % 128
    assert lib.lucid_fwd_sub(*args(512, 64, 1)) == -1       # head_dim
    assert lib.lucid_fwd_sub(*args(512, 128, 7)) == -2      # dtype
    assert lib.lucid_fwd_sub(*args(512, 128, 1, k=p + 2)) == -3   # misaligned base
    assert lib.lucid_fwd_sub(*args(512, 128, 1, k=None)) == -5
    assert lib.lucid_fwd_sub(*args(512, 128, 1, wsb=16)) == -4
    bad = I3(128 * 4 * 512, 130, 128)
    assert lib.lucid_fwd_sub(p, p, p, bad, st, st, 1, 512, 4, 128, 1, 1, 0, 0, p, 1 << 40, None) == -3


def test_shard_ranges():
    from lucid_kernels_b200.sharding import all_ranges, shard_range, to_systems, from_systems, take_shard

    for n in (16, 8, 5, 1):
        for w in (1, 2, 4, 8):
            r = all_ranges(n, w)
            assert r[0][0] == 0 and r[-1][1] == n
            assert all(r[i][1] == r[i + 1][0] for i in range(w - 1))
            assert max(b - a for a, b in r) - min(b - a for a, b in r) <= 1
    x = torch.arange(2 * 256 * 4 * 128, dtype=torch.float32).reshape(2, 256, 4, 128)
    assert torch.equal(from_systems(to_systems(x), 2, 4), x)
    sh = take_shard(x, 4, 1)
    lo, hi = shard_range(8, 4, 1)
    assert sh.shape == (1, 256, hi - lo, 128)
    assert torch.equal(sh[0, :, 0], x[0, :, 2])     # system 2 = (b=0, h=2)


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from lucid_kernels_b200.sharding import take_shard, gather_shards, shard_range
from oracle import lucid_oracle as orc
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
B, N, H = 2, 256, 3
K, V, G = orc.make_inputs(B, N, H, dtype=torch.float64)
lo, hi = shard_range(B * H, world, rank)
Ks, Vs, Gs = orc.make_inputs(B, N, H, dtype=torch.float64, hb_slice=(lo, hi))
assert torch.equal(Ks, take_shard(K, world, rank))
# every rank solves only its own systems (the CPU oracle stands in for the kernels here) ...
vp_local = orc.forward_sub_blockwise(Ks, Vs)
dv_local, dk_local = orc.backward_blockwise(Ks, vp_local, Gs)
# ... and the gathered result equals the unsharded solve: no exchange is needed on the data path
vp = gather_shards(vp_local, B, H)
dk = gather_shards(dk_local, B, H)
ref_vp = orc.forward_sub_blockwise(K, V)
_, ref_dk = orc.backward_blockwise(K, ref_vp, G)
assert torch.allclose(vp, ref_vp, rtol=1e-12, atol=1e-14), float((vp - ref_vp).abs().max())
assert torch.allclose(dk, ref_dk, rtol=1e-10, atol=1e-12)
dist.destroy_process_group()
print("OK", rank)
"""


def test_two_rank_gloo_shard_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER % ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29531", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("OK") == 2


def test_interface_mirrors_reference_signatures():
    import inspect
    from lucid_kernels_b200 import cute

    sig = inspect.signature(cute._forward_sub_fwd)
    assert list(sig.parameters)[:7] == ["k", "v", "block_size", "window_size", "no_sync", "instrument",
                                        "use_diag_solve"]
    assert sig.parameters["use_diag_solve"].default is True
    sig = inspect.signature(cute._forward_sub_bwd)
    assert list(sig.parameters)[:6] == ["k", "v_prime", "dv_prime", "block_size", "use_diag_solve",
                                        "use_combined_kernel"]
    assert sig.parameters["use_combined_kernel"].default is False
    sig = inspect.signature(cute._forward_sub_bwd_dv)
    assert list(sig.parameters)[:5] == ["k", "dv_prime", "block_size", "use_diag_solve", "instrument"]
    sig = inspect.signature(cute._forward_sub_bwd_combined)
    assert list(sig.parameters)[:6] == ["k", "v_prime", "dv_prime", "block_size", "use_diag_solve", "instrument"]


def test_work_item_order_keeps_every_chain_in_step_order(tmp_path):
    """The solve kernels' ticket order (csrc/schedule.h), compiled for the host: every (chain, step) exactly
    once and each chain's steps in increasing order, for plain groups, a common head, overlapping groups,
    ragged groups and the clamped cases - the property that makes the flag waits deadlock-free."""
    import random
    import shutil
    import subprocess

    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "ticket_order")
    subprocess.run([gxx, "-O1", "-std=c++17", "-I", os.path.join(root, "lucid_kernels_b200", "csrc"), "-o", exe,
                    os.path.join(root, "tests", "host", "ticket_order.cpp")], check=True)
    cases = ["16,256,4,0,0", "16,256,4,0,96", "16,256,4,32,96", "16,256,4,200,28", "16,256,4,200,29",
             "8,1024,1,0,512", "8,64,2,5,32", "6,10,2,3,3", "5,10,2,2,3", "6,10,3,10,3", "1,7,1,0,3", "3,1,2,0,1",
             # pairs of row-blocks solved by clusters of two CTAs: tickets name (chain, pair) with T/2 pairs per
             # chain, no head and no overlap
             "8,32,8,0,0", "1,128,1,0,0", "2,128,2,0,0", "16,128,4,0,0", "3,1,3,0,0"]
    rng = random.Random(0)
    for _ in range(200):
        C, T = rng.randint(1, 12), rng.randint(1, 40)
        cases.append(f"{C},{T},{rng.randint(1, C)},{rng.randint(-1, T + 1)},{rng.randint(0, T)}")
    out = subprocess.run([exe, *cases], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout
    assert out.stdout.strip() == f"ok {len(cases)}"


def test_dk_work_items_cover_every_tile_and_balance_the_a_buffer(tmp_path):
    """The dK kernel's work items (csrc/schedule.h) on the host: whole and split items, both ticket orders,
    with and without diagonal tiles, T = 1..40: every tile once, the right operand in the A buffer, and as many
    loads as waits as frees of it (tests/host/dk_items.cpp)."""
    import shutil
    import subprocess

    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "dk_items")
    subprocess.run([gxx, "-O1", "-std=c++17", "-I", os.path.join(root, "lucid_kernels_b200", "csrc"), "-o", exe,
                    os.path.join(root, "tests", "host", "dk_items.cpp")], check=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout
    assert out.stdout.startswith("ok ")
