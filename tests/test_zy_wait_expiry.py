"""A device-side wait that runs out must end in an error status, not in a hang.

Every wait in the kernels (mbarrier or flag) has a time limit (`lucid_set_wait_limit_ns`, 2 s by default).
Here the limit is set to 0, which the kernels read as "do not wait": the first wait that is not satisfied at
once (the first tile load, at the latest) counts as expired, in every CTA.  The call must come back with a LucidKernelError that
names the kernel and the place, the GPU must stay usable, and a normal call on the same workspace afterwards
must give the right answer.  Nothing is made to fault: the kernels simply give up, wait out their copies in
flight, free their tensor memory and return.  The reference has no counterpart (its waits spin without limit,
forward_sub_fwd.py:541-544).

Collected late on purpose (file name), after the parity tests.
"""
import pytest
import torch

from oracle import lucid_oracle as orc

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_the_next_call_is_fine():
    from lucid_kernels_b200 import _cabi
    from lucid_kernels_b200._cabi import LucidKernelError
    from lucid_kernels_b200.cute import _forward_sub_fwd

    lib = _cabi.load()
    K, V, _ = orc.make_inputs(1, 8192, 1, dtype=torch.bfloat16, seed=81)
    Kc, Vc = K.cuda(), V.cuda()
    good = _forward_sub_fwd(Kc, Vc, check=True)
    torch.cuda.synchronize()
    try:
        lib.lucid_set_pair_solve(0)                   # the plain one-CTA-per-row-block path
        lib.lucid_set_wait_limit_ns(0)
        with pytest.raises(LucidKernelError) as err:
            _forward_sub_fwd(Kc, Vc, check=True)
    finally:
        lib.lucid_set_wait_limit_ns(2_000_000_000)
        lib.lucid_set_pair_limits(8, 0)
    msg = str(err.value)
    assert "timed out" in msg or "never published" in msg or "left early" in msg, msg
    assert "kernel=" in msg and "row_block=" in msg
    torch.cuda.synchronize()
    # same workspace, default limit: the status words are cleared by the call and the result is right again
    again = _forward_sub_fwd(Kc, Vc, check=True)
    assert torch.equal(again, good)
    assert orc.rel_err(again, orc.forward_sub_blockwise(K, V)) < 0.01
