"""Generate golden vectors by executing the reference's own pure-torch functions on the CPU.

The reference package cannot be imported as a whole (its GPU kernels need the CuTe DSL and a Hopper
GPU, and one support module is missing), so the host-side functions that define the arithmetic are
extracted from the reference's source files by name with ``ast`` and executed unchanged:

  test_correctness.py            build_L, forward_sub_autograd
  forward_sub_interface.py       _compute_diag_inv, _compute_diag_inv_transpose,
                                 _add_diagonal_dk_correction, _backward_dk_reference
  bench_lucid_model.py           NaiveLUCIDSolve (forward only)

Usage (needs the reference checkout; run where it is mounted):
    python tests/golden/make_golden.py /path/to/reference

Outputs: tests/golden/*.npz.  Inputs are stored alongside the outputs, so the tests never need the
reference or this script's random generator.
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _extract(path, names):
    src = open(path).read()
    ns = {"torch": torch}
    try:
        tree = ast.parse(src)
    except SyntaxError:
        # bench_lucid_model.py does not parse as a whole (a dangling indented line near its top);
        # cut the wanted top-level definitions out by their text instead.
        tree = None
    if tree is not None:
        for node in tree.body:
            if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in names:
                code = compile(ast.Module(body=[node], type_ignores=[]), path, "exec")
                exec(code, ns)
    else:
        lines = src.splitlines(keepends=True)
        for name in names:
            start = next(i for i, l in enumerate(lines) if l.startswith(("class " + name, "def " + name)))
            end = start + 1
            while end < len(lines) and (lines[end].strip() == "" or lines[end][0] in " \t"):
                end += 1
            exec(compile("".join(lines[start:end]), path, "exec"), ns)
    missing = [n for n in names if n not in ns]
    assert not missing, missing
    return ns


def main(ref_root):
    tc = _extract(os.path.join(ref_root, "test_correctness.py"), ["build_L", "forward_sub_autograd"])
    itf = _extract(os.path.join(ref_root, "lucid_kernels/cute/forward_sub_interface.py"),
                   ["_compute_diag_inv", "_compute_diag_inv_transpose", "_add_diagonal_dk_correction",
                    "_backward_dk_reference"])
    mdl = _extract(os.path.join(ref_root, "bench_lucid_model.py"), ["NaiveLUCIDSolve"])

    cases = [
        # name, B, N, H, K scale, seed
        ("t2_b2h2_baseline", 2, 256, 2, 128 ** -0.25, 1),
        ("t3_b1h1_reftest", 1, 384, 1, 0.1, 2),
        ("t4_b1h2_baseline", 1, 512, 2, 128 ** -0.25, 3),
    ]
    for name, B, N, H, scale, seed in cases:
        torch.manual_seed(seed)
        # bf16-representable values so the same numbers can be fed to a 16-bit kernel unchanged
        K = (torch.randn(B, N, H, 128) * scale).bfloat16().double()
        V = torch.randn(B, N, H, 128).bfloat16().double()
        dVp = torch.randn(B, N, H, 128).bfloat16().double()

        Kg = K.clone().requires_grad_(True)
        Vg = V.clone().requires_grad_(True)
        Vp = tc["forward_sub_autograd"](Kg, Vg, 128)
        (Vp * dVp).sum().backward()
        L = tc["build_L"](K, 128)

        dinv = itf["_compute_diag_inv"](K.float(), 128)
        dinv_t = itf["_compute_diag_inv_transpose"](K.float(), 128)
        dk_ref = itf["_backward_dk_reference"](K.float(), Vp.detach().float(), Vg.grad.float(), 128)
        dk_diag = itf["_add_diagonal_dk_correction"](K.float(), Vp.detach().float(), Vg.grad.float(),
                                                    torch.zeros_like(K).float(), 128)

        class _Ctx:
            def save_for_backward(self, *a):
                pass

        naive = mdl["NaiveLUCIDSolve"].forward(_Ctx(), K.float(), V.float())

        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"),
            K=K.float().numpy(), V=V.float().numpy(), dVp=dVp.float().numpy(),
            Vp=Vp.detach().numpy(), dV=Vg.grad.numpy(), dK=Kg.grad.numpy(),
            L_checksum=np.array([float(L.sum()), float(L.abs().max()), float((L != 0).sum())]),
            L_row=L[0, 0, N - 1].numpy(),
            diag_inv=dinv.numpy(), diag_inv_t=dinv_t.numpy(),
            dK_reference_fp32=dk_ref.numpy(), dK_diag_only_fp32=dk_diag.numpy(),
            naive_fwd_fp32=naive.numpy(),
        )
        print(name, "Vp", float(Vp.norm()), "dV", float(Vg.grad.norm()), "dK", float(Kg.grad.norm()))

    # The benchmark's CPU configuration itself (B=1, N=512, H=4, fp32, seed 0): per-head norms and one
    # head's full result, to keep the fixture small.
    torch.manual_seed(0)
    B, N, H = 1, 512, 4
    K = torch.randn(B, N, H, 128) * 128 ** -0.25
    V = torch.randn(B, N, H, 128)
    dVp = torch.randn(B, N, H, 128)
    Kg = K.clone().requires_grad_(True)
    Vg = V.clone().requires_grad_(True)
    Vp = tc["forward_sub_autograd"](Kg, Vg, 128)
    (Vp * dVp).sum().backward()
    np.savez_compressed(
        os.path.join(HERE, "c1_fp32_seed0.npz"),
        K=K.numpy(), V=V.numpy(), dVp=dVp.numpy(),
        Vp_head0=Vp.detach()[:, :, 0].numpy(), dV_head0=Vg.grad[:, :, 0].numpy(), dK_head0=Kg.grad[:, :, 0].numpy(),
        Vp_head_norms=Vp.detach().permute(2, 0, 1, 3).reshape(H, -1).norm(dim=1).numpy(),
        dV_head_norms=Vg.grad.permute(2, 0, 1, 3).reshape(H, -1).norm(dim=1).numpy(),
        dK_head_norms=Kg.grad.permute(2, 0, 1, 3).reshape(H, -1).norm(dim=1).numpy(),
    )
    print("c1 done")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
