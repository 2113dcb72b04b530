"""Operand-delivery ceiling of the GPU this runs on: ``python -m lucid_kernels_b200.delivery_probe``.

Prints, for rings of 1 to 12 stages and for 4 and 16 systems of the benchmark shape (N = 32768, 128 columns,
bf16), how fast TMA brings 16 KiB operand boxes from L2 into the shared memory of all SMs at once
(``lucid_probe_tma_delivery``).  The solve and dK kernels stream 64 KiB of such boxes per tile of work, so
their time per tile cannot fall below 65536 / (bytes per clock per SM) clocks, whatever they compute.
"""
from __future__ import annotations

import json
import sys

import torch

from . import _cabi


def sweep(n: int = 32768, boxes_per_sm: int = 4000) -> list:
    rows = []
    for systems in (4, 16):
        b, h = (1, 4) if systems == 4 else (2, 8)
        k = torch.randn(b, n, h, 128, device="cuda").bfloat16()
        for slots in (1, 2, 4, 8, 12):
            r = _cabi.tma_delivery_rate(k, slots=slots, boxes_per_sm=boxes_per_sm)
            r.update(systems=systems, clocks_per_64KiB=65536.0 / r["bytes_per_clk_per_sm"])
            rows.append(r)
        del k
    return rows


def main() -> int:
    if not torch.cuda.is_available():
        print("no CUDA device", file=sys.stderr)
        return 1
    for r in sweep():
        print(json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
