"""Build the CUDA library in-tree: ``python -m lucid_kernels_b200.build``.

Compiles every ``csrc/*.cu`` for sm_100a with nvcc and links ``lucid_kernels_b200/_lucid_b200.so``.
nvcc cross-compiles without a GPU, so this runs on a build machine and the resulting ``.so`` is what
the GPU machine loads.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "_lucid_b200.so")
SOURCES = ["api.cu", "solve.cu", "diag_prep.cu", "dk.cu", "bwd_fused.cu", "rev_dk.cu", "probe.cu"]
# sources that textually include other sources
INCLUDES = {"bwd_fused.cu": ["solve.cu", "dk.cu"]}
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "lucid_b200.h"))
    return max(os.path.getmtime(d) for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    hdr_time = _newest_header()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        dep_time = max([os.path.getmtime(s), hdr_time] +
                       [os.path.getmtime(os.path.join(CSRC, d)) for d in INCLUDES.get(src, [])])
        if force or not os.path.exists(o) or os.path.getmtime(o) < dep_time:
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        r = subprocess.run([nvcc, *NVCC_FLAGS, "-c", s, "-o", o], capture_output=True, text=True)
        log = r.stdout + r.stderr
        with open(o[:-2] + ".ptxas.log", "w") as f:
            f.write(log)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{log}")
        return log

    with ThreadPoolExecutor(max_workers=4) as ex:
        for log in ex.map(compile_one, jobs):
            if verbose:
                print(log)
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in SOURCES]
    if jobs or not os.path.exists(LIB) or os.path.getmtime(LIB) < max(os.path.getmtime(o) for o in objs):
        r = subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
