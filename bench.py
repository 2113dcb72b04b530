#!/usr/bin/env python
"""Benchmark of the LUCID forward substitution + backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" = one forward solve (V') plus one backward pass (dV, dK) over the workload
B=2, N=32768, H=8, d=128, bf16 (use_diag_solve, combined backward), on synthetic seeded inputs
(K ~ N(0,1)*d^-1/4, V and dV' ~ N(0,1)).  With N > 1 ranks (torchrun, one process per GPU) the 16
independent (batch, head) systems are sharded over the ranks; there is no collective on the data path.

Prints ONE JSON line (rank 0).  `value` is whole-job algorithmic TFLOP/s with inputs resident in HBM, the
timed region replaying one CUDA graph per step at every N; `e2e` is the same metric through the operator
interface with host buffers (pinned host -> device copies of K, V, dV' and device -> host copies of V', dV,
dK inside the timed region).  After the timed regions the outputs of the last step are compared with the
fp64 block recurrence evaluated on the GPU (`parity`), on several GPUs the shards are also all-gathered over
NCCL and checked against per-system checksums (`gathered_ok`), and the two forward-only configurations
(B=1, N=8192, H=8 and B=1, N=131072, H=8) are timed and checked (`configs`).

`--impl reference` times the reference's own naive CPU path (dense L + torch.linalg.solve_triangular +
autograd, fp32) on a bounded sample of the same workload, on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(B=2, N=32768, H=8, D=128)
METRIC = "lucid_fwd_bwd_tflops"
UNIT = "TFLOP/s"
G = 2.0 * 128 ** 3
GATES = dict(vp=0.01, dv=0.01, dk=0.02)       # relative Frobenius error against the fp64 recurrence


def flops_split(nsys: int, N: int):
    """Algorithmic flops of `nsys` systems: (forward, reverse solve, dK).  Per system and pair of
    blocks: forward 2g (S, P V'), reverse solve 2g (S, P dV), dK 3g (G, W K_j, W^T K_i); per diagonal block
    1.5g, 1.5g and 2g.  forward + reverse + dK = pairs*7g ... the backward total pairs*5g + T*3.5g counts the
    S product once: the reverse solve is charged 2g and dK 3g."""
    T = N // 128
    pairs = T * (T - 1) / 2
    fwd = nsys * (pairs * 2 * G + T * 1.5 * G)
    rev = nsys * (pairs * 2 * G + T * 1.5 * G)
    dk = nsys * (pairs * 3 * G + T * 2.0 * G)
    return fwd, rev, dk


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d["bf16_tflops_sustained"],
                    hbm_gbs=d["hbm_gbs"], sustained_sm_mhz=d.get("clocks_under_load", {}).get("sm_mhz_median"),
                    source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, sustained_sm_mhz=1300.0,
                source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
                 str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        # samples taken while the timed region ran; a region shorter than the sampling period falls back to
        # the samples around it (which include idle moments and read high)
        rows = ([l for (t, l) in self.lines if t0 + 0.02 <= t <= t1] or
                [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for _, l in self.lines])
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            try:
                power.append(float(f[3]))
            except ValueError:
                pass
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    power_w=statistics.median(power) if power else None, power_w_max=max(power) if power else None,
                    reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------------------------------
# CPU path (reference arm and cpu_baseline leg)
# ------------------------------------------------------------------------------------------------
def _time_cpu(fn, warmup: int, steps: int):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return times


def cpu_naive_sample(steps: int = 20, warmup: int = 2):
    """The reference's naive path (dense L + solve_triangular + autograd, fp32) on a bounded sample of
    the workload: B=1, N=4096, H=2 of the same value distribution, `steps` timed runs after `warmup`.
    Returns the cpu_baseline object (TFLOP/s of forward + backward) and the median seconds per run."""
    from oracle import lucid_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B, N, H = 1, 4096, 2
    K, V, dVp = orc.make_inputs(B, N, H, dtype=torch.float32)
    f, b = orc.algorithmic_flops(B, N, H)
    times = _time_cpu(lambda: orc.naive_cpu_fwd_bwd(K, V, dVp), warmup, steps)
    med = statistics.median(times)
    return dict(value=(f + b) / med / 1e12, unit=UNIT, cores=cores, kind="port",
                sample=f"dense L + solve_triangular + autograd fp32, B={B} N={N} H={H} (same distribution), "
                       f"median of {len(times)} runs after {warmup} warm-ups, {med * 1e3:.0f} ms each"), med


def cpu_named_cases(blockwise_budget_s: float = 12.0):
    """The two CPU cases the metric's plan names, beside the bounded sample above: (i) B=1, N=512, H=4
    fp32, seed 0, dense L + solve_triangular (+ autograd), forward and forward+backward, all cores;
    (ii) the blockwise naive forward (one 128 x 128 solve_triangular per block) on one system at the
    largest power-of-two N whose run stays within the budget."""
    from oracle import lucid_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    out = {}
    K, V, dVp = orc.make_inputs(1, 512, 4, dtype=torch.float32, seed=0)
    f, b = orc.algorithmic_flops(1, 512, 4)
    tf = _time_cpu(lambda: orc.forward_sub_dense(K, V), 3, 30)
    tfb = _time_cpu(lambda: orc.naive_cpu_fwd_bwd(K, V, dVp), 3, 30)
    mf, mfb = statistics.median(tf), statistics.median(tfb)
    out["c1_b1_n512_h4_fp32"] = dict(fwd_ms=mf * 1e3, fwd_bwd_ms=mfb * 1e3, fwd_tflops=f / mf / 1e12,
                                     fwd_bwd_tflops=(f + b) / mfb / 1e12, runs=30, cores=cores)
    N, last = 4096, None
    while N <= 32768:
        Kb, Vb, _ = orc.make_inputs(1, N, 1, dtype=torch.float32)
        t0 = time.perf_counter()
        orc.naive_cpu_fwd_blockwise(Kb, Vb)
        dt = time.perf_counter() - t0
        fN, _ = orc.algorithmic_flops(1, N, 1)
        last = dict(N=N, systems=1, fwd_ms=dt * 1e3, fwd_tflops=fN / dt / 1e12, runs=1, cores=cores)
        if dt * 4.2 > blockwise_budget_s:          # the next size costs about four times as much
            break
        N *= 2
    out["blockwise_naive_fwd_fp32"] = last
    return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    cb, med = cpu_naive_sample(steps=max(1, args.steps), warmup=max(0, args.warmup))
    line = dict(impl="reference", metric=METRIC, value=cb["value"], unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=med * 1e3, higher_is_better=True, scaling="strong",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload="LUCID fwd+bwd B=2 N=32768 H=8 d=128 (each step = one run of the bounded CPU "
                                     "sample, see cpu_baseline.sample)"),
                cpu_baseline=cb,
                e2e=dict(value=cb["value"], unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0, wall_s=time.perf_counter() - t0)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# helpers of the GPU arm
# ------------------------------------------------------------------------------------------------
def pin_to_gpu_numa_node(local_rank: int):
    """Run this process (and so first-touch its pinned host buffers) on the CPUs next to its GPU."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        txt = open(f"/sys/bus/pci/devices/{bdf}/local_cpulist").read().strip()
        cpus = set()
        for part in txt.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"{len(cpus)} CPUs local to {bdf}"
    except Exception as exc:
        return f"not set ({type(exc).__name__})"
    return "not set"


def oracle_errors(orc, K, V, Gd, vp, dv, dk, systems):
    """Worst relative Frobenius errors of the given local systems against the fp64 block recurrence, evaluated
    on the GPU on the same 16-bit input values; the backward is given the kernels' own V', as the autograd
    wrapper gives it.  Tensors are (1, N, n_local, 128)."""
    worst = dict(vp=0.0, dv=0.0, dk=0.0)
    for s in systems:
        k1, v1, g1 = [t[:, :, s:s + 1].double() for t in (K, V, Gd)]
        rvp = orc.forward_sub_blockwise(k1, v1)
        worst["vp"] = max(worst["vp"], orc.rel_err(vp[:, :, s:s + 1], rvp))
        if dv is not None:
            rdv, rdk = orc.backward_blockwise(k1, vp[:, :, s:s + 1].double(), g1)
            worst["dv"] = max(worst["dv"], orc.rel_err(dv[:, :, s:s + 1], rdv))
            worst["dk"] = max(worst["dk"], orc.rel_err(dk[:, :, s:s + 1], rdk))
        del k1, v1, g1, rvp
    return worst


def system_checksums(x):
    """Two integer checksums per system of a (1, N, n, 128) 16-bit tensor: the sum of the bit patterns and a
    position-weighted sum (so that a permutation of rows or systems shows).  Exact in int64."""
    bits = x.contiguous().view(torch.int16).to(torch.int64)               # (1, N, n, 128)
    w = (torch.arange(bits.shape[1], device=x.device, dtype=torch.int64) % 8191 + 1)[None, :, None, None]
    return torch.stack((bits.sum(dim=(0, 1, 3)), (bits * w).sum(dim=(0, 1, 3))), dim=1)   # (n, 2)


def wavefront_stats(ts, pair_mode: bool):
    """From the (systems, T, 8) timestamps of an instrumented forward: the time between the publications of
    consecutive row-blocks of a chain and the share of CTA time spent waiting for flags."""
    ts3 = ts.cpu().double()
    flat = ts3.reshape(-1, 8)
    ns = flat[:, 2] - flat[:, 0]
    out = dict(flag_wait_frac=float(flat[:, 3].sum() / ns.sum().clamp_min(1.0)))
    keep = ns > 100e3
    out["sm_mhz_in_kernel"] = float((flat[:, 6][keep] / ns[keep]).median() * 1e3) if int(keep.sum()) else None
    pub = ts3[:, :, 2]
    if pub.shape[1] > 1:
        d = pub[:, 1:] - pub[:, :-1]
        out["chain_step_ns"] = float(d.median())
        out["chain_step_mean_ns"] = float(d.mean())
        if pair_mode and pub.shape[1] > 2:
            out["in_pair_step_ns"] = float(d[:, 0::2].median())          # row-block 2p -> 2p+1 (inside a cluster)
            out["between_pairs_step_ns"] = float(d[:, 1::2].median())    # 2p+1 -> 2p+2 (through global memory)
        out["chain_span_ms"] = float((pub[:, -1] - pub[:, 0]).max()) * 1e-6
        # critical path of one solve: T - 1 hand-overs at the median step (per kind of hand-over in pair mode)
        Tn = pub.shape[1]
        if "in_pair_step_ns" in out:
            out["critical_path_one_solve_ms"] = ((Tn // 2) * out["in_pair_step_ns"] +
                                                 (Tn // 2 - 1) * out["between_pairs_step_ns"]) * 1e-6
        else:
            out["critical_path_one_solve_ms"] = (Tn - 1) * out["chain_step_ns"] * 1e-6
    else:
        out["chain_step_ns"] = out["chain_step_mean_ns"] = out["critical_path_one_solve_ms"] = 0.0
    return out


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--seqlen", type=int, default=WORKLOAD["N"], help="override N (parity/profiling runs only)")
    ap.add_argument("--systems", type=int, default=0,
                    help="use only the first K of the B*H (batch, head) systems (scaling studies only: "
                         "--gpus 1 --systems 2 is one rank's share of the 8-GPU run)")
    ap.add_argument("--eager", action="store_true",
                    help="launch every call of the timed region from Python instead of replaying CUDA graphs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison (profiling runs only)")
    ap.add_argument("--no-configs", action="store_true", help="skip the two forward-only configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    from oracle import lucid_oracle as orc  # input generator, the parity check and the cpu_baseline leg only
    from lucid_kernels_b200 import _cabi
    from lucid_kernels_b200.cute import _forward_sub_fwd, _forward_sub_bwd
    from lucid_kernels_b200.sharding import shard_range, gather_shards, to_systems

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # several ranks share one host: each stays (with its pinned buffers) on the CPUs next to its own GPU
    numa = pin_to_gpu_numa_node(local_rank) if world > 1 else "not set (one rank)"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.load()
    mk = lambda: torch.cuda.Event(enable_timing=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    B, N, H, D = WORKLOAD["B"], args.seqlen, WORKLOAD["H"], WORKLOAD["D"]
    nsys = B * H if args.systems <= 0 else min(args.systems, B * H)
    lo, hi = shard_range(nsys, world, rank)
    n_local = hi - lo
    # each rank materialises only its own systems, as a (1, N, n_local, 128) BSHD tensor
    K, V, dVp = orc.make_inputs(B, N, H, dtype=torch.bfloat16, hb_slice=(lo, hi))
    Kh, Vh, Gh = K.pin_memory(), V.pin_memory(), dVp.pin_memory()
    # Two device copies of the inputs, used by alternate steps: every step then solves a k it has not seen in
    # the previous call.  The forward always recomputes the diagonal-block inverses; the backward of the same
    # step, which is handed the very k tensor of its forward, asks to reuse them (reuse_diag=True), as the
    # autograd wrapper does in training.
    sets = [(Kh.to(dev), Vh.to(dev), Gh.to(dev)) for _ in range(2)]
    f_fwd, f_rev, f_dk = flops_split(nsys, N)
    total_flops = f_fwd + f_rev + f_dk

    def step(i=0):
        kd, vd, gd = sets[i & 1]
        vp = _forward_sub_fwd(kd, vd, use_diag_solve=True)
        dv, dk = _forward_sub_bwd(kd, vp, gd, use_diag_solve=True, use_combined_kernel=True, reuse_diag=True)
        return vp, dv, dk

    def profiled_step(e, which):
        kd, vd, gd = sets[which]
        lib.lucid_profile_next_call(e[0].cuda_event, e[1].cuda_event, e[2].cuda_event, None)
        vp = _forward_sub_fwd(kd, vd, use_diag_solve=True)
        lib.lucid_profile_next_call(e[3].cuda_event, e[4].cuda_event, e[5].cuda_event, e[6].cuda_event)
        dv, dk = _forward_sub_bwd(kd, vp, gd, use_diag_solve=True, use_combined_kernel=True, reuse_diag=True)
        return vp, dv, dk

    def new_events():
        evs = [mk() for _ in range(7)]
        for e in evs:
            e.record()   # forces creation of the underlying handle
        return evs

    for w in range(args.warmup):
        step(w)
    barrier()

    # ---- launch discipline: one CUDA graph per input set, a whole step (two memsets, diagonal prep, the
    # solves, dK) in ONE launch, at every number of GPUs.  On several GPUs the step lasts only a few
    # milliseconds and N ranks share the host's cores with their clock samplers: replaying keeps a busy host
    # from starving the GPUs; on one GPU it is used as well, so that the scaling curve compares like with like
    # (the eager figure is printed beside it).  Same kernels, same arguments, same order as the eager calls.
    graphs, launch_mode, keep_alive = None, "eager", []
    if not args.eager:
        try:
            graphs = []
            for which in range(2):
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    keep_alive.append(step(which))
                graphs.append(g)
            for g in graphs:
                g.replay()
            torch.cuda.synchronize()
            launch_mode = "cuda_graph (one launch per step)"
        except Exception as exc:
            graphs, launch_mode = None, f"eager (graph capture failed: {str(exc)[:100]})"
            torch.cuda.synchronize()

    # ---- timed region: K steps, CUDA events on the launching stream ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    barrier()
    ev0, ev1 = mk(), mk()
    t_wall0 = time.time()
    ev0.record()
    last = None
    for s in range(args.steps):
        if graphs is not None:
            graphs[(args.warmup + s) & 1].replay()
        else:
            last = step(args.warmup + s)
    ev1.record()
    barrier()
    t_wall1 = time.time()
    ms_step = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps

    # ---- the same steps launched call by call, carrying per-kernel events (GPU still at its loaded state) ----
    n_prof = max(2, min(args.steps, 10))
    kern_ev = [new_events() for _ in range(n_prof)]
    for s in range(2):            # untimed: `last` keeps one step's outputs alive, so the allocator needs a second set
        last = profiled_step(kern_ev[s], (args.warmup + s) & 1)
    barrier()
    ea, eb = mk(), mk()
    ea.record()
    for s in range(n_prof):
        last = profiled_step(kern_ev[s], (args.warmup + s) & 1)
    last_set = (args.warmup + n_prof - 1) & 1
    eb.record()
    barrier()
    clocks = sampler.stop(t_wall0, t_wall1)
    ms_eager = max_over_ranks(ea.elapsed_time(eb)) / n_prof

    def avg(i, j):
        return sum(kern_ev[s][i].elapsed_time(kern_ev[s][j]) for s in range(n_prof)) / n_prof
    k_ms = dict(fwd_prep=avg(0, 1), fwd_solve=avg(1, 2), bwd_prep=avg(3, 4), bwd_solve=avg(4, 5), bwd_dk=avg(5, 6))

    # ---- the wavefront as measured: one instrumented forward straight after the timed region ----
    T_ = N // 128
    pair_mode = bool(lib.lucid_query_pair_solve(1, N, n_local))
    try:
        _, ts = _forward_sub_fwd(sets[0][0], sets[0][1], use_diag_solve=True, instrument=True)
        torch.cuda.synchronize()
        wavefront = wavefront_stats(ts, pair_mode)
        clocks["sm_mhz_in_kernel"] = wavefront.pop("sm_mhz_in_kernel")
    except Exception as exc:      # reporting only; never fails the benchmark
        clocks["sm_mhz_in_kernel"] = None
        clocks["sm_mhz_in_kernel_error"] = str(exc)[:80]
        wavefront = None

    # ---- the operand-delivery ceiling as measured: TMA boxes of this run's K from L2 into every SM at once ----
    try:
        # on as many systems as one scheduler group of the solve holds (four at N = 32768: an L2-resident stream)
        delivery = _cabi.tma_delivery_rate(sets[0][0][:1, :, :4], slots=4, boxes_per_sm=4000)
    except Exception as exc:      # reporting only; never fails the benchmark
        delivery = dict(error=str(exc)[:80])

    def check_status():
        for ent in list(_cabi._workspaces.values()):      # the eager calls' workspace and the graphs' ones
            st = _cabi.read_status(ent.buf, torch.cuda.current_stream().cuda_stream)
            if st[0] != 0:
                raise SystemExit(f"device-side error: {st}")
    check_status()

    # ---- parity of what was just timed: the last step's outputs against the fp64 recurrence (on the GPU) ----
    parity = None
    if not args.no_parity:
        vp, dv, dk = last
        kd, vd, gd = sets[last_set]
        group = max(1, min(n_local, (72 << 20) // (N * 512))) if T_ >= 256 else n_local
        n_groups = -(-n_local // group)
        gsz = -(-n_local // n_groups)
        systems = sorted(set(range(0, n_local, gsz)))[:4]     # one system of every scheduler group
        t0 = time.perf_counter()
        worst = oracle_errors(orc, kd, vd, gd, vp, dv, dk, systems)
        torch.cuda.synchronize()
        worst = {k: max_over_ranks(v) for k, v in worst.items()}
        ok = all(worst[k] < GATES[k] and worst[k] == worst[k] for k in GATES)
        parity = dict(vp=worst["vp"], dv=worst["dv"], dk=worst["dk"], gates=GATES, ok=ok,
                      systems_checked=[lo + s for s in systems], systems_checked_per_rank=len(systems),
                      oracle="fp64 block recurrence + closed-form backward on the same bf16 inputs, on the GPU",
                      seconds=time.perf_counter() - t0)
        # graph replays write their own output buffers: those of the last replay must carry the same bits
        if graphs is not None:
            rep = keep_alive[last_set]
            parity["graph_outputs_bit_identical"] = bool(all(torch.equal(a, b) for a, b in zip(rep, last)))
        # several GPUs: reassemble the outputs with an NCCL all-gather and check every system's checksums
        # against those its owner computed from its shard
        if world > 1:
            names = ("vp", "dv", "dk")
            local_sums = torch.stack([system_checksums(t) for t in last], dim=0)          # (3, n_local, 2)
            width = max(b - a for a, b in [shard_range(nsys, world, r) for r in range(world)])
            padded = torch.zeros(3, width, 2, dtype=torch.int64, device=dev)
            padded[:, :n_local] = local_sums
            all_sums = [torch.empty_like(padded) for _ in range(world)]
            dist.all_gather(all_sums, padded)
            owner_sums = torch.cat([all_sums[r][:, : shard_range(nsys, world, r)[1] - shard_range(nsys, world, r)[0]]
                                    for r in range(world)], dim=1)                       # (3, nsys, 2)
            good = True
            Bf, Hf = (B, H) if nsys == B * H else (1, nsys)
            for ti, t in enumerate(last):
                full = gather_shards(t, Bf, Hf)                                          # (Bf, N, Hf, 128) via NCCL
                got = system_checksums(to_systems(full))
                good = good and bool(torch.equal(got, owner_sums[ti]))
                del full
            flag = torch.tensor([1 if good else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            parity["gathered_ok"] = bool(flag.item())
            parity["gathered"] = f"{', '.join(names)} all-gathered over NCCL ({world} ranks), {nsys} systems' checksums equal"
            parity["ok"] = parity["ok"] and parity["gathered_ok"]

    # ---- e2e: host buffers in, host buffers out, through the operator interface ----
    e2e = None
    if not args.no_e2e:
        # Every step copies its K, V, dV' from pinned host memory and copies V', dV, dK back to pinned host
        # memory.  The copies run on their own streams and are double-buffered, so a step's uploads overlap
        # the previous step's kernels and its downloads overlap the next step's kernels, the way a caller that
        # feeds host data would drive it.  The operator calls of a buffer set are captured once into a CUDA
        # graph and replayed, so a step costs the host one launch and six copies; events are created once,
        # not per step.
        outs_h = [torch.empty_like(Kh).pin_memory() for _ in range(3)]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        main_s = torch.cuda.current_stream(dev)
        dev_in = [[torch.empty_like(t, device=dev) for t in (Kh, Vh, Gh)] for _ in range(2)]
        ev = [dict(in_ready=mk(), in_free=mk(), end=mk(), out_done=mk()) for _ in range(2)]
        for e in ev:
            e["in_free"].record(main_s)
            e["out_done"].record(main_s)
        e2e_graphs, e2e_out = [None, None], [None, None]
        e2e_mode = "eager calls"
        if not args.eager:
            try:
                for bi in range(2):
                    kd, vd, gd = dev_in[bi]
                    kd.copy_(Kh); vd.copy_(Vh); gd.copy_(Gh)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, capture_error_mode="thread_local"):
                        vp_ = _forward_sub_fwd(kd, vd, use_diag_solve=True)
                        dv_, dk_ = _forward_sub_bwd(kd, vp_, gd, use_diag_solve=True, use_combined_kernel=True,
                                                    reuse_diag=True)
                    e2e_graphs[bi], e2e_out[bi] = g, (vp_, dv_, dk_)
                torch.cuda.synchronize()
                e2e_mode = "one CUDA graph per step for the operator calls, copies issued per step"
            except Exception as exc:
                e2e_graphs = [None, None]
                e2e_mode = f"eager calls (graph capture failed: {str(exc)[:80]})"
                torch.cuda.synchronize()

        def e2e_step(i, copies=True, kernels=True):
            bi = i & 1
            kd, vd, gd = dev_in[bi]
            e = ev[bi]
            if copies:
                with torch.cuda.stream(s_in):
                    s_in.wait_event(e["in_free"])           # the kernels of step i-2 are done with this buffer
                    kd.copy_(Kh, non_blocking=True)
                    vd.copy_(Vh, non_blocking=True)
                    gd.copy_(Gh, non_blocking=True)
                    e["in_ready"].record(s_in)
                main_s.wait_event(e["in_ready"])
            main_s.wait_event(e["out_done"])                # the downloads of step i-2 have read the outputs
            if kernels:
                if e2e_graphs[bi] is not None:
                    e2e_graphs[bi].replay()
                else:
                    vp = _forward_sub_fwd(kd, vd, use_diag_solve=True)
                    dv, dk = _forward_sub_bwd(kd, vp, gd, use_diag_solve=True, use_combined_kernel=True,
                                              reuse_diag=True)
                    e2e_out[bi] = (vp, dv, dk)
            vp, dv, dk = e2e_out[bi]
            e["end"].record(main_s)
            e["in_free"].record(main_s)
            if copies:
                # the downloads of this step overlap the kernels of the next one (which uses the other buffers)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(e["end"])
                    outs_h[0].copy_(vp, non_blocking=True)
                    outs_h[1].copy_(dv, non_blocking=True)
                    outs_h[2].copy_(dk, non_blocking=True)
                    e["out_done"].record(s_out)
                if e2e_graphs[bi] is None:
                    for t in (vp, dv, dk):
                        t.record_stream(s_out)

        def timed_e2e(n, **kw):
            for w in range(2):
                e2e_step(w, **kw)
            torch.cuda.synchronize()
            barrier()
            a, b_ = mk(), mk()
            a.record(main_s)
            for i in range(n):
                e2e_step(i, **kw)
            s_out.wait_stream(main_s)
            main_s.wait_stream(s_out)
            b_.record(main_s)
            torch.cuda.synchronize()
            barrier()
            return max_over_ranks(a.elapsed_time(b_)) / n

        n_e2e = max(4, min(args.steps, 10))
        ms_e2e = timed_e2e(n_e2e)
        nbytes = Kh.numel() * Kh.element_size()
        e2e = dict(value=total_flops / (ms_e2e * 1e-3) / 1e12, unit=UNIT, ms_per_step=ms_e2e,
                   h2d_bytes_per_step=3 * nbytes, d2h_bytes_per_step=3 * nbytes, steps=n_e2e, launch=e2e_mode,
                   host_affinity=numa)
        # where an end-to-end step goes: the same loop with only the copies, and with only the kernels
        e2e["breakdown_ms"] = dict(copies_only=timed_e2e(n_e2e, kernels=False), kernels_only=timed_e2e(n_e2e, copies=False),
                                   both=ms_e2e)
        # The timed region starts with an empty pipeline and ends when the last download has landed, so it holds
        # one upload and one download that nothing overlaps; the same loop over four times as many steps shows
        # how much of the per-step figure that is.
        e2e["ms_per_step_over_4x_steps"] = timed_e2e(4 * n_e2e)
        if not args.no_parity:
            torch.cuda.synchronize()
            e2e["host_outputs_equal_device_outputs"] = bool(
                all(torch.equal(h, d.cpu()) for h, d in zip(outs_h, e2e_out[(n_e2e - 1) & 1])))
        check_status()

    # ---- the two forward-only configurations, on this rank's share of their systems ----
    configs = None
    if not args.no_configs and args.systems <= 0 and N == WORKLOAD["N"]:
        configs = {}
        for name, (cB, cN, cH) in (("fwd_B1_N8192_H8", (1, 8192, 8)), ("fwd_B1_N131072_H8", (1, 131072, 8))):
            clo, chi = shard_range(cB * cH, world, rank)
            if chi <= clo:
                continue
            cK, cV, _ = orc.make_inputs(cB, cN, cH, dtype=torch.bfloat16, hb_slice=(clo, chi))
            cK, cV = cK.to(dev), cV.to(dev)
            for _ in range(3):
                out = _forward_sub_fwd(cK, cV, use_diag_solve=True)
            barrier()
            reps = 10 if cN <= 8192 else 3
            a, b_ = mk(), mk()
            a.record()
            for _ in range(reps):
                out = _forward_sub_fwd(cK, cV, use_diag_solve=True)
            b_.record()
            barrier()
            ms = max_over_ranks(a.elapsed_time(b_)) / reps
            cT = cN // 128
            c_pair = bool(lib.lucid_query_pair_solve(1, cN, chi - clo))
            _, cts = _forward_sub_fwd(cK, cV, use_diag_solve=True, instrument=True)
            torch.cuda.synchronize()
            wf = wavefront_stats(cts, c_pair)
            fl, _ = orc.algorithmic_flops(cB, cN, cH)
            entry = dict(ms=ms, tflops=fl / (ms * 1e-3) / 1e12, systems_per_rank=chi - clo, pair_mode=c_pair,
                         chain_step_ns=wf.get("chain_step_ns"), in_pair_step_ns=wf.get("in_pair_step_ns"),
                         between_pairs_step_ns=wf.get("between_pairs_step_ns"),
                         flag_wait_frac=wf["flag_wait_frac"], sm_mhz_in_kernel=wf["sm_mhz_in_kernel"],
                         critical_path_bound_ms=wf["critical_path_one_solve_ms"],
                         tensor_bound_ms=fl / (world * load_peaks()["bf16_tflops"] * 1e12) * 1e3)
            entry["frac_of_tighter_bound"] = max(entry["critical_path_bound_ms"], entry["tensor_bound_ms"]) / ms
            if not args.no_parity:
                e_ = oracle_errors(orc, cK, cV, cV, out, None, None, [0])
                entry["parity_vp"] = max_over_ranks(e_["vp"])
                entry["parity_ok"] = entry["parity_vp"] < GATES["vp"]
            configs[name] = entry
            del cK, cV, out
            torch.cuda.empty_cache()
        check_status()

    ok = True
    if rank == 0:
        peaks = load_peaks()
        # Roofline of the dominant kernel (the longest of the step) against the measured bf16 tensor peaks.
        # Algorithmic flops per kernel: forward solve and reverse solve 2g per pair of blocks + 1.5g per diagonal
        # block each; dK 3g per pair + 2g per diagonal block.  With more than two systems per GPU the reverse solve
        # also accumulates the upper-triangle dK terms (kernel revdk), and the dK kernel runs the lower part: each
        # of the two is then credited half of dK's pair flops.  Executed flops: 2g per pair in a solve, 3g per
        # ORDERED pair handled by the dK kernel, 2g more per pair in revdk.
        pairs_local = n_local * T_ * (T_ - 1) / 2
        diag_local = n_local * T_
        fused = k_ms["bwd_dk"] < 0.05 * k_ms["bwd_solve"]
        upper_in_solve = (not fused) and bool(lib.lucid_query_upper_in_solve(1, N, n_local))
        kern = {}
        kern["solve_kernel (forward)"] = dict(ms=k_ms["fwd_solve"], algo=pairs_local * 2 * G + diag_local * 1.5 * G,
                                              executed=pairs_local * 2 * G + diag_local * 3 * G)
        if fused:
            # one or two systems per GPU: the library ran the reverse solve and dK in ONE launch (timed as bwd_solve)
            kern["bwd_fused_kernel (reverse solve + dK in one launch)"] = dict(
                ms=k_ms["bwd_solve"] + k_ms["bwd_dk"], algo=pairs_local * 5 * G + diag_local * 3.5 * G,
                executed=pairs_local * 8 * G + diag_local * 9 * G)
        elif upper_in_solve:
            kern["revdk_kernel (reverse solve + upper-triangle dK)"] = dict(
                ms=k_ms["bwd_solve"], algo=pairs_local * 3.5 * G + diag_local * 1.5 * G,
                executed=pairs_local * 4 * G + diag_local * 3 * G)
            kern["dk_kernel (lower part, diagonal tiles, first upper tile)"] = dict(
                ms=k_ms["bwd_dk"], algo=pairs_local * 1.5 * G + diag_local * 2 * G,
                executed=pairs_local * 3 * G + diag_local * 9 * G)
        else:
            kern["solve_kernel (reverse)"] = dict(ms=k_ms["bwd_solve"], algo=pairs_local * 2 * G + diag_local * 1.5 * G,
                                                  executed=pairs_local * 2 * G + diag_local * 3 * G)
            kern["dk_kernel"] = dict(ms=k_ms["bwd_dk"], algo=pairs_local * 3 * G + diag_local * 2 * G,
                                     executed=pairs_local * 6 * G + diag_local * 6 * G)
        for v in kern.values():
            v["tflops"] = v["algo"] / (v["ms"] * 1e-3) / 1e12
            v["executed_tflops"] = v["executed"] / (v["ms"] * 1e-3) / 1e12
        # Operand bytes the kernels stream from L2 into shared memory: two 32 KiB tiles per tile of work (K_j and
        # Y_j / dV_j / V'_j) and three per row-block (its own K_i, X_i or A_i and right-hand side); the dK kernel
        # in its lower-part mode visits the lower tiles, the diagonal tile twice and one upper tile per row-block.
        tile_b = 32768.0
        for name, v in kern.items():
            tiles = pairs_local + (2 * diag_local if name.startswith("dk_kernel (lower") else
                                   pairs_local + diag_local if name.startswith("dk_kernel") else 0)
            v["operand_bytes"] = (2 * tiles + 3 * diag_local) * tile_b * (2 if name.startswith("bwd_fused") else 1)
            v["operand_tb_per_s"] = v["operand_bytes"] / (v["ms"] * 1e-3) / 1e12
            if delivery and "tb_per_s" in delivery:
                v["frac_of_delivery"] = v["operand_tb_per_s"] / delivery["tb_per_s"]
        dom_kernel = max(kern, key=lambda name: kern[name]["ms"])
        dom_tflops = kern[dom_kernel]["tflops"]
        # DRAM bytes per launch of the dominant kernel: its compulsory bytes (every ncu capture of these kernels
        # on L2-sized scheduler groups showed DRAM traffic within 10 % of them): tensors of n_local * N * 256 bytes
        tensor_bytes = n_local * N * 256.0
        traffic = tensor_bytes * (3 if dom_kernel.startswith("solve") else 4 if dom_kernel.startswith("dk_kernel") else 5)
        # The burst peak is the denominator unless the kernels ran at the clock of the sustained measurement
        mhz = clocks.get("sm_mhz_in_kernel")
        at_sustained = bool(mhz and peaks["sustained_sm_mhz"] and abs(mhz / peaks["sustained_sm_mhz"] - 1.0) < 0.05)
        peak = peaks["bf16_tflops_sustained"] if at_sustained else peaks["bf16_tflops"]
        roofline = dict(bound="tensor", kernel=dom_kernel, achieved=dom_tflops, peak=peak, unit="TFLOP/s",
                        frac=dom_tflops / peak, frac_burst=dom_tflops / peaks["bf16_tflops"],
                        frac_sustained=dom_tflops / peaks["bf16_tflops_sustained"], traffic=traffic,
                        peak_source=peaks["source"] + (" (sustained: kernels ran at its clock)" if at_sustained else " (burst)"),
                        per_kernel_ms=k_ms, executed_tflops=kern[dom_kernel]["executed_tflops"],
                        per_kernel={name: {k: v[k] for k in ("ms", "tflops", "executed_tflops", "operand_tb_per_s",
                                                             "frac_of_delivery") if k in v}
                                    for name, v in kern.items()},
                        delivery=dict(delivery or {}, what="TMA delivery of 16 KiB operand boxes from L2 into all SMs "
                                                           "at once, measured in this run (lucid_probe_tma_delivery): "
                                                           "the ceiling of per_kernel.operand_tb_per_s"))
        # Bounds asked for by the metric: the tensor roofline of the algorithmic flops on this many GPUs and
        # the critical path of the two solves - T - 1 hand-overs each at the median chain step measured in THIS
        # run by the instrumented forward (in pair mode the two kinds of hand-over separately); the fraction
        # is taken against the tighter (larger) one.
        if wavefront is not None:
            tensor_ms = total_flops / (world * peaks["bf16_tflops"] * 1e12) * 1e3
            crit_ms = 2 * wavefront["critical_path_one_solve_ms"]
            wavefront.update(pair_mode=pair_mode, tensor_bound_ms=tensor_ms, critical_path_bound_ms=crit_ms,
                             frac_of_tighter_bound=max(tensor_ms, crit_ms) / ms_step)
        value = total_flops / (ms_step * 1e-3) / 1e12
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
                    scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
                    config=dict(workload=f"LUCID fwd+bwd (V', dV, dK) B={B} N={N} H={H} d={D} bf16 BSHD, "
                                         "use_diag_solve, combined backward",
                                sharding=f"{nsys} (batch, head) systems over {world} rank(s), no collective",
                                l2="inputs (3 x 128 MiB per step at N=32768) exceed the 126 MB L2; no flush",
                                launch=launch_mode,
                                scheduler_groups=(f"{os.environ['LUCID_B200_CHAIN_GROUP']} systems per group (set by "
                                                  "LUCID_B200_CHAIN_GROUP)"
                                                  if os.environ.get("LUCID_B200_CHAIN_GROUP", "0") not in ("", "0") else
                                                  f"{lib.lucid_query_chain_group(1, N, n_local, 0)} systems per group in "
                                                  f"the forward solve, {lib.lucid_query_chain_group(1, N, n_local, 1)} in "
                                                  "the backward (on rank 0)"),
                                seed=0),
                    frac_of_bf16_peak=value / (world * peaks["bf16_tflops"]),
                    eager=dict(ms_per_step=ms_eager, value=total_flops / (ms_eager * 1e-3) / 1e12, steps=n_prof,
                               note="the same steps launched call by call straight after the timed region"),
                    roofline=roofline, wavefront=wavefront, clocks=clocks,
                    gpu_launches=(3 if fused else 4) * args.steps, parity=parity, e2e=e2e, configs=configs)
        if not args.no_cpu_baseline and world == 1:
            cb, _ = cpu_naive_sample()
            cb["named_cases"] = cpu_named_cases()
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
        ok = parity is None or parity["ok"]
        if configs:
            ok = ok and all(c.get("parity_ok", True) for c in configs.values())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed (see the `parity` / `configs` objects of the JSON line)")


if __name__ == "__main__":
    main()
