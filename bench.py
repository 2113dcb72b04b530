#!/usr/bin/env python
"""Benchmark of the LUCID forward substitution + backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" = one forward solve (V') plus one backward pass (dV, dK) over the workload
B=2, N=32768, H=8, d=128, bf16 (use_diag_solve, combined backward), on synthetic seeded inputs
(K ~ N(0,1)*d^-1/4, V and dV' ~ N(0,1)).  With N > 1 ranks (torchrun, one process per GPU) the 16
independent (batch, head) systems are sharded over the ranks; there is no collective on the data path.

Prints ONE JSON line (rank 0).  `value` is whole-job algorithmic TFLOP/s with inputs resident in HBM;
`e2e` is the same metric through the operator interface with host buffers (pinned host -> device copies
of K, V, dV' and device -> host copies of V', dV, dK inside the timed region).

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
                    hbm_gbs=d["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


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
        sm, smax, reasons = [], [], set()
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
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------------------------------
# CPU path (reference arm and cpu_baseline leg)
# ------------------------------------------------------------------------------------------------
def cpu_naive_sample(budget_s: float = 15.0):
    """The reference's naive path (dense L + solve_triangular + autograd, fp32) on a bounded sample of
    the workload: B=1, N=4096, H=2 of the same value distribution.  Returns TFLOP/s and a description."""
    from oracle import lucid_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B, N, H = 1, 4096, 2
    K, V, dVp = orc.make_inputs(B, N, H, dtype=torch.float32)
    f, b = orc.algorithmic_flops(B, N, H)
    times = []
    t_begin = time.perf_counter()
    orc.naive_cpu_fwd_bwd(K, V, dVp)  # warm-up
    while len(times) < 3 or (time.perf_counter() - t_begin < budget_s and len(times) < 50):
        t0 = time.perf_counter()
        orc.naive_cpu_fwd_bwd(K, V, dVp)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > 2 * budget_s:
            break
    med = statistics.median(times)
    return dict(value=(f + b) / med / 1e12, unit=UNIT, cores=cores, kind="port",
                sample=f"dense L + solve_triangular + autograd fp32, B={B} N={N} H={H} (same distribution), "
                       f"median of {len(times)} runs, {med * 1e3:.0f} ms each"), med


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    cb, med = cpu_naive_sample(budget_s=max(5.0, 4.0 * (args.steps + args.warmup)))
    line = dict(impl="reference", metric=METRIC, value=cb["value"], unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=med * 1e3, higher_is_better=True, scaling="strong",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload="LUCID fwd+bwd B=2 N=32768 H=8 d=128 (bounded CPU sample, see cpu_baseline.sample)"),
                cpu_baseline=cb,
                e2e=dict(value=cb["value"], unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0, wall_s=time.perf_counter() - t0)
    print(json.dumps(line), flush=True)


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
                    help="launch every call of the timed region from Python also on several GPUs")
    ap.add_argument("--graphs", action="store_true", help="replay CUDA graphs in the timed region also on one GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    from oracle import lucid_oracle as orc  # input generator and the cpu_baseline leg only
    from lucid_kernels_b200 import _cabi
    from lucid_kernels_b200.cute import _forward_sub_fwd, _forward_sub_bwd
    from lucid_kernels_b200.sharding import shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.load()

    B, N, H, D = WORKLOAD["B"], args.seqlen, WORKLOAD["H"], WORKLOAD["D"]
    nsys = B * H if args.systems <= 0 else min(args.systems, B * H)
    lo, hi = shard_range(nsys, world, rank)
    n_local = hi - lo
    # each rank materialises only its own systems, as a (1, N, n_local, 128) BSHD tensor
    K, V, dVp = orc.make_inputs(B, N, H, dtype=torch.bfloat16, hb_slice=(lo, hi))
    Kh, Vh, Gh = K.pin_memory(), V.pin_memory(), dVp.pin_memory()
    # Two device copies of the inputs, used by alternate steps: every step then solves a k it has not seen in
    # the previous call, so the forward always recomputes the diagonal-block inverses (only the backward
    # of the same step reuses them, as it would in training).
    sets = [(Kh.to(dev), Vh.to(dev), Gh.to(dev)) for _ in range(2)]
    Kd, Vd, Gd = sets[0]
    f_fwd, f_rev, f_dk = flops_split(nsys, N)
    total_flops = f_fwd + f_rev + f_dk

    def step(i=0):
        kd, vd, gd = sets[i & 1]
        vp = _forward_sub_fwd(kd, vd, use_diag_solve=True)
        dv, dk = _forward_sub_bwd(kd, vp, gd, use_diag_solve=True, use_combined_kernel=True)
        return vp, dv, dk

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for w in range(args.warmup):
        step(w)
    barrier()

    # ---- timed region: K steps, CUDA events on the launching stream, per-kernel events inside ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    mk = lambda: torch.cuda.Event(enable_timing=True)

    def new_events():
        evs = [mk() for _ in range(7)]
        for e in evs:
            e.record()   # forces creation of the underlying handle
        return evs

    def profiled_step(e, which):
        kd, vd, gd = sets[which]
        lib.lucid_profile_next_call(e[0].cuda_event, e[1].cuda_event, e[2].cuda_event, None)
        vp = _forward_sub_fwd(kd, vd, use_diag_solve=True)
        lib.lucid_profile_next_call(e[3].cuda_event, e[4].cuda_event, e[5].cuda_event, e[6].cuda_event)
        dv, dk = _forward_sub_bwd(kd, vp, gd, use_diag_solve=True, use_combined_kernel=True)
        return vp, dv, dk

    # On several GPUs the step lasts only a few milliseconds and N ranks share the host's cores with their
    # clock samplers and with other tenants: there the timed region replays one CUDA graph per input set, a
    # whole step (two memsets, diagonal prep, the solves, dK) in ONE launch, so that a busy host cannot starve
    # the GPUs (measured on 8 GPUs: 3.4 to 6.0 ms per step for 2.9 ms of kernels when launched call by call).
    # Same kernels, same arguments, same order as the eager calls.  Events recorded inside a graph cannot be
    # read back, so the per-kernel times then come from eager steps run straight after the timed region; on one
    # GPU the timed region itself is eager and carries the per-kernel events.
    graphs, launch_mode, keep = None, "eager", []
    if (world > 1 or args.graphs) and not args.eager:
        try:
            graphs = []
            for which in range(2):
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    keep.append(step(which))
                graphs.append(g)
            for g in graphs:
                g.replay()
            torch.cuda.synchronize()
            launch_mode = "cuda_graph (one launch per step)"
        except Exception as exc:
            graphs, launch_mode = None, f"eager (graph capture failed: {str(exc)[:100]})"
            torch.cuda.synchronize()
    n_prof = args.steps if graphs is None else min(args.steps, 4)
    kern_ev = [new_events() for _ in range(n_prof)]
    barrier()
    ev0, ev1 = mk(), mk()
    t_wall0 = time.time()
    ev0.record()
    for s in range(args.steps):
        if graphs is not None:
            graphs[(args.warmup + s) & 1].replay()
        else:
            profiled_step(kern_ev[s], (args.warmup + s) & 1)
    ev1.record()
    if graphs is not None:
        for s in range(n_prof):                      # per-kernel times: eager steps on the still-loaded GPU
            profiled_step(kern_ev[s], (args.warmup + s) & 1)
    barrier()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1)
    ms_total = ev0.elapsed_time(ev1)
    # The SM clock as the kernels see it: one instrumented forward straight after the timed region (GPU
    # still at its loaded power state) records wall time and SM cycles per row-block; nvidia-smi's
    # instantaneous readings at 50 ms intervals catch idle moments of a sub-second region and read high.
    try:
        _, ts = _forward_sub_fwd(sets[0][0], sets[0][1], use_diag_solve=True, instrument=True)
        torch.cuda.synchronize()
        ts3 = ts.cpu().double()                      # (systems, T, 8): start, loop end, published, flag wait ns, ...
        ts = ts3.reshape(-1, 8)
        ns = ts[:, 2] - ts[:, 0]
        keep = ns > 100e3
        if int(keep.sum()) > 0:
            clocks["sm_mhz_in_kernel"] = float((ts[:, 6][keep] / ns[keep]).median() * 1e3)
        # The wavefront as measured: time between the publications of consecutive row-blocks of a chain
        # (its critical path is T such steps per solve) and the share of CTA time spent waiting for flags.
        pub = ts3[:, :, 2]
        step_ns = float((pub[:, 1:] - pub[:, :-1]).median()) if pub.shape[1] > 1 else 0.0
        wavefront = dict(chain_step_ns=step_ns, flag_wait_frac=float(ts[:, 3].sum() / ns.sum()))
    except Exception as exc:      # reporting only; never fails the benchmark
        clocks["sm_mhz_in_kernel"] = None
        clocks["sm_mhz_in_kernel_error"] = str(exc)[:80]
        wavefront = None
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    # per-kernel averages (this rank)
    n_ev = len(kern_ev)
    def avg(i, j):
        return sum(kern_ev[s][i].elapsed_time(kern_ev[s][j]) for s in range(n_ev)) / n_ev
    k_ms = dict(fwd_prep=avg(0, 1), fwd_solve=avg(1, 2), bwd_prep=avg(3, 4), bwd_solve=avg(4, 5), bwd_dk=avg(5, 6))
    for ws_ in list(_cabi._workspaces.values()):      # the eager calls' workspace and the graphs' one
        st = _cabi.read_status(ws_, torch.cuda.current_stream().cuda_stream)
        if st[0] != 0:
            raise SystemExit(f"device-side error during the timed region: {st}")

    # ---- e2e: host buffers in, host buffers out, through the operator interface ----
    e2e = None
    if not args.no_e2e:
        # Every step copies its K, V, dV' from pinned host memory and copies V', dV, dK back to pinned host
        # memory.  The copies run on their own streams and are double-buffered, so a step's uploads overlap
        # the previous step's kernels and its downloads overlap the following kernels (V' leaves while the
        # backward runs, dV while the dK kernel runs), the way a caller that feeds host data would drive it.
        outs_h = [torch.empty_like(Kh).pin_memory() for _ in range(3)]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        main = torch.cuda.current_stream(dev)
        dev_in = [[torch.empty_like(t, device=dev) for t in (Kh, Vh, Gh)] for _ in range(2)]
        in_ready = [mk() for _ in range(2)]
        in_free = [mk() for _ in range(2)]
        for e in in_free:
            e.record(main)

        def e2e_step(i):
            bi = i & 1
            kd, vd, gd = dev_in[bi]
            with torch.cuda.stream(s_in):
                s_in.wait_event(in_free[bi])          # the kernels of step i-2 are done with this buffer
                kd.copy_(Kh, non_blocking=True)
                vd.copy_(Vh, non_blocking=True)
                gd.copy_(Gh, non_blocking=True)
                in_ready[bi].record(s_in)
            main.wait_event(in_ready[bi])
            vp = _forward_sub_fwd(kd, vd, use_diag_solve=True)
            e_vp, e_dv, e_end = mk(), mk(), mk()
            e_vp.record(main)
            e_dv.record(main)                         # creates the handle; re-recorded after the reverse solve
            lib.lucid_profile_next_call(None, None, e_dv.cuda_event, None)
            dv, dk = _forward_sub_bwd(kd, vp, gd, use_diag_solve=True, use_combined_kernel=True)
            e_end.record(main)
            in_free[bi].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(e_vp)
                outs_h[0].copy_(vp, non_blocking=True)
                s_out.wait_event(e_dv)
                outs_h[1].copy_(dv, non_blocking=True)
                s_out.wait_event(e_end)
                outs_h[2].copy_(dk, non_blocking=True)
            for t in (vp, dv, dk):
                t.record_stream(s_out)

        for w in range(2):
            e2e_step(w)
        torch.cuda.synchronize()
        barrier()
        n_e2e = max(4, min(args.steps, 10))
        a, b_ = mk(), mk()
        a.record(main)
        for i in range(n_e2e):
            e2e_step(i)
        s_out.wait_stream(main)
        b_.record(s_out)
        torch.cuda.synchronize()
        barrier()
        te = torch.tensor([a.elapsed_time(b_)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e2e = float(te.item()) / n_e2e
        nbytes = Kh.numel() * Kh.element_size()
        e2e = dict(value=total_flops / (ms_e2e * 1e-3) / 1e12, unit=UNIT, ms_per_step=ms_e2e,
                   h2d_bytes_per_step=3 * nbytes, d2h_bytes_per_step=3 * nbytes, steps=n_e2e)

    if rank == 0:
        peaks = load_peaks()
        # dominant kernel = the dK kernel; roofline against the burst tensor peak
        f_dk_local = f_dk * n_local / nsys
        dk_tflops = f_dk_local / (k_ms["bwd_dk"] * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"]
        # DRAM bytes per dk_kernel launch: 254.9 MB measured by ncu at N=16384 with 16 systems (profiles/), equal to the
        # compulsory bytes (read K, V', dV; write dK), which scale with N and with the systems on this rank
        traffic = 254.9e6 * (N / 16384.0) * (n_local / 16.0)
        T_ = N // 128
        dk_exec = (T_ * (T_ + 1)) * 3 * G * n_local       # S, G and W*K for every ORDERED pair of row-blocks
        fused = k_ms["bwd_dk"] < 0.05 * k_ms["bwd_solve"]
        if fused:
            # one or two systems per GPU: the library ran the reverse solve and dK in ONE launch (timed here
            # as bwd_solve); the dominant kernel is then that launch, with the flops of both programs
            dom_kernel = "bwd_fused_kernel (reverse solve + dK in one launch)"
            t_dom = (k_ms["bwd_solve"] + k_ms["bwd_dk"]) * 1e-3
            f_dom = (f_dk + f_rev) * n_local / nsys
            exec_dom = dk_exec + f_rev * n_local / nsys
        else:
            dom_kernel, t_dom, f_dom, exec_dom = "dk_kernel", k_ms["bwd_dk"] * 1e-3, f_dk_local, dk_exec
        dk_tflops = f_dom / t_dom / 1e12
        roofline = dict(bound="tensor", kernel=dom_kernel, achieved=dk_tflops, peak=peak, unit="TFLOP/s",
                        frac=dk_tflops / peak, traffic=traffic, peak_source=peaks["source"] + " (sustained)",
                        per_kernel_ms=k_ms,
                        # The dK program forms W for every ordered pair (6 g per unordered pair, against the 3 g
                        # the algorithmic count allows), so the tensor pipe executes about twice `achieved`.
                        executed_tflops=exec_dom / t_dom / 1e12,
                        per_kernel_tflops=dict(
                            fwd_solve=f_fwd * n_local / nsys / (k_ms["fwd_solve"] * 1e-3) / 1e12,
                            bwd_solve=None if fused else f_rev * n_local / nsys / (k_ms["bwd_solve"] * 1e-3) / 1e12,
                            bwd_dk=None if fused else dk_tflops,
                            bwd_fused=dk_tflops if fused else None))
        # Bounds asked for by the metric: the tensor roofline of the algorithmic flops on this many GPUs and
        # the critical path of the two solves (2 * T chain steps at the step time of an unloaded chain, 3.3 us
        # measured on B200 with one chain per GPU); the fraction is taken against the tighter (larger) one.
        if wavefront is not None:
            tensor_ms = total_flops / (world * peaks["bf16_tflops"] * 1e12) * 1e3
            crit_ms = 2 * (N // 128) * 3.3e-3
            wavefront.update(tensor_bound_ms=tensor_ms, critical_path_bound_ms=crit_ms,
                             frac_of_tighter_bound=max(tensor_ms, crit_ms) / ms_step)
        line = dict(metric=METRIC, value=total_flops / (ms_step * 1e-3) / 1e12, unit=UNIT, n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
                    scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
                    config=dict(workload=f"LUCID fwd+bwd (V', dV, dK) B={B} N={N} H={H} d={D} bf16 BSHD, "
                                         "use_diag_solve, combined backward",
                                sharding=f"{nsys} (batch, head) systems over {world} rank(s), no collective",
                                l2="inputs (3 x 128 MiB per step at N=32768) exceed the 126 MB L2; no flush",
                                launch=launch_mode,
                                seed=0),
                    frac_of_bf16_peak=total_flops / (ms_step * 1e-3) / 1e12 / (world * peaks["bf16_tflops"]),
                    roofline=roofline, wavefront=wavefront, clocks=clocks, gpu_launches=(3 if fused else 4) * args.steps, e2e=e2e)
        if not args.no_cpu_baseline and world == 1:
            cb, _ = cpu_naive_sample()
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
