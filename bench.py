#!/usr/bin/env python3
"""Benchmark of the RNN-T loss hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3]
                    [--impl reference | reference-cuda]

One step = one forward + backward pass of the loss over one batch of the synthetic
workload (default "c3": B=32 per GPU, T=2000, U=100, V=10000, N(0,2) scores,
input_lengths in [1500,2000], label_lengths in [60,100]).  With N>1 (launched under
torch.distributed.run, one rank per GPU) every rank holds its own shard of the batch
(weak scaling) and the only exchange is an NCCL all-reduce of the scalar loss sum.

Rank 0 prints ONE JSON line.  `value` is utterances/s over all ranks with inputs
resident in HBM; `e2e` is the same through TransducerLoss with HOST (pinned) buffers,
host<->device copies inside the timed region; `roofline` describes the dominant
kernel; `cpu_baseline` is the reference's CPU path timed on this host on a bounded
sample.  `--impl reference` times only that CPU path; `--impl reference-cuda` times the
reference's own GPU path (its CUDA backend rebuilt unchanged for sm_100a) on the same
workload, for the speed-up over the GPU incumbent.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

A100_README_MS = 223.33  # B=32,T=2000,U=100,V=10000 on A100 (reference README.md:80)


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback (earlier measurement on this pool)"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the
    timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU path on host cores
# ----------------------------------------------------------------------------

def cpu_path_step(O, case, impl):
    E, P, labels, il, ll = case
    return O.loss_and_grads(E, P, labels, il, ll, blank=0, impl=impl)


def time_cpu_path(w, budget_s, steps, warmup):
    """Times fwd+bwd of the reference's CPU path (torch CPU ops + its OpenMP backend
    compiled from its own sources; the C restatement if that build is absent) on the
    first n utterances of workload `w`, n sized so one step fits `budget_s`."""
    from oracle import oracle as O
    from transducer_b200 import workloads
    impl = "reference" if O.have_reference() else "port"
    kind = "reference" if impl == "reference" else "port"
    # all the host cores this process may use, also under torch.distributed.run, which sets
    # OMP_NUM_THREADS=1 for its workers: torch's pool and the OpenMP runtime of the backend
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    try:
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    probe = [t.numpy() for t in workloads.generate(w, "cpu", first=0, count=1)]
    cpu_path_step(O, probe, impl)
    t0 = time.perf_counter()
    cpu_path_step(O, probe, impl)
    per_utt = time.perf_counter() - t0
    n = int(max(1, min(w.B, budget_s / max(per_utt, 1e-6))))
    case = [t.numpy() for t in workloads.generate(w, "cpu", first=0, count=n)]
    for _ in range(warmup):
        cpu_path_step(O, case, impl)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_path_step(O, case, impl)
    dt = (time.perf_counter() - t0) / steps
    return {"value": n / dt, "unit": "utterances/s", "cores": cores, "kind": kind,
            "sample": "first %d utterances of %s, %d timed pass(es), %.2f s/pass, torch %d threads + OpenMP"
                      % (n, w.name, steps, dt, cores),
            "ms_per_step": dt * 1e3, "n": n}


def run_reference_arm(args, w):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    steps = max(1, args.steps)
    budget = max(0.5, min(4.0, 150.0 / (steps + args.warmup)))
    r = time_cpu_path(w, budget, steps, args.warmup)
    line = {
        "impl": "reference",
        "metric": "rnnt_loss_fwd_bwd_utterances_per_s", "value": r["value"], "unit": "utterances/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(w, args.gpus, w.B),
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": "utterances/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_cuda_arm(args, w):
    """The reference's own GPU path on this GPU: its CUDA backend compiled unchanged for
    sm_100a plus the torch CUDA ops of its wrapper (transducer/torch_binding.py:25-90), the
    whole batch of `w`, forward + backward, timed with CUDA events on the default stream (where
    that backend launches).  Rank 0 only; a comparison line, not the product."""
    if env_int("RANK", 0) != 0:
        return
    from oracle import oracle as O
    from transducer_b200 import workloads
    if not O.have_reference_cuda():
        print(json.dumps({"impl": "reference-cuda",
                          "unavailable": "oracle/_ref/libref_transducer_cuda.so was not built"}))
        return
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference-cuda", "unavailable": "no CUDA device"}))
        return
    dev = torch.device("cuda", env_int("LOCAL_RANK", 0))
    torch.cuda.set_device(dev)
    B = args.batch if args.batch > 0 else w.B
    E, P, labels, il, ll = workloads.generate(w, dev, first=0, count=B)
    deltas = torch.ones(B, device=dev)
    steps = max(1, args.steps)

    def step():
        out = O.loss_and_grads_cuda(E, P, labels, il, ll, blank=w.blank, deltas=deltas)
        return out["costs"]

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        ev0.record()
        for _ in range(steps):
            costs = step()
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / steps
    line = {
        "impl": "reference-cuda",
        "metric": "rnnt_loss_fwd_bwd_utterances_per_s", "value": B / (ms * 1e-3),
        "unit": "utterances/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(w, 1, B),
        "clocks": clocks.summary(),
        "note": "reference CUDA backend (transducer_cuda.cu, unchanged, sm_100a) + torch CUDA ops "
                "of its wrapper; inputs resident in HBM; loss sum %.6g" % float(costs.sum()),
    }
    print(json.dumps(line), flush=True)


def workload_config(w, n_gpus, per_rank_batch):
    return {"workload": "%s: B=%d per GPU, T=%d, U=%d, V=%d, N(0,%g) fp32, ragged lengths %s/%s"
                        % (w.name, per_rank_batch, w.T, w.U, w.V, w.std, w.t_range, w.u_range),
            "per_gpu_batch": per_rank_batch, "global_batch": per_rank_batch * n_gpus,
            "T": w.T, "U": w.U, "V": w.V, "task": "loss fwd+bwd",
            "parallelism": "batch-sharded x%d, NCCL all-reduce of the loss sum" % n_gpus,
            "l2_policy": "inputs (%.2f GB per rank) larger than the 126 MB L2" %
                         (4.0 * per_rank_batch * w.T * w.V / 1e9)}


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--batch", type=int, default=0,
                    help="utterances per GPU instead of the workload's own batch (smaller cases "
                         "for profiler captures; the headline number is the default batch)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step eagerly instead of replaying a captured CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    from transducer_b200 import workloads
    w = workloads.CONFIGS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, w)
        return
    if args.impl == "reference-cuda":
        run_reference_cuda_arm(args, w)
        return

    from transducer_b200 import TransducerLoss, _lib
    import torch.distributed as dist

    rank, world = env_int("RANK", 0), env_int("WORLD_SIZE", 1)
    local_rank = env_int("LOCAL_RANK", 0)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=dev)

    B = args.batch if args.batch > 0 else w.B
    E, P, labels, il, ll = workloads.generate(w, dev, first=rank * B, count=B)
    deltas = torch.ones(B, device=dev)
    # lengths come from the workload generator and fit the padded shapes: skip the wrapper's
    # per-call read-back of their maxima (a host synchronisation; it also forbids graph capture)
    crit = TransducerLoss(blank=w.blank, validate_lengths=False)
    E.requires_grad_(True)
    P.requires_grad_(True)

    def local_step():
        """Forward + backward on this rank's shard; returns the shard's loss sum (device)."""
        E.grad = None
        P.grad = None
        costs = crit(E, P, labels, il, ll)
        costs.backward(deltas)
        return crit.last_loss_sum

    def step():
        loss_sum = local_step()
        if distributed:
            dist.all_reduce(loss_sum)   # the path's one collective: 4 bytes
        return loss_sum

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    # The local part of the step only enqueues kernels and memsets: capture it once in a CUDA
    # graph and replay it, which removes the host-side launch gaps between the kernels.  The NCCL
    # all-reduce stays outside the graph and is issued by every rank on every step, whether or
    # not its own capture succeeded, so ranks cannot end up waiting for each other.
    eager_step, graphed = step, False
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            n0 = _lib.lib.tb200_launch_count()
            with torch.cuda.graph(graph, stream=side):
                captured_sum = local_step()
            kernels_per_step = _lib.lib.tb200_launch_count() - n0  # kernel nodes of the graph
            torch.cuda.current_stream().wait_stream(side)

            def step():
                graph.replay()
                if distributed:
                    dist.all_reduce(captured_sum)
                return captured_sum
            graphed = True
        except Exception as exc:  # capture is an optimisation; the eager step is always valid
            print("bench.py: CUDA graph capture failed (%s); running eagerly" % exc, file=sys.stderr)
            step = eager_step
            torch.cuda.synchronize()
        # (the same calls on every rank, whichever way its capture went)
        for _ in range(2):
            step()
        barrier()

    # ---- timed region: K steps, device-timed, max over ranks -----------------------
    launches0 = _lib.lib.tb200_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
        # (a replayed graph launches its kernel nodes without passing the library's counter)
        launches = kernels_per_step * args.steps if graphed \
            else _lib.lib.tb200_launch_count() - launches0
        ms_total = ev0.elapsed_time(ev1)
        # Same K steps once more with every kernel bracketed by CUDA events on its stream (the
        # library's own accounting): per-kernel durations for the roofline.  Kept out of the
        # headline region because the event records themselves cost a few microseconds each.
        _lib.lib.tb200_profile_reset()
        _lib.lib.tb200_profile_enable(1)
        evp0, evp1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        evp0.record()
        for _ in range(args.steps):
            eager_step()   # (event records are not captured in the graph)
        evp1.record()
        barrier()
        _lib.lib.tb200_profile_enable(0)
        ms_profiled_step = evp0.elapsed_time(evp1) / args.steps
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if distributed:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = world * B / (ms_step * 1e-3)
    kernels = _lib.profile_report()
    loss_sum = float(step().item())
    barrier()

    # ---- roofline of the dominant kernel -------------------------------------------
    peaks = load_peaks()
    il_c, ll_c = il.cpu(), ll.cpu()
    alg = workloads.algorithmic_bytes(w, il_c, ll_c)
    per_kernel = {k: {"launches": n, "ms_per_launch": ms / n} for k, (n, ms) in kernels.items() if n}
    total_kernel_ms = sum(v["ms_per_launch"] * v["launches"] for v in per_kernel.values()) / args.steps
    top = max(per_kernel, key=lambda k: per_kernel[k]["ms_per_launch"] * per_kernel[k]["launches"]) \
        if per_kernel else None
    kernel_bytes = kernel_algorithmic_bytes(w, il_c, ll_c)
    roofline = None
    if top is not None:
        ab = kernel_bytes.get(top)
        ms = per_kernel[top]["ms_per_launch"]
        achieved = (ab / (ms * 1e-3) / 1e9) if ab else None
        roofline = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": (achieved / peaks["hbm_gbs"]) if achieved else None,
                    "traffic": NCU_TRAFFIC_BYTES.get((w.name, top)) if B == w.B else None,
                    "peak_source": peaks["source"], "ms_per_launch": ms,
                    "algorithmic_bytes_per_launch": ab}
    whole = {"algorithmic_bytes_per_step": alg["total"],
             "hbm_floor_ms": alg["total"] / (peaks["hbm_gbs"] * 1e9) * 1e3,
             "frac_of_hbm_roofline": alg["total"] / (peaks["hbm_gbs"] * 1e9) / (ms_step * 1e-3),
             "kernel_ms_per_step": total_kernel_ms,
             "ms_per_step_with_kernel_events": ms_profiled_step,
             "kernels": {k: round(v["ms_per_launch"] * v["launches"] / args.steps, 4)
                         for k, v in per_kernel.items()}}

    # ---- end to end with host buffers ------------------------------------------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(w, crit, (E, P, labels, il, ll), dev, distributed, world,
                      steps=max(2, min(args.steps, 5)))

    # ---- CPU baseline (rank 0, single-GPU run only) -----------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = time_cpu_path(w, budget_s=12.0, steps=1, warmup=0)
        cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {
            "metric": "rnnt_loss_fwd_bwd_utterances_per_s", "value": value, "unit": "utterances/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "fwd_bwd_ms": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (B / (ms_step * 1e-3)) / (32 / (A100_README_MS * 1e-3))
            if w.name == "c3" and B == w.B else None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(w, world, B),
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches),
            "cuda_graph": graphed, "roofline": roofline, "whole_step": whole, "cpu_baseline": cpu,
            "loss_sum": loss_sum,
        }
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of the
# named kernel; see the summaries under profiles/.  Keyed by (workload, kernel).
NCU_TRAFFIC_BYTES = {
    ("c3", "grads_umma"): 2466260480 + 2679300608,     # profiles/launch_list_bench_c3.md
    ("c3", "lognorm_umma"): 2625806848 + 14500608,
    ("c3", "alpha_warp"): 60119296 + 1955328,          # profiles/lattice_sweeps_c3.md
    ("c3", "gamma_warp"): 91227136 + 11807488,
    ("c3", "lattice_prep"): 532158720 + 43793664,
    ("c3", "expp_split"): 144711680 + 230021888,
    ("c3", "lattice_unskew_round"): 65938432 + 18867200,
}


def kernel_algorithmic_bytes(w, il, ll):
    """Bytes each kernel of the path must move per launch (fp32): E/P rows it reads,
    gradient rows it writes, lattice cells it touches."""
    sum_t = float(il.sum())
    sum_u = float((ll + 1).sum())
    sum_tu = float((il.double() * (ll.double() + 1)).sum())
    n = len(il)
    V = w.V
    return {
        "lognorm_exact": 4.0 * V * (sum_t + sum_u) + 4.0 * sum_tu,
        "lognorm_umma": 4.0 * V * (sum_t + sum_u) + 4.0 * sum_tu,
        "alpha_wavefront": 3 * 4.0 * sum_tu,
        "gamma_wavefront": 5 * 4.0 * sum_tu,
        "alpha_warp": 3 * 4.0 * sum_tu,    # arc terms (2 floats) in, alpha out
        "gamma_warp": 5 * 4.0 * sum_tu,    # arc terms + alpha in, stay + step out
        "egrad_simt": 4.0 * V * sum_t + 4.0 * V * n * w.T + 4.0 * V * sum_u,
        "pgrad_simt": 4.0 * V * sum_t + 4.0 * V * n * (w.U + 1) + 4.0 * V * sum_u,
        "grads_umma": 4.0 * V * (sum_t + sum_u) + 4.0 * V * n * (w.T + w.U + 1) + 4.0 * sum_tu,
        "row_max": 4.0 * V * sum_t,
        "exp_rows": 2 * 4.0 * V * sum_u,
    }


def run_e2e(w, crit, device_case, dev, distributed, world, steps):
    """fwd+bwd with HOST buffers through the library's host-buffer entry point
    (HostLossPipeline): every step copies this step's inputs from pinned host memory to the
    device and the costs and both gradients back, chunk by chunk, copies in both directions
    overlapping the kernels."""
    import torch.distributed as dist
    from transducer_b200 import HostLossPipeline
    E, P, labels, il, ll = device_case
    host = [t.detach().cpu().pin_memory() for t in (E, P, labels, il, ll)]
    B = E.shape[0]
    out_costs = torch.empty(B, dtype=torch.float32).pin_memory()
    out_eg = torch.empty(E.shape, dtype=torch.float32).pin_memory()
    out_pg = torch.empty(P.shape, dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in (out_costs, out_eg, out_pg))
    pipe = HostLossPipeline(blank=crit.blank, chunk=2, slots=4, device=dev)

    def step():
        loss_sum = pipe(*host, out_costs, out_eg, out_pg)
        if distributed:
            dist.all_reduce(loss_sum)
        return loss_sum

    step()
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
    if distributed:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / steps
    return {"value": world * B / (ms * 1e-3), "unit": "utterances/s", "ms_per_step": ms,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": steps,
            "api": "transducer_b200.HostLossPipeline(chunk=2, slots=4)"}


if __name__ == "__main__":
    main()
