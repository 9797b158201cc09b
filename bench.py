#!/usr/bin/env python3
"""Benchmark of the RNN-T loss / Viterbi hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3]
                    [--impl reference | reference-cuda]

One step = one pass of the workload's task over one batch of synthetic input
(transducer_b200.workloads.CONFIGS):

    c3 (default)     loss forward + backward, B=32 per GPU, T=2000, U=100, V=10000, N(0,2)
                     scores, ragged lengths -- the configuration the headline metric is quoted on
    c2_v100 .. c2_v10000   loss forward + backward, B=8 per GPU, T=2000, U=100, full lengths
    c4               loss forward only, B=256 IN ALL (sharded over the ranks: strong scaling),
                     T=1000, U=200, V=32000, peaky emissions
    c5               Viterbi decode, B=64 per GPU, T=1500, U=150, V=4096
    c1               the small plumbing case

With N>1 (launched under torch.distributed.run, one rank per GPU) every rank holds its own
shard and the only exchange is an NCCL all-reduce of the scalar loss sum, issued on a side
stream so that it overlaps the next step's kernels.

Rank 0 prints ONE JSON line.  `value` is utterances/s over all ranks with inputs resident in
HBM; `e2e` is the same through the library's host-buffer API with HOST (pinned) buffers,
host<->device copies inside the timed region; `roofline` describes the dominant kernel;
`cpu_baseline` is the reference's CPU path timed on this host on a bounded sample; `parity`
compares this run's GPU outputs with that CPU path on the same utterances.
`--impl reference` times only that CPU path; `--impl reference-cuda` times the reference's own
GPU path (its CUDA backend rebuilt unchanged for sm_100a) on the same workload.
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

import numpy as np  # noqa: E402
import torch  # noqa: E402

# fwd+bwd milliseconds the reference publishes for these shapes (A100, its README.md:68-71,80):
# workload -> (batch, ms)
PUBLISHED_MS = {"c3": (32, 223.33), "c2_v100": (8, 8.18), "c2_v1000": (8, 13.64),
                "c2_v2000": (8, 18.83), "c2_v10000": (8, 59.18)}

METRICS = {"loss": "rnnt_loss_fwd_bwd_utterances_per_s",
           "loss_fwd": "rnnt_loss_fwd_utterances_per_s",
           "viterbi": "rnnt_viterbi_utterances_per_s"}
TASK_TEXT = {"loss": "loss fwd+bwd", "loss_fwd": "loss fwd only", "viterbi": "viterbi decode"}


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

def cpu_path_step(O, w, case, impl):
    """One pass of workload `w`'s task through the reference's CPU path."""
    E, P, labels, il, ll = case
    if w.task == "viterbi":
        return {"labels": O.viterbi(E, P, il, ll, blank=w.blank, impl=impl)}
    return O.loss_and_grads(E, P, labels, il, ll, blank=w.blank, impl=impl,
                            want_grads=(w.task == "loss"))


def time_cpu_path(w, budget_s, steps, warmup, keep_outputs=False, source=None):
    """Times the task of `w` on the reference's CPU path (torch CPU ops + its OpenMP backend
    compiled from its own sources; the C restatement if that build is absent) on the first n
    utterances of the workload, n sized so one step fits `budget_s` (and at most 32, the
    chunk in which the 32-bit offsets of the reference still hold at every configuration).
    `source`: device tensors of a batch of `w` whose leading utterances are to be used (so that
    the CPU outputs can be compared with the GPU's on the very same inputs; the device's random
    generator does not produce the host generator's numbers); default: generated on the host."""
    from oracle import oracle as O
    from transducer_b200 import workloads
    impl = "reference" if O.have_reference() else "port"
    # all the host cores this process may use, also under torch.distributed.run, which sets
    # OMP_NUM_THREADS=1 for its workers: torch's pool and the OpenMP runtime of the backend
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    try:
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    def take(count):
        if source is not None:
            return [(t[:count].detach().float() if t.is_floating_point() else t[:count].detach())
                    .cpu().numpy() for t in source]
        return [t.numpy() for t in workloads.generate(w, "cpu", first=0, count=count)]

    probe = take(1)
    cpu_path_step(O, w, probe, impl)
    t0 = time.perf_counter()
    cpu_path_step(O, w, probe, impl)
    per_utt = time.perf_counter() - t0
    limit = w.B if source is None else int(source[0].shape[0])
    n = int(max(1, min(limit, 32, budget_s / max(per_utt, 1e-6))))
    case = take(n)
    out = None
    for _ in range(warmup):
        out = cpu_path_step(O, w, case, impl)
    t0 = time.perf_counter()
    for _ in range(steps):
        out = cpu_path_step(O, w, case, impl)
    dt = (time.perf_counter() - t0) / steps
    r = {"value": n / dt, "unit": "utterances/s", "cores": cores, "kind": impl,
         "sample": "first %d utterances of %s (%s), %d warm-up + %d timed pass(es), %.2f s/pass, "
                   "torch %d threads + OpenMP" % (n, w.name, TASK_TEXT[w.task], warmup, steps, dt, cores),
         "ms_per_step": dt * 1e3, "n": n}
    if keep_outputs:
        r["outputs"], r["case"] = out, case
    return r


def run_reference_arm(args, w):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    steps = max(1, args.steps)
    budget = max(0.5, min(4.0, 150.0 / (steps + args.warmup)))
    r = time_cpu_path(w, budget, steps, args.warmup)
    per_rank = per_rank_batch(w, args.gpus, 0, args.batch)
    line = {
        "impl": "reference",
        "metric": METRICS[w.task], "value": r["value"], "unit": "utterances/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": scaling_of(w), "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(w, args.gpus, per_rank),
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": "utterances/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_reference_cuda(w, dev, B, steps, warmup):
    """The reference's own GPU path on this GPU: its CUDA backend compiled unchanged for
    sm_100a plus the torch CUDA ops of its wrapper (transducer/torch_binding.py:25-90 and
    :130-177), timed with CUDA events on the default stream (where that backend launches)."""
    from oracle import oracle as O
    from transducer_b200 import workloads
    E, P, labels, il, ll = workloads.generate(w, dev, first=0, count=B)
    deltas = torch.ones(B, device=dev)

    def step():
        if w.task == "viterbi":
            return O.viterbi_cuda(E, P, il, ll, blank=w.blank).float()
        out = O.loss_and_grads_cuda(E, P, labels, il, ll, blank=w.blank, deltas=deltas,
                                    want_grads=(w.task == "loss"))
        return out["costs"]

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(torch.cuda.default_stream(dev))
    for _ in range(steps):
        res = step()
    ev1.record(torch.cuda.default_stream(dev))
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / steps, float(res.sum())


def run_reference_cuda_arm(args, w):
    """Rank 0 only; a comparison line, not the product."""
    if env_int("RANK", 0) != 0:
        return
    from oracle import oracle as O
    if not O.have_reference_cuda():
        print(json.dumps({"impl": "reference-cuda",
                          "unavailable": "oracle/_ref/libref_transducer_cuda.so was not built"}))
        return
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference-cuda", "unavailable": "no CUDA device"}))
        return
    dev = torch.device("cuda", env_int("LOCAL_RANK", 0))
    torch.cuda.set_device(dev)
    # (its 32-bit offsets hold up to 2^31 emission elements: c4 is cut to 64 utterances)
    B = args.batch if args.batch > 0 else min(w.B, (2 ** 31 - 1) // (w.T * w.V))
    steps = max(1, args.steps)
    with ClockSampler(dev.index) as clocks:
        ms, checksum = time_reference_cuda(w, dev, B, steps, max(args.warmup, 3))
    line = {
        "impl": "reference-cuda",
        "metric": METRICS[w.task], "value": B / (ms * 1e-3),
        "unit": "utterances/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": scaling_of(w), "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(w, 1, B),
        "clocks": clocks.summary(),
        "note": "reference CUDA backend (transducer_cuda.cu, unchanged, sm_100a) + torch CUDA ops "
                "of its wrapper; inputs resident in HBM; checksum %.6g" % checksum,
    }
    print(json.dumps(line), flush=True)


def scaling_of(w):
    return "strong" if w.task == "loss_fwd" else "weak"


def per_rank_batch(w, world, rank, override=0):
    """Utterances of rank `rank`.  c4 (loss_fwd) is ONE batch of w.B utterances split over the
    ranks (strong scaling); the other workloads give every rank its own w.B (weak scaling)."""
    from transducer_b200 import distributed as D
    if override > 0:
        return override
    if scaling_of(w) == "strong":
        return D.shard_range(w.B, rank, world)[1]
    return w.B


def workload_config(w, n_gpus, per_rank, reduce="nccl"):
    strong = scaling_of(w) == "strong"
    return {"workload": "%s: %s, B=%d %s, T=%d, U=%d, V=%d, N(0,%g) fp32, lengths %s/%s%s%s"
                        % (w.name, TASK_TEXT[w.task], w.B if strong else per_rank,
                           "in all" if strong else "per GPU", w.T, w.U, w.V, w.std,
                           w.t_range or "full", w.u_range or "full",
                           ", %g%% of entries per frame +%g" % (100 * w.peaky, w.boost) if w.peaky else "",
                           ", blank column +%g" % w.blank_bias if w.blank_bias else ""),
            "per_gpu_batch": per_rank, "global_batch": w.B if strong else per_rank * n_gpus,
            "T": w.T, "U": w.U, "V": w.V, "task": TASK_TEXT[w.task],
            "parallelism": ("batch-sharded x%d, " % n_gpus +
                            ("NCCL all-reduce of the loss sum" if reduce == "nccl" else
                             "loss sums exchanged by peer stores (tb200_loss_sum_exchange)"))
                           if w.task != "viterbi" else "batch-sharded x%d, no exchange" % n_gpus,
            "l2_policy": "inputs (%.2f GB per rank) larger than the 126 MB L2" %
                         (4.0 * per_rank * w.T * w.V / 1e9)}


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
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"],
                    help="storage type of emissions, predictions and gradients (loss tasks; "
                         "the arithmetic is fp32 either way)")
    ap.add_argument("--reduce", default="nccl", choices=["nccl", "peer"],
                    help="how the ranks' loss sums are added: an NCCL all-reduce, or the library's "
                         "own exchange by peer stores (transducer_b200.distributed.PeerLossSum)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-incumbent", action="store_true",
                    help="skip timing the reference's CUDA backend beside the c3 run")
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
    from transducer_b200 import distributed as D
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

    B = per_rank_batch(w, world, rank, args.batch)
    if scaling_of(w) == "strong" and args.batch <= 0:
        first = D.shard_range(w.B, rank, world)[0]
    else:
        first = rank * B
    global_B = w.B if (scaling_of(w) == "strong" and args.batch <= 0) else world * B
    E, P, labels, il, ll = workloads.generate(w, dev, first=first, count=B)
    bf16 = args.dtype == "bf16"
    if bf16:
        if w.task == "viterbi":
            raise SystemExit("bench.py: --dtype bf16 applies to the loss tasks")
        E, P = E.to(torch.bfloat16), P.to(torch.bfloat16)
    elem_bytes = 2 if bf16 else 4
    deltas = torch.ones(B, device=dev)
    # lengths come from the workload generator and fit the padded shapes: skip the wrapper's
    # per-call read-back of their maxima (a host synchronisation; it also forbids graph capture)
    crit = TransducerLoss(blank=w.blank, validate_lengths=False)
    if w.task == "loss":
        E.requires_grad_(True)
        P.requires_grad_(True)
    has_loss = w.task != "viterbi"
    state = {}

    def local_step():
        """This rank's shard through the task; returns the shard's loss sum (device), or the
        decoded labels for the Viterbi task."""
        if w.task == "viterbi":
            state["labels"] = crit.viterbi(E, P, il, ll)
            return state["labels"]
        if w.task == "loss":
            E.grad = None
            P.grad = None
            costs = crit(E, P, labels, il, ll)
            costs.backward(deltas)
        else:
            with torch.no_grad():
                costs = crit(E, P, labels, il, ll)
        state["costs"] = costs.detach()   # (a reference to `costs` would keep its autograd graph alive)
        return crit.last_loss_sum

    # The path's one collective (4 bytes) runs on a side stream: the main stream copies the loss
    # sum into a slot of its own and goes on with the next step, the side stream reduces the slot.
    side = torch.cuda.Stream(device=dev) if distributed and has_loss else None
    reduced = torch.zeros(1, device=dev)
    peer_sum = D.PeerLossSum(device=dev) if side is not None and args.reduce == "peer" else None

    def reduce_async(loss_sum):
        if side is None:
            return loss_sum
        main = torch.cuda.current_stream()
        main.wait_stream(side)          # the slot is free again (previous reduction done)
        reduced.copy_(loss_sum)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            if peer_sum is not None:
                return peer_sum(reduced)
            dist.all_reduce(reduced)
        return reduced

    def step():
        return reduce_async(local_step())

    def barrier():
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
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
    eager_step, graphed, kernels_per_step = step, False, 0
    if not args.no_graph:
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            n0 = _lib.lib.tb200_launch_count()
            with torch.cuda.graph(graph, stream=cap):
                captured = local_step()
            kernels_per_step = _lib.lib.tb200_launch_count() - n0  # kernel nodes of the graph
            torch.cuda.current_stream().wait_stream(cap)

            def step():
                graph.replay()
                return reduce_async(captured)
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
            result = step()
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)   # the last reduction is part of the job
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
    _lib.check(_lib.lib.tb200_check_status())   # no kernel gave up on a bounded wait
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if distributed:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = global_B / (ms_step * 1e-3)
    kernels = _lib.profile_report()
    if has_loss:
        checksum = float(result.sum().item())
    else:   # sum of the decoded labels (entries past label_lengths are unspecified padding)
        live = torch.arange(w.U, device=dev)[None, :] < ll[:, None]
        checksum = int((result.long() * live).sum().item())
    barrier()

    # ---- what a drop-in user gets: TransducerLoss() as the reference is called -------------
    # (length validation on, no graph, a synchronisation per iteration as in
    # benchmarks/torch_benchmarks.py:8-20)
    saved_crit, crit = crit, TransducerLoss(blank=w.blank)   # (local_step uses `crit`)
    try:
        for _ in range(2):
            local_step()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_eager = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(n_eager):
            local_step()
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        eager_ms = e0.elapsed_time(e1) / n_eager
    finally:
        crit = saved_crit
    barrier()

    # ---- roofline of the dominant kernel -------------------------------------------
    peaks = load_peaks()
    il_c, ll_c = il.cpu(), ll.cpu()
    alg = workloads.algorithmic_bytes(w, il_c, ll_c, elem_bytes)
    alg_step = {"loss": alg["total"], "loss_fwd": alg["fwd"],
                "viterbi": viterbi_algorithmic_bytes(w, il_c, ll_c)}[w.task]
    per_kernel = {k: {"launches": n, "ms_per_launch": ms / n} for k, (n, ms) in kernels.items() if n}
    total_kernel_ms = sum(v["ms_per_launch"] * v["launches"] for v in per_kernel.values()) / args.steps
    top = max(per_kernel, key=lambda k: per_kernel[k]["ms_per_launch"] * per_kernel[k]["launches"]) \
        if per_kernel else None
    kernel_bytes = kernel_algorithmic_bytes(w, il_c, ll_c, elem_bytes)
    roofline = None
    clk = clocks.summary()
    if top is not None:
        ab = kernel_bytes.get(top)
        ms = per_kernel[top]["ms_per_launch"]
        achieved = (ab / (ms * 1e-3) / 1e9) if ab else None
        roofline = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": (achieved / peaks["hbm_gbs"]) if achieved else None,
                    "traffic": NCU_TRAFFIC_BYTES.get((w.name, top)) if B == w.B and not bf16 else None,
                    "peak_source": peaks["source"], "ms_per_launch": ms,
                    "algorithmic_bytes_per_launch": ab}
        if top.startswith("maxplus"):
            # (max,+) has no tensor-core form: the full loop is bound by fp32 issue, one add and
            # one max per (t,u,v).  Peak: 128 fp32 lanes per SM per clock at the sampled SM clock.
            # The figure covers all maxplus_* kernels of a step (lists, evaluation, leftovers).
            lane_ops = 2.0 * w.V * float((il_c.double() * ll_c.double()).sum())
            mhz = clk.get("sm_mhz") or 1965.0
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            peak_ops = sms * 128 * mhz * 1e6
            group_ms = sum(v["ms_per_launch"] for k, v in per_kernel.items() if k.startswith("maxplus"))
            pruned = top != "maxplus"
            roofline["simt_issue"] = {
                "lane_ops_full_loop": lane_ops, "ms_all_maxplus_kernels": group_ms,
                "achieved_per_s": lane_ops / (group_ms * 1e-3), "peak_per_s": peak_ops,
                "frac": lane_ops / (group_ms * 1e-3) / peak_ops,
                "note": ("operations of the reference's full loop over the alphabet; the list "
                         "evaluation skips most of them with an exact bound, so this is a "
                         "speed-up over the issue bound of the full loop, not a utilisation"
                         if pruned else
                         "binding unit of this kernel; the HBM figure above is reported beside "
                         "it, not as its bound")}
    whole = {"algorithmic_bytes_per_step": alg_step,
             "hbm_floor_ms": alg_step / (peaks["hbm_gbs"] * 1e9) * 1e3,
             "frac_of_hbm_roofline": alg_step / (peaks["hbm_gbs"] * 1e9) / (ms_step * 1e-3),
             "kernel_ms_per_step": total_kernel_ms,
             "ms_per_step_with_kernel_events": ms_profiled_step,
             "kernels": {k: round(v["ms_per_launch"] * v["launches"] / args.steps, 4)
                         for k, v in per_kernel.items()}}

    # ---- end to end with host buffers ------------------------------------------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(w, crit, (E, P, labels, il, ll), dev, distributed, world, global_B,
                      steps=max(2, min(args.steps, 5)))

    # ---- CPU baseline + parity against it (rank 0, single-GPU run only) -------------------
    cpu, parity = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = time_cpu_path(w, budget_s=12.0, steps=1, warmup=1, keep_outputs=True,
                          source=(E, P, labels, il, ll))
        cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        parity = parity_block(w, r, (E, P, labels, il, ll), state)

    # ---- the GPU incumbent beside the headline (reference CUDA backend, same GPU) ----------
    incumbent = None
    if rank == 0 and world == 1 and not args.no_incumbent and w.name == "c3" and args.batch <= 0:
        try:
            from oracle import oracle as O
            if O.have_reference_cuda():
                torch.cuda.empty_cache()
                ms_inc, _ = time_reference_cuda(w, dev, w.B, steps=3, warmup=3)
                incumbent = {"impl": "reference-cuda", "ms_per_step": ms_inc,
                             "what": "reference transducer_cuda.cu rebuilt unchanged for sm_100a + "
                                     "the torch CUDA ops of its wrapper, same batch, inputs resident"}
        except Exception as exc:
            incumbent = {"impl": "reference-cuda", "unavailable": str(exc)[:200]}

    if rank == 0:
        line = {
            "metric": METRICS[w.task], "value": value, "unit": "utterances/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": scaling_of(w),
            "vs_baseline": value / (PUBLISHED_MS[w.name][0] / (PUBLISHED_MS[w.name][1] * 1e-3))
            if w.name in PUBLISHED_MS and B == w.B and not bf16 else None,
            "dtype": "f32 arithmetic on bf16 storage (emissions, predictions, gradients)" if bf16 else "f32",
            "data": "synthetic", "config": workload_config(w, world, B, args.reduce),
            "clocks": clk, "e2e": e2e, "gpu_launches": int(launches),
            "cuda_graph": graphed, "eager_ms_per_step": eager_ms, "roofline": roofline,
            "whole_step": whole, "cpu_baseline": cpu, "parity": parity, "incumbent": incumbent,
            "checksum": checksum,
        }
        if w.task == "loss":
            line["fwd_bwd_ms"] = ms_step
        print(json.dumps(line), flush=True)
    if distributed:
        if peer_sum is not None:
            peer_sum.close()
        dist.destroy_process_group()


def parity_block(w, r, device_case, state):
    """This run's GPU outputs against the CPU path's outputs on the utterances the CPU
    baseline was timed on (the first r['n'] of the batch).  Outside every timed region."""
    from oracle import oracle as O
    E, P, labels, il, ll = device_case
    n, want = r["n"], r["outputs"]
    out = {"utterances": n, "oracle": r["kind"]}
    if w.task == "viterbi":
        got = state["labels"][:n].cpu().numpy()
        lens = ll[:n].cpu().numpy()
        bad = sum(0 if np.array_equal(got[b, :lens[b]], want["labels"][b, :lens[b]]) else 1
                  for b in range(n))
        out.update({"label_mismatches": int(bad), "bar": "bit-exact"})
        return out
    costs = state["costs"][:n].detach().cpu().numpy().astype(np.float64)
    wc = want["costs"].astype(np.float64)
    fin = np.isfinite(wc)
    out["loss_rel_max"] = float((np.abs(costs[fin] - wc[fin]) / np.maximum(np.abs(wc[fin]), 1e-30)).max())
    out["bar_loss"] = 1e-4
    if w.task == "loss":
        def rel(got, ref):
            d, m = 0.0, 0.0
            for b in range(n):
                x = torch.from_numpy(np.ascontiguousarray(ref[b])).to(got.device).double()
                d = max(d, float((got[b].double() - x).abs().max()))
                m = max(m, float(x.abs().max()))
            return d / max(m, 1e-30)
        out["egrad_rel_to_max"] = rel(E.grad, want["egrads"])
        out["pgrad_rel_to_max"] = rel(P.grad, want["pgrads"])
        out["bar"] = 1e-3
        if E.dtype is torch.bfloat16:
            out["bar"] = 2.0 ** -8 + 1e-3
            out["note"] = ("reference run on the up-converted inputs; a bf16 gradient carries 8 "
                           "significant bits: the bar is the fp32 bar plus one rounding (2^-8) of "
                           "the maximum")
        # the oracle's own distance to a float64 evaluation of the same formulas (its fp32 noise
        # floor), and this run's distance to it, over the same utterances (0.2 s each, untimed)
        floor = {"egrad": 0.0, "pgrad": 0.0}
        ours = {"egrad": 0.0, "pgrad": 0.0}
        for b in range(n):
            c = [a[b:b + 1] for a in r["case"]]
            truth = O.truth64(c[0], c[1], c[2], c[3], c[4], blank=w.blank)
            for key, grad, ref in (("egrad", E.grad, "egrads"), ("pgrad", P.grad, "pgrads")):
                den = np.abs(truth[ref]).max()
                floor[key] = max(floor[key], float(np.abs(want[ref][b:b + 1] - truth[ref]).max() / den))
                got = grad[b:b + 1].detach().float().cpu().numpy().astype(np.float64)
                ours[key] = max(ours[key], float(np.abs(got - truth[ref]).max() / den))
        out["oracle_vs_fp64_floor"] = floor
        out["ours_vs_fp64"] = ours
    return out


# dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of the named
# kernel on this workload (1-pass captures at the bench size).  Keyed by (workload, kernel).
NCU_TRAFFIC_BYTES = {
    ("c3", "grads_umma"): 2460688896 + 2661452288,
    ("c3", "lognorm_umma"): 2626279936 + 35040256,
    ("c3", "alpha_warp"): 60133120 + 2445056,
    ("c3", "gamma_warp"): 91231744 + 11596032,
    ("c3", "lattice_prep"): 42460416 + 7390976,
    ("c3", "expp_split"): 146920704 + 230604288,
    ("c3", "lattice_unskew_round"): 65933568 + 19291904,
}


def viterbi_algorithmic_bytes(w, il, ll):
    """Viterbi decode: E and P read once (shared by the log-normaliser and the max-plus pass),
    three lattices written and read (log-normalisers, best label scores, packed records)."""
    sum_t = float(il.sum())
    sum_u = float((ll + 1).sum())
    sum_tu = float((il.double() * (ll.double() + 1)).sum())
    return 4.0 * w.V * (sum_t + sum_u) + 6 * 4.0 * sum_tu


def kernel_algorithmic_bytes(w, il, ll, elem_bytes=4):
    """Bytes each kernel of the path must move per launch: E/P rows it reads and gradient rows
    it writes (elem_bytes per element), lattice cells it touches (fp32)."""
    eb = float(elem_bytes)
    sum_t = float(il.sum())
    sum_u = float((ll + 1).sum())
    sum_tu = float((il.double() * (ll.double() + 1)).sum())
    n = len(il)
    V = w.V
    return {
        "lognorm_exact": 4.0 * V * (sum_t + sum_u) + 4.0 * sum_tu,
        "lognorm_umma": eb * V * (sum_t + sum_u) + 4.0 * sum_tu,
        "maxplus": 4.0 * V * (sum_t + sum_u) + 4.0 * sum_tu,
        "maxplus_pruned": 4.0 * V * sum_t + 4.0 * sum_tu,    # E rows in, scores out
        "maxplus_select_e": 4.0 * V * sum_t,
        "alpha_wavefront": 3 * 4.0 * sum_tu,
        "gamma_wavefront": 5 * 4.0 * sum_tu,
        "alpha_warp": 3 * 4.0 * sum_tu,    # arc terms (2 floats) in, alpha out
        "gamma_warp": 5 * 4.0 * sum_tu,    # arc terms + alpha in, stay + step out
        "viterbi_warp": 4 * 4.0 * sum_tu,  # one float4 record per node in
        "egrad_simt": 4.0 * V * sum_t + 4.0 * V * n * w.T + 4.0 * V * sum_u,
        "pgrad_simt": 4.0 * V * sum_t + 4.0 * V * n * (w.U + 1) + 4.0 * V * sum_u,
        "grads_umma": eb * V * (sum_t + sum_u) + eb * V * n * (w.T + w.U + 1) + 4.0 * sum_tu,
        "row_max": 4.0 * V * sum_t,
        "exp_rows": 2 * 4.0 * V * sum_u,
    }


def run_e2e(w, crit, device_case, dev, distributed, world, global_B, steps):
    """The task with HOST buffers: every step copies this step's inputs from pinned host memory
    to the device and the results back (costs and both gradients; costs; labels), chunk by
    chunk, copies in both directions overlapping the kernels (HostLossPipeline for the loss
    tasks, the same slot scheme around criterion.viterbi for decoding).  A rank whose shard
    would need more than 8 GB of pinned memory runs it on a leading part of the shard; the
    figure then extrapolates by utterances (the chunks are independent)."""
    import torch.distributed as dist
    from transducer_b200 import HostLossPipeline
    E, P, labels, il, ll = device_case
    B = E.shape[0]
    per_utt = float(E.element_size()) * (E[0].numel() + P[0].numel()) * (2 if w.task == "loss" else 1)
    n = int(max(1, min(B, 8e9 // per_utt)))
    host = [t[:n].detach().cpu().pin_memory() for t in (E, P, labels, il, ll)]
    out_costs = torch.empty(n, dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host)
    if w.task == "loss":
        out_eg = torch.empty(host[0].shape, dtype=E.dtype).pin_memory()
        out_pg = torch.empty(host[1].shape, dtype=E.dtype).pin_memory()
        d2h = sum(t.numel() * t.element_size() for t in (out_costs, out_eg, out_pg))
        pipe = HostLossPipeline(blank=crit.blank, chunk=2, slots=4, device=dev, valid_rows_only=True)
        api = "transducer_b200.HostLossPipeline(chunk=2, slots=4, valid_rows_only=True)"
        valid = host[3].clamp(max=w.T).double()
        valid_u = (host[4] + 1).clamp(max=w.U + 1).double()
        moved = float(valid.sum()) * w.V * host[0].element_size() + \
            float(valid_u.sum()) * w.V * host[1].element_size()
        h2d = moved + sum(t.numel() * t.element_size() for t in host[2:])
        d2h = moved + out_costs.numel() * 4

        def local():
            return pipe(*host, out_costs, out_eg, out_pg)
    elif w.task == "loss_fwd":
        d2h = out_costs.numel() * 4
        pipe = HostLossPipeline(blank=crit.blank, chunk=4, slots=3, device=dev, forward_only=True,
                                valid_rows_only=True)
        api = "transducer_b200.HostLossPipeline(chunk=4, slots=3, forward_only=True, valid_rows_only=True)"
        valid = host[3].clamp(max=w.T).double()
        valid_u = (host[4] + 1).clamp(max=w.U + 1).double()
        h2d = float(valid.sum()) * w.V * host[0].element_size() + \
            float(valid_u.sum()) * w.V * host[1].element_size() + \
            sum(t.numel() * t.element_size() for t in host[2:])

        def local():
            return pipe(*host, out_costs, None, None)
    else:
        out_labels = torch.empty((n, w.U), dtype=torch.int32).pin_memory()
        d2h = out_labels.numel() * 4
        h2d -= host[2].numel() * 4   # labels are an output here
        api = "TransducerLoss.viterbi on chunks of 8 utterances, 3 streams, valid frames / positions only over the link"
        slots = [(torch.cuda.Stream(device=dev), {}) for _ in range(3)]
        chunk = 8
        t_len = [min(int(x), w.T) for x in host[3].tolist()]
        u_len = [min(int(x) + 1, w.U + 1) for x in host[4].tolist()]
        h2d = (sum(t_len) * host[0].element_size() + sum(u_len) * host[1].element_size()) * w.V + \
            host[3].numel() * 4 + host[4].numel() * 4 + host[2].numel() * 4

        def local():
            main = torch.cuda.current_stream()
            for i, lo in enumerate(range(0, n, chunk)):
                hi = min(n, lo + chunk)
                s, buf = slots[i % len(slots)]
                s.wait_stream(main)
                with torch.cuda.stream(s):
                    if buf.get("n") != hi - lo:
                        buf["E"] = torch.empty((hi - lo,) + tuple(host[0].shape[1:]), device=dev)
                        buf["P"] = torch.empty((hi - lo,) + tuple(host[1].shape[1:]), device=dev)
                        buf["il"] = torch.empty((hi - lo,), dtype=torch.int32, device=dev)
                        buf["ll"] = torch.empty((hi - lo,), dtype=torch.int32, device=dev)
                        buf["n"] = hi - lo
                    for k in range(hi - lo):   # (the kernels never read the padding)
                        buf["E"][k, :t_len[lo + k]].copy_(host[0][lo + k, :t_len[lo + k]], non_blocking=True)
                        buf["P"][k, :u_len[lo + k]].copy_(host[1][lo + k, :u_len[lo + k]], non_blocking=True)
                    buf["il"].copy_(host[3][lo:hi], non_blocking=True)
                    buf["ll"].copy_(host[4][lo:hi], non_blocking=True)
                    lab = crit.viterbi(buf["E"], buf["P"], buf["il"], buf["ll"])
                    out_labels[lo:hi].copy_(lab, non_blocking=True)
            for s, _ in slots:
                main.wait_stream(s)
            return None

    def step():
        loss_sum = local()
        if distributed and loss_sum is not None:
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
    ms = t.item() / steps                      # for n utterances per rank
    ms_full = ms * B / n                       # the rank's whole shard
    return {"value": global_B / (ms_full * 1e-3), "unit": "utterances/s", "ms_per_step": ms_full,
            "h2d_bytes_per_step": int(h2d * B / n), "d2h_bytes_per_step": int(d2h * B / n),
            "h2d_gbs_per_rank": h2d / (ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (ms * 1e-3) / 1e9,
            "h2d_gbs_all_ranks": world * h2d / (ms * 1e-3) / 1e9,
            "d2h_gbs_all_ranks": world * d2h / (ms * 1e-3) / 1e9,
            "utterances_timed_per_rank": n, "steps": steps, "api": api,
            "limiter": "the host<->device link of the box (shared by its GPUs), not a kernel"}


if __name__ == "__main__":
    main()
