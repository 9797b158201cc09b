"""GPU parity tests on the benchmark configurations themselves (transducer_b200.workloads.CONFIGS,
the seeded synthetic stand-ins for the shapes of the reference's benchmarks/torch_benchmarks.py):
every utterance of every configuration goes through the C ABI and is compared with the CPU
oracle (the reference's own CPU backend where it was built, else its restatement).

Bars: per-utterance losses within 1e-4 relative, gradients within 1e-3 of the gradient's largest
magnitude, Viterbi labels bit-exact.  The oracle's own fp32 recursion is noisy at T = 2000 (its
distance to a float64 evaluation is measured here for one utterance per configuration and
reported beside ours): where our distance to the oracle exceeds 1e-3 but stays within twice
that floor, the test reports XFAIL instead of FAIL; beyond that it fails.

Set TB200_PARITY_REPORT=<path> to have the measured distances written there as JSON."""
import json
import os

import numpy as np
import pytest
import torch

import abi
from oracle import oracle as O
from transducer_b200 import workloads

pytestmark = pytest.mark.gpu

LOSS_RTOL = 1e-4
GRAD_TOL = 1e-3
IMPL = "reference" if O.have_reference() else "port"


def npy(t):
    return t.detach().cpu().numpy()


def report(row):
    path = os.environ.get("TB200_PARITY_REPORT")
    print("parity:", json.dumps(row))
    if not path:
        return
    rows = []
    if os.path.exists(path):
        with open(path) as f:
            rows = json.load(f)
    rows = [r for r in rows if r.get("config") != row["config"]] + [row]
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(rows, f, indent=1)


def device_distance(got, want_np):
    """(max|got - want|, max|want|) in float64, evaluated on the device one utterance at a
    time (the arrays are gigabytes)."""
    diff, mag = 0.0, 0.0
    for b in range(got.shape[0]):
        w = torch.from_numpy(np.ascontiguousarray(want_np[b])).cuda().double()
        diff = max(diff, float((got[b].double() - w).abs().max()))
        mag = max(mag, float(w.abs().max()))
    return diff, mag


def loss_rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf])
    return float((np.abs(got[~inf] - want[~inf]) / np.maximum(np.abs(want[~inf]), 1e-30)).max())


def fwd_bwd_against_oracle(w, floor_utt=1):
    """Whole configuration `w` (forward + backward, one call each) against the oracle."""
    torch.cuda.empty_cache()
    E, P, labels, il, ll = workloads.generate(w, "cuda")
    fwd = abi.loss_forward(E, P, labels, il, ll, blank=w.blank)
    eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd, blank=w.blank)
    torch.cuda.synchronize()
    abi.check(abi.lib.tb200_check_status())
    costs = npy(fwd["costs"])
    l_err, e_diff, e_mag, p_diff, p_mag = 0.0, 0.0, 0.0, 0.0, 0.0
    step = 8
    for lo in range(0, w.B, step):
        sl = slice(lo, min(w.B, lo + step))
        want = O.loss_and_grads(npy(E[sl]), npy(P[sl]), npy(labels[sl]), npy(il[sl]), npy(ll[sl]),
                                blank=w.blank, impl=IMPL)
        l_err = max(l_err, loss_rel(costs[sl], want["costs"]))
        d, m = device_distance(eg[sl], want["egrads"])
        e_diff, e_mag = max(e_diff, d), max(e_mag, m)
        d, m = device_distance(pg[sl], want["pgrads"])
        p_diff, p_mag = max(p_diff, d), max(p_mag, m)
        if lo <= floor_utt < lo + step:
            k = floor_utt - lo
            one = slice(floor_utt, floor_utt + 1)
            truth = O.truth64(npy(E[one]), npy(P[one]), npy(labels[one]), npy(il[one]), npy(ll[one]),
                              blank=w.blank)
            e_floor = abi.rel_to_max(want["egrads"][k:k + 1], truth["egrads"])
            p_floor = abi.rel_to_max(want["pgrads"][k:k + 1], truth["pgrads"])
            e_ours64 = abi.rel_to_max(npy(eg[one]), truth["egrads"])
            p_ours64 = abi.rel_to_max(npy(pg[one]), truth["pgrads"])
    # size-independent properties on the full batch
    assert np.isclose(npy(fwd["loss_sum"])[0], costs.sum(), rtol=1e-5)
    for b in range(w.B):   # padding exactly zero
        if int(il[b]) < w.T:
            assert float(eg[b, int(il[b]):].abs().max()) == 0.0
        if int(ll[b]) + 1 < w.U + 1:
            assert float(pg[b, int(ll[b]) + 1:].abs().max()) == 0.0
    row = {"config": w.name, "utterances": w.B, "oracle": IMPL, "loss_rel_max": l_err,
           "egrad_rel_to_max": e_diff / e_mag, "pgrad_rel_to_max": p_diff / p_mag,
           "oracle_vs_fp64_egrad": e_floor, "oracle_vs_fp64_pgrad": p_floor,
           "ours_vs_fp64_egrad": e_ours64, "ours_vs_fp64_pgrad": p_ours64, "floor_utterance": floor_utt}
    report(row)
    assert l_err <= LOSS_RTOL, row
    for err, floor in ((row["egrad_rel_to_max"], e_floor), (row["pgrad_rel_to_max"], p_floor)):
        if err > GRAD_TOL:
            assert err <= 2 * floor, row   # beyond the oracle's own noise: a real failure
            pytest.xfail("gradient distance %.2e above 1e-3 but within twice the oracle's own "
                         "distance to float64 (%.2e)" % (err, floor))


@pytest.mark.parametrize("name", ["c2_v100", "c2_v1000", "c2_v2000", "c2_v10000"])
def test_c2_readme_shape_all_utterances(name):
    """B=8, T=2000, U=100, full lengths, V swept (benchmarks/torch_benchmarks.py:101-105)."""
    fwd_bwd_against_oracle(workloads.CONFIGS[name])


def test_c3_large_batch_all_utterances():
    """B=32, T=2000, U=100, V=10000, N(0,2), ragged lengths: the headline shape, all 32."""
    fwd_bwd_against_oracle(workloads.CONFIGS["c3"])


def test_c4_wordpiece_whole_batch_in_one_call_loss_only():
    """B=256, T=1000, U=200, V=32000, peaky emissions, loss only, ONE forward call: 8.2e9
    emission elements, i.e. offsets beyond 2^31 (where the reference's 32-bit indexing
    overflows, transducer_cpu.cpp:246 -- so the oracle is run in chunks of 16 utterances)."""
    w = workloads.CONFIGS["c4"]
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info()
    need = 4.0 * w.B * w.V * (w.T + 3 * (w.U + 8)) + 8e9
    if free < need:
        pytest.skip("needs %.0f GB of free device memory" % (need / 1e9))
    E, P, labels, il, ll = workloads.generate(w, "cuda")
    assert E.numel() > 2 ** 31
    fwd = abi.loss_forward(E, P, labels, il, ll, blank=w.blank)
    torch.cuda.synchronize()
    abi.check(abi.lib.tb200_check_status())
    costs = npy(fwd["costs"])
    assert np.isfinite(costs).all()
    l_err, step = 0.0, 16
    for lo in range(0, w.B, step):
        sl = slice(lo, lo + step)
        want = O.loss_and_grads(npy(E[sl]), npy(P[sl]), npy(labels[sl]), npy(il[sl]), npy(ll[sl]),
                                blank=w.blank, impl=IMPL, want_grads=False)
        l_err = max(l_err, loss_rel(costs[sl], want["costs"]))
    assert np.isclose(npy(fwd["loss_sum"])[0], costs.astype(np.float64).sum(), rtol=1e-5)
    report({"config": w.name, "utterances": w.B, "oracle": IMPL + " (chunks of 16)",
            "loss_rel_max": l_err, "elements_of_E": int(E.numel())})
    assert l_err <= LOSS_RTOL, l_err


def test_c5_viterbi_all_utterances_bit_exact():
    """B=64, T=1500, U=150, V=4096, +4 on the blank column: labels bit-exact on all 64."""
    w = workloads.CONFIGS["c5"]
    torch.cuda.empty_cache()
    E, P, labels, il, ll = workloads.generate(w, "cuda")
    got = npy(abi.viterbi_decode(E, P, il, ll, blank=w.blank))
    abi.check(abi.lib.tb200_check_status())
    want = O.viterbi(npy(E), npy(P), npy(il), npy(ll), blank=w.blank, impl=IMPL)
    bad = [b for b in range(w.B) if not np.array_equal(got[b, :int(ll[b])], want[b, :int(ll[b])])]
    report({"config": w.name, "utterances": w.B, "oracle": IMPL, "label_mismatches": len(bad)})
    assert not bad, bad
    assert all((got[b, :int(ll[b])] > 0).all() for b in range(w.B))
