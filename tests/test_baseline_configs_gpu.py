"""GPU parity tests on the benchmark configurations themselves (transducer_b200.workloads.CONFIGS,
the seeded synthetic stand-ins for the shapes of the reference's benchmarks/torch_benchmarks.py):
every utterance of every configuration goes through the C ABI and is compared with the CPU
oracle (the reference's own CPU backend where it was built, else its restatement).

Bars: per-utterance losses within 1e-4 relative, gradients within 1e-3 of the gradient's largest
magnitude, Viterbi labels bit-exact.

The gradient bar needs a third party.  The reference carries its alphas in fp32 at a magnitude
of 1e4 after 2000 frames (one ulp = 1e-3), and its gradients are measurably noisy there: its CPU
backend sits 1e-3 .. 6e-3 (of the gradient's maximum) away from a float64 evaluation of the same
formulas, and its own CUDA backend sits up to 2.5e-3 away from its CPU backend.  No
implementation can be within 1e-3 of a result that is itself 5e-3 from the exact value, except
by reproducing its rounding errors bit for bit.  So every utterance is also evaluated in float64
(oracle.truth64) and the tests assert
  * strictly: this library is within 1e-3 of the float64 gradients (it is ~1e-4: its alphas are
    stored relative to per-block offsets), and its losses within 1e-4 of the oracle's;
  * the bar itself against the oracle: where the distance exceeds 1e-3 but stays within 1.5x the
    oracle's OWN distance to float64 on the same utterances, the test reports XFAIL with the
    numbers; beyond that it fails.
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


def loss_rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf])
    return float((np.abs(got[~inf] - want[~inf]) / np.maximum(np.abs(want[~inf]), 1e-30)).max())


def fwd_bwd_against_oracle(w):
    """Whole configuration `w` (forward + backward, one call each) against the oracle, the
    float64 evaluation and, where it was built, the reference's own CUDA backend."""
    torch.cuda.empty_cache()
    E, P, labels, il, ll = workloads.generate(w, "cuda")
    fwd = abi.loss_forward(E, P, labels, il, ll, blank=w.blank)
    eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd, blank=w.blank)
    torch.cuda.synchronize()
    abi.check(abi.lib.tb200_check_status())
    costs = npy(fwd["costs"])
    have_cuda_ref = O.have_reference_cuda() and E.numel() < 2 ** 31
    names = ("ours_vs_oracle", "ours_vs_fp64", "oracle_vs_fp64", "refcuda_vs_oracle")
    dist = {n: {"e": 0.0, "p": 0.0} for n in names}
    l_err, l_err64, l_oracle64 = 0.0, 0.0, 0.0

    def rel(got, want):   # one utterance, on the device, float64
        w64 = torch.as_tensor(np.ascontiguousarray(want)).cuda().double()
        return float((got.double() - w64).abs().max() / w64.abs().max())

    step = 8
    for lo in range(0, w.B, step):
        sl = slice(lo, min(w.B, lo + step))
        host = [npy(t[sl]) for t in (E, P, labels, il, ll)]
        want = O.loss_and_grads(*host, blank=w.blank, impl=IMPL)
        l_err = max(l_err, loss_rel(costs[sl], want["costs"]))
        rc = O.loss_and_grads_cuda(E[sl], P[sl], labels[sl], il[sl], ll[sl], blank=w.blank) \
            if have_cuda_ref else None
        for k in range(sl.stop - lo):
            b = lo + k
            tr = O.truth64(*[h[k:k + 1] for h in host], blank=w.blank)
            for key, ours, theirs, truth, ref in (("e", eg, want["egrads"], tr["egrads"], "egrads"),
                                                  ("p", pg, want["pgrads"], tr["pgrads"], "pgrads")):
                o_dev = torch.as_tensor(np.ascontiguousarray(theirs[k])).cuda()
                dist["ours_vs_oracle"][key] = max(dist["ours_vs_oracle"][key], rel(ours[b], theirs[k]))
                dist["ours_vs_fp64"][key] = max(dist["ours_vs_fp64"][key], rel(ours[b], truth[0]))
                dist["oracle_vs_fp64"][key] = max(dist["oracle_vs_fp64"][key], rel(o_dev, truth[0]))
                if rc is not None:
                    dist["refcuda_vs_oracle"][key] = max(dist["refcuda_vs_oracle"][key],
                                                         rel(rc[ref][k], theirs[k]))
            l_err64 = max(l_err64, abs(float(costs[b]) - tr["costs"][0]) / tr["costs"][0])
            l_oracle64 = max(l_oracle64, abs(float(want["costs"][k]) - tr["costs"][0]) / tr["costs"][0])
    # size-independent properties on the full batch
    assert np.isclose(npy(fwd["loss_sum"])[0], costs.sum(), rtol=1e-5)
    for b in range(w.B):   # padding exactly zero
        if int(il[b]) < w.T:
            assert float(eg[b, int(il[b]):].abs().max()) == 0.0
        if int(ll[b]) + 1 < w.U + 1:
            assert float(pg[b, int(ll[b]) + 1:].abs().max()) == 0.0
    row = {"config": w.name, "utterances": w.B, "oracle": IMPL, "loss_rel_max_vs_oracle": l_err,
           "loss_rel_max_vs_fp64": l_err64, "oracle_loss_rel_max_vs_fp64": l_oracle64}
    for n in names:
        if n != "refcuda_vs_oracle" or have_cuda_ref:
            row[n + "_egrad"], row[n + "_pgrad"] = dist[n]["e"], dist[n]["p"]
    report(row)
    assert l_err <= LOSS_RTOL, row
    assert dist["ours_vs_fp64"]["e"] <= GRAD_TOL and dist["ours_vs_fp64"]["p"] <= GRAD_TOL, row
    for key in ("e", "p"):
        err, floor = dist["ours_vs_oracle"][key], dist["oracle_vs_fp64"][key]
        if err > GRAD_TOL:
            assert err <= 1.5 * floor, row   # more than the oracle's own noise: a real failure
    worst = max(dist["ours_vs_oracle"].values())
    if worst > GRAD_TOL:
        pytest.xfail("distance to the oracle %.2e above 1e-3, within the oracle's own distance to "
                     "float64 (%.2e / %.2e); ours to float64: %.2e / %.2e"
                     % (worst, dist["oracle_vs_fp64"]["e"], dist["oracle_vs_fp64"]["p"],
                        dist["ours_vs_fp64"]["e"], dist["ours_vs_fp64"]["p"]))


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
