"""CPU tests of the oracle itself: the plain-C restatement must reproduce the
reference's literal known-answer vectors and, bit for bit, the stored outputs of the
reference's own CPU backend."""
import numpy as np
import pytest

from conftest import kat_arrays
from oracle import oracle as O

IMPLS = ["port"] + (["reference"] if O.have_reference() else [])


def close(a, b, rtol=1e-6, atol=1e-5):
    # transducer/test.h:19-29
    return np.all(np.abs(a - b) <= np.maximum(rtol * np.maximum(np.abs(a), np.abs(b)), atol))


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("name", ["tiny", "small", "big"])
def test_kat_exact_lognorm_harness(kats, name, impl):
    """The harness of transducer/test.cpp:7-90: exact log-normalisers, ABI forward and
    backward, brute-force dense gradient."""
    k = kat_arrays(kats[name])
    LN = O.log_norms_exact(k["E"], k["P"], k["in_lens"], k["lab_lens"])
    costs, alphas = O.forward(k["E"], k["P"], LN, k["labels"], k["in_lens"], k["lab_lens"], impl=impl)
    assert close(costs, k["costs"])
    eg, pg, lg = O.backward(k["E"], k["P"], alphas, LN, k["labels"], k["in_lens"], k["lab_lens"],
                            impl=impl)
    O.accumulate_grads_exact(k["E"], k["P"], eg, pg, lg, LN, k["in_lens"], k["lab_lens"])
    assert close(eg, k["egrads"])
    assert close(pg, k["pgrads"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("name", ["tiny", "small", "big"])
def test_kat_torch_path(kats, name, impl):
    """torch_test.py:41-129: the same vectors through the factored (torch-op) path."""
    k = kat_arrays(kats[name])
    r = O.loss_and_grads(k["E"], k["P"], k["labels"], k["in_lens"], k["lab_lens"], impl=impl)
    assert np.allclose(r["costs"], k["costs"], rtol=1e-5, atol=1e-8)
    assert np.allclose(r["egrads"], k["egrads"], rtol=1e-5, atol=1e-6)
    assert np.allclose(r["pgrads"], k["pgrads"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_viterbi(kats, impl):
    for v in kats["viterbi"]:
        B, T, U, V = v["B"], v["T"], v["U"], v["V"]
        # the reference's "empty transcript" block lists more emissions than T*V: the
        # call only addresses the first B*T*V of them
        E = np.asarray(v["emissions"], np.float32)[:B * T * V].reshape(B, T, V)
        P = np.asarray(v["predictions"], np.float32)[:B * U * V].reshape(B, U, V) \
            if v["predictions"] else np.zeros((B, U, V), np.float32)
        il, ll = np.asarray(v["input_lengths"], np.int32), np.asarray(v["label_lengths"], np.int32)
        LN = O.log_norms_exact(E, P, il, ll)
        got = O.viterbi_abi(E, P, LN, il, ll, blank=v["blank"], impl=impl)
        n = len(v["labels"])
        assert list(got[0, :n]) == v["labels"], v["title"]


def test_port_bit_exact_with_reference_runs(reference_runs):
    """The restatement against stored outputs of the reference's CPU path."""
    for name, c in reference_runs.items():
        r = O.loss_and_grads(c["E"], c["P"], c["labels"], c["in_lens"], c["lab_lens"],
                             deltas=c["deltas"], impl="port")
        for f in ("costs", "egrads", "pgrads", "log_norms"):
            assert np.array_equal(r[f], c[f], equal_nan=True), (name, f)
        v = O.viterbi(c["E"], c["P"], c["in_lens"], c["lab_lens"], impl="port")
        assert np.array_equal(v, c["viterbi"]), name


@pytest.mark.skipif(not O.have_reference(), reason="reference CPU backend not built")
def test_port_bit_exact_with_live_reference():
    rng = np.random.default_rng(7)
    for (B, T, U, V) in [(3, 40, 9, 33), (2, 120, 30, 64), (5, 9, 1, 7)]:
        E = rng.standard_normal((B, T, V)).astype(np.float32)
        P = rng.standard_normal((B, U, V)).astype(np.float32)
        labels = rng.integers(1, V, (B, max(U - 1, 0))).astype(np.int32)
        il = rng.integers(0, T + 1, B).astype(np.int32)
        ll = rng.integers(0, U, B).astype(np.int32)
        a = O.loss_and_grads(E, P, labels, il, ll, impl="port")
        b = O.loss_and_grads(E, P, labels, il, ll, impl="reference")
        for f in a:
            assert np.array_equal(a[f], b[f], equal_nan=True), f
        assert np.array_equal(O.viterbi(E, P, il, ll, impl="port"),
                              O.viterbi(E, P, il, ll, impl="reference"))


def test_exact_and_factored_lognorms_agree():
    rng = np.random.default_rng(3)
    E = rng.standard_normal((2, 20, 50)).astype(np.float32)
    P = rng.standard_normal((2, 6, 50)).astype(np.float32)
    il, ll = np.array([20, 11], np.int32), np.array([5, 2], np.int32)
    a = O.log_norms_exact(E, P, il, ll)
    b = O.log_norms_factored_c(E, P)
    c = O.log_norms_torch(E, P)[0].numpy()
    m = np.zeros(a.shape, bool)
    for i in range(2):
        m[i, :il[i], :ll[i] + 1] = True
    assert np.abs(a - b)[m].max() < 5e-6 and np.abs(b - c).max() < 5e-6


def test_truth64_brackets_fp32_oracle(reference_runs):
    c = reference_runs["c1"]
    t = O.truth64(c["E"], c["P"], c["labels"], c["in_lens"], c["lab_lens"])
    d = c["deltas"].astype(np.float64)[:, None, None]
    assert np.allclose(t["costs"], c["costs"], rtol=1e-5)
    assert np.abs(d * t["egrads"] - c["egrads"]).max() < 1e-4 * np.abs(c["egrads"]).max()
    assert np.abs(d * t["pgrads"] - c["pgrads"]).max() < 1e-4 * np.abs(c["pgrads"]).max()
