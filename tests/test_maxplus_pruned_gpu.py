"""Label-arc scores best[b,t,u] = max over v != blank of E[b,t,v] + P[b,u,v]
(transducer/transducer_cuda.cu:233-242, transducer_cpu.cpp:156-169): the evaluation from
candidate lists with an exact bound must be bit-identical to the full loop over the alphabet,
whatever the data look like -- also where the bound settles nothing."""
import numpy as np
import pytest
import torch

import abi

pytestmark = pytest.mark.gpu


def both_paths(E, P, il, ll, blank):
    out = {}
    try:
        for name, path in (("full", 1), ("lists", 2)):
            abi.set_option("maxplus_path", path)
            out[name] = abi.label_arc_scores(E, P, il, ll, blank=blank)
            torch.cuda.synchronize()
    finally:
        abi.set_option("maxplus_path", 0)
    return out["full"], out["lists"]


def assert_identical(full, lists, il, ll):
    B, T, U = full.shape
    t = torch.arange(T, device="cuda")[None, :, None]
    u = torch.arange(U, device="cuda")[None, None, :]
    valid = (t < il[:, None, None]) & (u < ll[:, None, None])
    a, b = full[valid], lists[valid]
    assert not torch.isnan(a).any()
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    # nothing outside the lattice is touched
    assert torch.isnan(lists[~valid]).all()


def numpy_scores(E, P, blank):
    s = E[:, :, None, :].astype(np.float32) + P[:, None, :, :].astype(np.float32)
    s[..., blank] = -np.inf
    return s.max(-1)


def lengths(B, T, U, gen, full_first=True):
    il = torch.randint(max(1, T // 2), T + 1, (B,), generator=gen, dtype=torch.int32)
    ll = torch.randint(max(1, (U - 1) // 2), U, (B,), generator=gen, dtype=torch.int32)
    if full_first:
        il[0], ll[0] = T, U - 1
    return il.cuda(), ll.cuda()


CASES = [
    # B, T, U', V, blank, kind
    (3, 70, 20, 1024, 0, "normal"),
    (2, 130, 41, 4096, 7, "normal"),
    (2, 90, 33, 2049, 2048, "normal"),       # odd alphabet (scalar loads), blank last
    (2, 64, 17, 1500, 3, "flat"),            # all scores equal: the bound settles nothing
    (2, 64, 40, 2048, 0, "quantised"),       # many exact ties
    (2, 50, 19, 3000, 5, "peaky"),           # a few dominant words per row
    (2, 40, 12, 1200, 1, "masked"),          # -inf entries, some rows with few finite words
    (1, 33, 70, 5000, 0, "uniform"),         # no tail: the normal quantile guess is wrong
    (1, 300, 151, 4096, 0, "blank_boost"),   # the Viterbi benchmark's value distribution
]


def make(kind, B, T, U, V, blank, gen):
    E = torch.randn(B, T, V, generator=gen)
    P = torch.randn(B, U, V, generator=gen)
    if kind == "flat":
        E.fill_(0.25)
        P.fill_(-1.5)
    elif kind == "quantised":
        E, P = torch.round(E * 2) / 2, torch.round(P * 2) / 2
    elif kind == "peaky":
        E += 8.0 * (torch.rand(B, T, V, generator=gen) < 0.002)
        P += 8.0 * (torch.rand(B, U, V, generator=gen) < 0.002)
    elif kind == "masked":
        E[torch.rand(B, T, V, generator=gen) < 0.6] = -float("inf")
        P[torch.rand(B, U, V, generator=gen) < 0.97] = -float("inf")
        E[:, 3] = -float("inf")          # a frame without any finite score
    elif kind == "uniform":
        E, P = torch.rand(B, T, V, generator=gen), torch.rand(B, U, V, generator=gen)
    elif kind == "blank_boost":
        E[:, :, blank] += 4.0
    return E.cuda(), P.cuda()


@pytest.mark.parametrize("B,T,U,V,blank,kind", CASES)
def test_lists_match_full_loop_bit_for_bit(B, T, U, V, blank, kind):
    gen = torch.Generator().manual_seed(hash((B, T, U, V, kind)) % (2 ** 31))
    E, P = make(kind, B, T, U, V, blank, gen)
    il, ll = lengths(B, T, U, gen)
    full, lists = both_paths(E, P, il, ll, blank)
    assert_identical(full, lists, il, ll)
    # and the full loop against a plain numpy restatement of the reference's loop
    if B * T * U * V <= 3e8:
        want = torch.as_tensor(numpy_scores(E.cpu().numpy(), P.cpu().numpy(), blank)).cuda()
        t = torch.arange(T, device="cuda")[None, :, None]
        u = torch.arange(U, device="cuda")[None, None, :]
        valid = (t < il[:, None, None]) & (u < ll[:, None, None])
        assert torch.equal(full[valid], want[valid])


def test_small_alphabets_use_the_full_loop():
    gen = torch.Generator().manual_seed(5)
    E, P = make("normal", 2, 30, 9, 200, 0, gen)
    il, ll = lengths(2, 30, 9, gen)
    assert abi.lib.tb200_label_arc_scores_workspace_bytes(2, 30, 9, 200) == 0
    try:
        abi.set_option("maxplus_path", 2)
        with pytest.raises(ValueError):
            abi.label_arc_scores(E, P, il, ll)
    finally:
        abi.set_option("maxplus_path", 0)
    got = abi.label_arc_scores(E, P, il, ll)
    want = torch.as_tensor(numpy_scores(E.cpu().numpy(), P.cpu().numpy(), 0)).cuda()
    assert torch.equal(got[0, :, :8], want[0, :, :8])


def test_viterbi_labels_do_not_depend_on_the_path():
    gen = torch.Generator().manual_seed(11)
    B, T, U, V = 3, 200, 60, 2048
    E, P = make("blank_boost", B, T, U, V, 0, gen)
    il, ll = lengths(B, T, U, gen)
    got = {}
    try:
        for path in (1, 2):
            abi.set_option("maxplus_path", path)
            got[path] = abi.viterbi_decode(E, P, il, ll, blank=0)
    finally:
        abi.set_option("maxplus_path", 0)
    assert torch.equal(got[1], got[2])
