"""GPU tests of the tensor-core gradient kernel against the SIMT gradient kernels (same
weights, same sparse terms) and the CPU oracle: every tile size, K tails, ragged lengths,
blank inside/outside a column block, repeated labels, both operand-split modes."""
import numpy as np
import pytest
import torch

import abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def make(B, T, U, V, std=1.0, seed=0, repeat_labels=False, blank=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    E = torch.empty((B, T, V), device="cuda").normal_(0, std, generator=g)
    P = torch.empty((B, U, V), device="cuda").normal_(0, std, generator=g)
    hi = 4 if repeat_labels else V
    labels = torch.randint(1, hi, (B, max(U - 1, 0)), generator=g, device="cuda", dtype=torch.int32)
    if blank != 0:
        labels[labels == blank] = 0
    il = torch.randint(max(1, T // 2), T + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    ll = torch.randint(0, U, (B,), generator=g, device="cuda", dtype=torch.int32)
    il[0], ll[0] = T, U - 1
    deltas = torch.empty((B,), device="cuda").uniform_(0.5, 1.5, generator=g)
    return E, P, labels, il, ll, deltas


def grads(E, P, labels, il, ll, deltas, path, passes=2, blank=0):
    abi.set_option("grads_path", path)
    abi.set_option("grad_passes", passes)
    try:
        fwd = abi.loss_forward(E, P, labels, il, ll, blank=blank)
        eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd, deltas, blank=blank)
        torch.cuda.synchronize()
    finally:
        abi.set_option("grads_path", 0)
        abi.set_option("grad_passes", 2)
    return fwd, eg, pg


SHAPES = [
    (2, 200, 33, 128, 1.0), (2, 150, 21, 260, 2.0), (3, 300, 101, 1000, 1.0), (1, 130, 1, 64, 1.0),
    (2, 100, 128, 160, 1.0), (2, 90, 64, 96, 1.0), (1, 64, 17, 32, 1.0), (2, 500, 101, 4000, 2.0),
    # label axes of more than 128 positions: two launches over halves of the axis, the second
    # adding to egrads (the lengths of the second utterance put it below / inside the second half)
    (2, 260, 151, 512, 1.0), (3, 180, 201, 1000, 1.0), (2, 300, 256, 264, 1.0), (2, 150, 129, 128, 1.0),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("passes", [3, 2, 1])
def test_matches_simt_kernels(shape, passes):
    B, T, U, V, std = shape
    case = make(B, T, U, V, std, seed=B + T + U + V)
    _, eg_s, pg_s = grads(*case, path=1)
    _, eg_t, pg_t = grads(*case, path=2, passes=passes)
    assert not torch.isnan(eg_t).any() and not torch.isnan(pg_t).any()
    tol = {3: 3e-4, 2: 1e-3, 1: 2e-3}[passes]
    e_err = (eg_t - eg_s).abs().max().item() / eg_s.abs().max().item()
    p_err = (pg_t - pg_s).abs().max().item() / pg_s.abs().max().item()
    assert e_err <= tol and p_err <= tol, (shape, passes, e_err, p_err)
    # padding rows are exact zeros
    il, ll = case[3], case[4]
    for b in range(B):
        if il[b] < T:
            assert eg_t[b, il[b]:].abs().max().item() == 0.0
        if ll[b] + 1 < U:
            assert pg_t[b, ll[b] + 1:].abs().max().item() == 0.0


def test_repeated_labels_and_nonzero_blank_against_oracle():
    B, T, U, V, blank = 2, 120, 40, 256, 130   # blank sits in the second column block
    E, P, labels, il, ll, deltas = make(B, T, U, V, seed=4, repeat_labels=True, blank=blank)
    _, eg, pg = grads(E, P, labels, il, ll, deltas, path=2, blank=blank)
    n = lambda t: t.cpu().numpy()
    # against exact arithmetic (float64): tighter than against the reference's own fp32
    # arithmetic, which is itself 5e-5 away from it on this case
    truth = O.truth64(n(E), n(P), n(labels), n(il), n(ll), blank=blank)
    dl = n(deltas).astype(np.float64)[:, None, None]
    assert abi.rel_to_max(n(eg), truth["egrads"] * dl) <= 1e-4
    assert abi.rel_to_max(n(pg), truth["pgrads"] * dl) <= 1e-4
    want = O.loss_and_grads(n(E), n(P), n(labels), n(il), n(ll), blank=blank, deltas=n(deltas))
    assert abi.rel_to_max(n(eg), want["egrads"]) <= 3e-4
    assert abi.rel_to_max(n(pg), want["pgrads"]) <= 3e-4


def test_wide_label_axis_against_oracle_with_repeats_and_blank():
    """U' = 201, few distinct labels (so that more than 16 of them fall into one column block in
    both halves of the label axis) and a blank that is not 0."""
    B, T, U, V, blank = 2, 230, 201, 256, 70
    E, P, labels, il, ll, deltas = make(B, T, U, V, seed=14, repeat_labels=True, blank=blank)
    ll[1] = 140
    fwd, eg, pg = grads(E, P, labels, il, ll, deltas, path=2, blank=blank)
    abi.check(abi.lib.tb200_check_status())
    n = lambda t: t.cpu().numpy()
    want = O.loss_and_grads(n(E), n(P), n(labels), n(il), n(ll), blank=blank, deltas=n(deltas))
    np.testing.assert_allclose(n(fwd["costs"]), want["costs"], rtol=1e-4)
    assert abi.rel_to_max(n(eg), want["egrads"]) <= 1e-3
    assert abi.rel_to_max(n(pg), want["pgrads"]) <= 1e-3
    assert pg[1, 141:].abs().max().item() == 0.0


def test_zero_length_utterances_give_zero_gradients():
    E, P, labels, il, ll, deltas = make(3, 70, 9, 64, seed=8)
    il[1] = 0
    _, eg, pg = grads(E, P, labels, il, ll, deltas, path=2)
    assert eg[1].abs().max().item() == 0.0 and pg[1].abs().max().item() == 0.0
    assert torch.isfinite(eg).all() and torch.isfinite(pg).all()


def test_unsupported_shape_is_refused_when_forced():
    case = make(1, 40, 5, 30, seed=1)
    with pytest.raises(ValueError, match="tensor-core gradients"):
        grads(*case, path=2)
