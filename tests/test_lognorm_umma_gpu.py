"""GPU tests of the tensor-core log-normaliser against the exact SIMT one and the CPU
oracle: K tails, several frame tiles, every label-axis padding, ragged lengths, and
inputs built to drive the factored sum out of fp32 range (exact recompute path)."""
import ctypes

import numpy as np
import pytest
import torch

import abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def run_paths(E, P, il, ll):
    abi.set_option("lognorm_path", 2)
    try:
        ln_tc, ref_tc, mp_tc = abi.log_norms(E, P, il, ll)
        torch.cuda.synchronize()
    finally:
        abi.set_option("lognorm_path", 1)
    try:
        ln_ex, _, mp_ex = abi.log_norms(E, P, il, ll)
        torch.cuda.synchronize()
    finally:
        abi.set_option("lognorm_path", 0)
    return ln_tc, ref_tc, mp_tc, ln_ex, mp_ex


def make(B, T, U, V, std=1.0, seed=0, ragged=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    E = torch.empty((B, T, V), device="cuda").normal_(0, std, generator=g)
    P = torch.empty((B, U, V), device="cuda").normal_(0, std, generator=g)
    if ragged:
        il = torch.randint(1, T + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
        ll = torch.randint(0, U, (B,), generator=g, device="cuda", dtype=torch.int32)
    else:
        il = torch.full((B,), T, device="cuda", dtype=torch.int32)
        ll = torch.full((B,), U - 1, device="cuda", dtype=torch.int32)
    il[0], ll[0] = T, U - 1
    return E, P, il, ll


@pytest.mark.parametrize("shape", [
    (1, 128, 16, 32), (2, 200, 33, 128), (2, 150, 21, 260), (3, 300, 101, 1000),
    (1, 130, 1, 64), (2, 257, 151, 512), (1, 64, 201, 96), (2, 140, 256, 160),
    (4, 1000, 101, 10000),
])
def test_matches_exact_path(shape):
    B, T, U, V = shape
    E, P, il, ll = make(B, T, U, V, std=2.0 if V >= 1000 else 1.0, seed=sum(shape))
    ln_tc, ref_tc, mp_tc, ln_ex, mp_ex = run_paths(E, P, il, ll)
    m = torch.as_tensor(abi.valid_mask(il.cpu().numpy(), ll.cpu().numpy(), T, U), device="cuda")
    assert torch.isfinite(ln_tc[m]).all()
    err = (ln_tc - ln_ex)[m].abs().max().item()
    scale = ln_ex[m].abs().max().item()
    # both are fp32 evaluations of the same sum: a few ulp of the result (the tensor
    # core's truncating adds inside one 2-chunk group cost ~1.5e-6, uniformly)
    assert err <= 4e-7 * max(scale, 1.0) + 3e-6, (shape, err, scale)
    mu = torch.as_tensor(abi.valid_mask(np.ones(B, np.int32), ll.cpu().numpy(), 1, U)[:, 0],
                         device="cuda")
    assert torch.equal(mp_tc[mu], mp_ex[mu])
    # the row shift is a lower bound of the row maximum
    assert (ref_tc <= E.max(dim=2)[0] + 1e-6)[:, :1].all()


def test_matches_oracle_factored_form():
    E, P, il, ll = make(2, 160, 20, 256, seed=3)
    ln_tc, _, _, _, _ = run_paths(E, P, il, ll)
    want = O.log_norms_torch(E.cpu().numpy(), P.cpu().numpy())[0].numpy()
    m = abi.valid_mask(il.cpu().numpy(), ll.cpu().numpy(), 160, 20)
    assert np.abs(ln_tc.cpu().numpy() - want)[m].max() <= 4e-6


def test_out_of_range_rows_are_recomputed_exactly():
    """Rows whose first 32 entries are far below (overflow) or far above (underflow) the
    rest cannot be served by the prefix shift; they must come out exact anyway."""
    B, T, U, V = 1, 128, 8, 256
    E, P, il, ll = make(B, T, U, V, seed=9, ragged=False)
    E[0, 5, :32] -= 200.0      # later entries overflow exp(E - ref)
    E[0, 9, :32] += 200.0      # everything after the prefix underflows against exp(P)
    P[0, :, :32] -= 300.0      # ... because exp(P) is ~0 where E is large
    E[0, 17, 3] = 1e4          # huge outlier inside the prefix
    ln_tc, _, _, ln_ex, _ = run_paths(E, P, il, ll)
    assert torch.isfinite(ln_tc).all()
    assert (ln_tc - ln_ex).abs().max().item() <= 1e-5 * ln_ex.abs().max().item()
    want = O.log_norms_exact(E.cpu().numpy(), P.cpu().numpy(), il.cpu().numpy(), ll.cpu().numpy())
    assert np.abs(ln_tc.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()


def test_unsupported_shape_is_refused_when_forced():
    E, P, il, ll = make(1, 40, 5, 30, seed=1)
    abi.set_option("lognorm_path", 2)
    try:
        with pytest.raises(ValueError, match="tensor-core log-normaliser"):
            abi.log_norms(E, P, il, ll)
    finally:
        abi.set_option("lognorm_path", 0)
