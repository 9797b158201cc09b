"""bfloat16 storage for emissions, predictions and their gradients (tb200_loss_forward_bf16 /
tb200_loss_backward_bf16; not in the reference, which takes fp32 only,
transducer/torch_binding.py:195-197).

Contract: every bf16 value is converted exactly to fp32 on the way in and all arithmetic is the
fp32 path's, so
  * the costs are those of the fp32 entry points on the up-converted inputs (compared bit for
    bit, and with the CPU oracle run on the up-converted inputs at the usual 1e-4),
  * the gradients are those of the fp32 entry points rounded once to bf16: within one bf16
    unit in the last place of them, and within 1e-3 + 2^-8 of the gradient's maximum of the
    oracle's (the fp32 bar plus one rounding: a bf16 value carries 8 significant bits)."""
import numpy as np
import pytest
import torch

import abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu

BF16_GRAD_TOL = 1e-3 + 2.0 ** -8


def make_case(B, T, U, V, blank, seed, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    E = (torch.randn(B, T, V, generator=gen) * scale).to(torch.bfloat16)
    P = (torch.randn(B, U, V, generator=gen) * scale).to(torch.bfloat16)
    il = torch.randint(max(1, T // 2), T + 1, (B,), generator=gen, dtype=torch.int32)
    ll = torch.randint(max(1, (U - 1) // 2), U, (B,), generator=gen, dtype=torch.int32)
    il[0], ll[0] = T, U - 1
    labels = torch.randint(0, V - 1, (B, U - 1), generator=gen, dtype=torch.int32)
    labels[labels >= blank] += 1
    return [t.cuda() for t in (E, P, labels, il, ll)]


CASES = [
    # B, T, U', V, blank
    (3, 70, 12, 64, 0),
    (2, 200, 40, 1000, 0),
    (2, 130, 128, 256, 255),     # widest label axis, blank last
    (2, 300, 33, 4104, 7),       # alphabet not a multiple of 32 or 128 (tail chunk / tail block)
    (1, 129, 2, 32, 0),          # single label, smallest alphabet
]


@pytest.mark.parametrize("B,T,U,V,blank", CASES)
def test_bf16_storage_matches_fp32_path_on_upconverted_inputs(B, T, U, V, blank):
    E, P, labels, il, ll = make_case(B, T, U, V, blank, seed=B * 1000 + T)
    deltas = torch.linspace(0.5, 1.5, B, device="cuda")
    fwd = abi.loss_forward(E, P, labels, il, ll, blank=blank)
    eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd, deltas=deltas, blank=blank)
    Ef, Pf = E.float(), P.float()
    fwd32 = abi.loss_forward(Ef, Pf, labels, il, ll, blank=blank)
    eg32, pg32 = abi.loss_backward(Ef, Pf, labels, il, ll, fwd32, deltas=deltas, blank=blank)
    torch.cuda.synchronize()
    abi.check(abi.lib.tb200_check_status())
    assert eg.dtype == torch.bfloat16 and pg.dtype == torch.bfloat16
    # costs: the same arithmetic on the same values
    assert torch.equal(fwd["costs"], fwd32["costs"])
    assert torch.equal(fwd["loss_sum"], fwd32["loss_sum"])
    # gradients: the fp32 results rounded once (one bf16 ulp of slack: the two gradient kernels
    # may tile the frames differently)
    # (more than 16 labels inside one block of 128 columns: the label-arc terms beyond the 16th
    # are subtracted from the stored bf16 value by a second kernel, i.e. those elements are
    # rounded twice -- one ulp of the value BEFORE the subtraction, bounded here by the maximum)
    twice = U - 1 > 16
    for got, ref in ((eg, eg32), (pg, pg32)):
        assert not torch.isnan(got.float()).any()
        want = ref.to(torch.bfloat16).float()
        ulp = torch.maximum(want.abs(), ref.abs()) * 2.0 ** -7 + 1e-30
        if twice and got is eg:
            ulp = ulp + ref.abs().max() * 2.0 ** -8
        assert bool(((got.float() - want).abs() <= ulp).all())
    # padding exactly zero
    for b in range(B):
        if int(il[b]) < T:
            assert float(eg[b, int(il[b]):].float().abs().max()) == 0.0
        if int(ll[b]) + 1 < U:
            assert float(pg[b, int(ll[b]) + 1:].float().abs().max()) == 0.0
    # and against the CPU oracle on the up-converted inputs
    want = O.loss_and_grads(Ef.cpu().numpy(), Pf.cpu().numpy(), labels.cpu().numpy(),
                            il.cpu().numpy(), ll.cpu().numpy(), blank=blank,
                            deltas=deltas.cpu().numpy())
    np.testing.assert_allclose(fwd["costs"].cpu().numpy(), want["costs"], rtol=1e-4)
    assert abi.rel_to_max(eg.float().cpu().numpy(), want["egrads"]) <= BF16_GRAD_TOL
    assert abi.rel_to_max(pg.float().cpu().numpy(), want["pgrads"]) <= BF16_GRAD_TOL


def test_unsupported_shapes_are_refused_not_converted():
    # alphabet not a multiple of 8
    E, P, labels, il, ll = make_case(2, 40, 9, 100, 0, seed=1)
    with pytest.raises(ValueError):
        abi.loss_forward(E, P, labels, il, ll)
    # label axis beyond the single-warp sweeps
    E, P, labels, il, ll = make_case(1, 40, 140, 64, 0, seed=2)
    with pytest.raises(ValueError):
        abi.loss_forward(E, P, labels, il, ll)


def test_python_surface_takes_bf16_and_returns_bf16_gradients():
    from transducer_b200 import TransducerLoss
    E, P, labels, il, ll = make_case(3, 90, 20, 512, 0, seed=9)
    E.requires_grad_(True)
    P.requires_grad_(True)
    crit = TransducerLoss(blank=0)
    costs = crit(E, P, labels, il, ll)
    assert costs.dtype == torch.float32
    costs.sum().backward()
    assert E.grad.dtype == torch.bfloat16 and P.grad.dtype == torch.bfloat16
    E32 = E.detach().float().requires_grad_(True)
    P32 = P.detach().float().requires_grad_(True)
    costs32 = crit(E32, P32, labels, il, ll)
    costs32.sum().backward()
    assert torch.equal(costs, costs32)
    assert abi.rel_to_max(E.grad.float().cpu().numpy(), E32.grad.cpu().numpy()) <= 2.0 ** -8
    assert abi.rel_to_max(P.grad.float().cpu().numpy(), P32.grad.cpu().numpy()) <= 2.0 ** -8
    # (against the fp32 path of this library the distance is one rounding, no more)
    # mixed storage types are refused with the reference's exception type
    with pytest.raises(TypeError):
        crit(E, P32, labels, il, ll)
