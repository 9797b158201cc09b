"""GPU tests of the Python surface (TransducerLoss / criterion.viterbi), modelled on
the reference's torch_test.py."""
import numpy as np
import pytest
import torch

import abi
from conftest import kat_arrays
from oracle import oracle as O
from transducer_b200 import TransducerLoss

pytestmark = pytest.mark.gpu


def run_loss(c, deltas=None):
    E = torch.tensor(c["E"], device="cuda", requires_grad=True)
    P = torch.tensor(c["P"], device="cuda", requires_grad=True)
    labels = torch.tensor(c["labels"], dtype=torch.int32, device="cuda")
    il = torch.tensor(c["in_lens"], dtype=torch.int32, device="cuda")
    ll = torch.tensor(c["lab_lens"], dtype=torch.int32, device="cuda")
    crit = TransducerLoss()
    costs = crit(E, P, labels, il, ll)
    w = torch.ones_like(costs) if deltas is None else torch.tensor(deltas, device="cuda")
    finite = torch.isfinite(costs)
    (w * costs)[finite].sum().backward()
    return costs.detach().cpu(), E.grad.cpu(), P.grad.cpu(), crit


@pytest.mark.parametrize("name", ["small", "big"])
def test_known_answers(kats, name):
    # torch_test.py:41-129 (CUDA tolerance 1e-3/1e-3 there)
    k = kat_arrays(kats[name])
    costs, eg, pg, crit = run_loss(k)
    assert torch.allclose(costs, torch.tensor(k["costs"]), 1e-3, 1e-3)
    assert torch.allclose(eg, torch.tensor(k["egrads"]), 1e-3, 1e-3)
    assert torch.allclose(pg, torch.tensor(k["pgrads"]), 1e-3, 1e-3)
    assert torch.isclose(crit.last_loss_sum.cpu()[0], costs.sum(), rtol=1e-5)


def test_viterbi_known_answer(kats):
    # torch_test.py:131-158
    v = kats["viterbi"][3]
    E = torch.tensor(v["emissions"], device="cuda").reshape(1, 3, 3)
    P = torch.tensor(v["predictions"], device="cuda").reshape(1, 3, 3)
    il = torch.tensor([3], dtype=torch.int32, device="cuda")
    ll = torch.tensor([2], dtype=torch.int32, device="cuda")
    labels = TransducerLoss().viterbi(E, P, il, ll)
    assert labels.dtype == torch.int32 and labels.shape == (1, 2)
    assert labels.cpu().tolist() == [v["labels"]]


def test_stored_reference_outputs(reference_runs):
    for name, c in reference_runs.items():
        if (c["in_lens"] == 0).any():
            continue  # +inf costs: covered through the C ABI
        costs, eg, pg, _ = run_loss(c, c["deltas"])
        assert np.allclose(costs.numpy(), c["costs"], rtol=1e-4), name
        assert np.abs(eg.numpy() - c["egrads"]).max() <= 1e-3 * np.abs(c["egrads"]).max(), name
        assert np.abs(pg.numpy() - c["pgrads"]).max() <= 1e-3 * np.abs(c["pgrads"]).max(), name


def test_finite_difference_gradients():
    # torch_test.py:209-269: central differences, eps 1e-2, isclose(1e-3, 1e-3)
    g = torch.Generator().manual_seed(0)
    B, T, U, V, eps = 3, 6, 3, 4, 1e-2
    E = torch.rand((B, T, V), generator=g).cuda()
    P = torch.rand((B, U, V), generator=g).cuda()
    labels = torch.randint(1, V, (B, U - 1), generator=g, dtype=torch.int32).cuda()
    il = torch.randint(1, T + 1, (B,), generator=g, dtype=torch.int32)
    ll = torch.randint(1, U, (B,), generator=g, dtype=torch.int32)
    il[0], ll[0] = T, U - 1
    il, ll = il.cuda(), ll.cuda()
    crit = TransducerLoss()
    E.requires_grad_(True)
    P.requires_grad_(True)
    crit(E, P, labels, il, ll).sum().backward()
    eg, pg = E.grad.clone(), P.grad.clone()
    E = E.detach()
    P = P.detach()
    with torch.no_grad():
        for X, G in ((E, eg), (P, pg)):
            flat = X.view(-1)
            for i in range(flat.numel()):
                old = flat[i].item()
                flat[i] = old + eps
                up = crit(E, P, labels, il, ll).sum().item()
                flat[i] = old - eps
                dn = crit(E, P, labels, il, ll).sum().item()
                flat[i] = old
                num = (up - dn) / (2 * eps)
                assert abs(num - G.view(-1)[i].item()) <= 1e-3 + 1e-3 * abs(G.view(-1)[i].item()), i


def test_non_default_stream_and_blank():
    g = torch.Generator().manual_seed(1)
    B, T, U, V, blank = 2, 30, 6, 16, 3
    E = torch.randn((B, T, V), generator=g)
    P = torch.randn((B, U, V), generator=g)
    labels = torch.randint(0, V - 1, (B, U - 1), generator=g, dtype=torch.int32)
    labels[labels == blank] = V - 1
    il = torch.tensor([T, T - 7], dtype=torch.int32)
    ll = torch.tensor([U - 1, 2], dtype=torch.int32)
    want = O.loss_and_grads(E.numpy(), P.numpy(), labels.numpy(), il.numpy(), ll.numpy(), blank=blank)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        Ed = E.cuda().requires_grad_(True)
        Pd = P.cuda().requires_grad_(True)
        costs = TransducerLoss(blank=blank)(Ed, Pd, labels.cuda(), il.cuda(), ll.cuda())
        costs.sum().backward()
        vit = TransducerLoss(blank=blank).viterbi(Ed.detach(), Pd.detach(), il.cuda(), ll.cuda())
    s.synchronize()
    assert np.allclose(costs.detach().cpu().numpy(), want["costs"], rtol=1e-5)
    # 1e-4 of the largest gradient element (two fp32 evaluations of a sum of 30 occupancies of
    # magnitude 10 differ by that much in absolute terms)
    assert np.abs(Ed.grad.cpu().numpy() - want["egrads"]).max() < 1e-4 * np.abs(want["egrads"]).max()
    assert np.abs(Pd.grad.cpu().numpy() - want["pgrads"]).max() < 1e-4 * np.abs(want["pgrads"]).max()
    wv = O.viterbi(E.numpy(), P.numpy(), il.numpy(), ll.numpy(), blank=blank)
    for b in range(B):
        assert np.array_equal(vit.cpu().numpy()[b, :ll[b]], wv[b, :ll[b]])


def test_host_pipeline_matches_whole_batch_call():
    from transducer_b200 import HostLossPipeline
    g = torch.Generator().manual_seed(11)
    B, T, U, V = 7, 90, 12, 256
    E = torch.randn((B, T, V), generator=g).pin_memory()
    P = torch.randn((B, U, V), generator=g).pin_memory()
    labels = torch.randint(1, V, (B, U - 1), generator=g, dtype=torch.int32).pin_memory()
    il = torch.randint(T // 2, T + 1, (B,), generator=g, dtype=torch.int32).pin_memory()
    ll = torch.randint(0, U, (B,), generator=g, dtype=torch.int32).pin_memory()
    deltas = torch.rand((B,), generator=g).add_(0.5).pin_memory()
    costs = torch.empty(B).pin_memory()
    eg = torch.empty_like(E).pin_memory()
    pg = torch.empty_like(P).pin_memory()
    pipe = HostLossPipeline(chunk=3, slots=2)      # chunks of 3, 3 and 1 utterances
    for _ in range(2):                             # second call reuses the slots
        loss_sum = pipe(E, P, labels, il, ll, costs, eg, pg, deltas)
        torch.cuda.synchronize()
    Ed, Pd = E.cuda().requires_grad_(True), P.cuda().requires_grad_(True)
    want = TransducerLoss()(Ed, Pd, labels.cuda(), il.cuda(), ll.cuda())
    want.backward(deltas.cuda())
    assert torch.allclose(costs, want.detach().cpu(), rtol=1e-6, atol=1e-5)
    assert abs(loss_sum.item() - want.sum().item()) <= 1e-5 * abs(want.sum().item())
    assert abi.rel_to_max(eg.numpy(), Ed.grad.cpu().numpy()) <= 1e-5
    assert abi.rel_to_max(pg.numpy(), Pd.grad.cpu().numpy()) <= 1e-5
    with pytest.raises(ValueError):
        pipe(E.cuda(), P, labels, il, ll, costs, eg, pg)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_host_pipeline_moving_valid_rows_only_gives_the_same_outputs(dtype):
    """valid_rows_only: the padding never crosses the link; the outputs are complete all the same
    (the padding of the gradients is zero-filled on the host)."""
    from transducer_b200 import HostLossPipeline
    g = torch.Generator().manual_seed(23)
    B, T, U, V = 5, 140, 20, 512
    E = torch.randn((B, T, V), generator=g).to(dtype).pin_memory()
    P = torch.randn((B, U, V), generator=g).to(dtype).pin_memory()
    labels = torch.randint(1, V, (B, U - 1), generator=g, dtype=torch.int32).pin_memory()
    il = torch.randint(T // 3, T + 1, (B,), generator=g, dtype=torch.int32).pin_memory()
    ll = torch.randint(0, U, (B,), generator=g, dtype=torch.int32).pin_memory()
    il[1], ll[1] = T, U - 1
    outs = {}
    for sparse in (False, True):
        costs = torch.full((B,), float("nan")).pin_memory()
        eg = torch.full(E.shape, float("nan"), dtype=dtype).pin_memory()
        pg = torch.full(P.shape, float("nan"), dtype=dtype).pin_memory()
        pipe = HostLossPipeline(chunk=2, slots=2, valid_rows_only=sparse)
        for _ in range(2):   # (the second call finds other utterances' rows in the slots)
            pipe(E, P, labels, il, ll, costs, eg, pg)
            torch.cuda.synchronize()
        outs[sparse] = (costs, eg, pg)
    for a, b in zip(outs[False], outs[True]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_forward_backward_can_be_captured_in_a_cuda_graph():
    """The fused calls only enqueue work (kernels, memsets) on the chosen stream, so a training
    step can be captured once and replayed."""
    g = torch.Generator().manual_seed(5)
    B, T, U, V = 3, 70, 9, 128
    E = torch.randn((B, T, V), generator=g).cuda()
    P = torch.randn((B, U, V), generator=g).cuda()
    labels = torch.randint(1, V, (B, U - 1), generator=g, dtype=torch.int32).cuda()
    il = torch.tensor([T, T - 9, T - 30], dtype=torch.int32).cuda()
    ll = torch.tensor([U - 1, 3, 0], dtype=torch.int32).cuda()
    fwd = abi.loss_forward(E, P, labels, il, ll)          # warm-up outside capture (attributes)
    want_eg, want_pg = abi.loss_backward(E, P, labels, il, ll, fwd)
    want_costs = fwd["costs"].clone()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):   # abi.* enqueue on torch's current stream
        cap = abi.loss_forward(E, P, labels, il, ll)
        eg, pg = abi.loss_backward(E, P, labels, il, ll, cap)
    E2 = E.clone()
    E.mul_(0.5)                                            # new inputs in the captured buffers
    graph.replay()
    torch.cuda.synchronize()
    assert not torch.allclose(cap["costs"], want_costs)
    E.copy_(E2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(cap["costs"], want_costs)
    assert torch.equal(eg, want_eg) and torch.equal(pg, want_pg)


def test_wrapper_without_length_validation_gives_the_same_result():
    g = torch.Generator().manual_seed(6)
    B, T, U, V = 2, 40, 7, 64
    E = torch.randn((B, T, V), generator=g).cuda().requires_grad_(True)
    P = torch.randn((B, U, V), generator=g).cuda().requires_grad_(True)
    labels = torch.randint(1, V, (B, U - 1), generator=g, dtype=torch.int32).cuda()
    il = torch.tensor([T, T - 5], dtype=torch.int32).cuda()
    ll = torch.tensor([U - 1, 2], dtype=torch.int32).cuda()
    want = TransducerLoss()(E, P, labels, il, ll)
    want.sum().backward()
    want_eg, want_pg = E.grad.clone(), P.grad.clone()
    E.grad = None
    P.grad = None
    costs = TransducerLoss(validate_lengths=False)(E, P, labels, il, ll)
    costs.sum().backward()
    assert torch.equal(costs.detach(), want.detach())
    assert torch.equal(E.grad, want_eg) and torch.equal(P.grad, want_pg)
    # the default wrapper still refuses lengths that do not fit (it reads them back)
    with pytest.raises(ValueError):
        TransducerLoss()(E, P, labels, il + 100, ll)
