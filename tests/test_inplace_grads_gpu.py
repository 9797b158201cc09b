"""Gradients written over their inputs: tb200_loss_backward (and its bf16 form) may be given
egrads == emissions and pgrads == predictions.  The gradient kernel reads every tile of E, and
every column block of P, into shared / tensor memory before it writes the same tile of the
gradient, and nothing else in the backward call reads E or P (the forward call kept what it
needs in `saved`), so the result is the out-of-place one bit for bit.  The reference allocates
fresh gradients (transducer/torch_binding.py:62-70); this halves the footprint of the
largest tensors of a step."""
import pytest
import torch

import abi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,U,V", [(3, 150, 30, 1000), (2, 97, 120, 264)])
def test_backward_in_place_equals_out_of_place(dtype, B, T, U, V):
    gen = torch.Generator().manual_seed(B * T + U)
    E = torch.randn(B, T, V, generator=gen).to(dtype).cuda()
    P = torch.randn(B, U, V, generator=gen).to(dtype).cuda()
    il = torch.randint(T // 2, T + 1, (B,), generator=gen, dtype=torch.int32).cuda()
    ll = torch.randint(U // 2, U, (B,), generator=gen, dtype=torch.int32).cuda()
    labels = torch.randint(1, V, (B, U - 1), generator=gen, dtype=torch.int32).cuda()
    fwd = abi.loss_forward(E, P, labels, il, ll)
    eg, pg = abi.loss_backward(E, P, labels, il, ll, fwd)
    E2, P2 = E.clone(), P.clone()
    n = abi.lib.tb200_loss_backward_workspace_bytes(B, T, U, V)
    ws = abi.workspace(n)
    deltas = torch.ones(B, device="cuda")
    fn = abi.lib.tb200_loss_backward_bf16 if dtype is torch.bfloat16 else abi.lib.tb200_loss_backward
    abi.use_torch_stream()
    abi.check(fn(abi.ptr(E2), abi.ptr(P2), abi.ptr(labels), abi.ptr(il), abi.ptr(ll),
                 abi.ptr(fwd["saved"]), fwd["saved"].numel(), abi.ptr(deltas), abi.ptr(E2),
                 abi.ptr(P2), B, T, U, V, 0, abi.ptr(ws), n))
    torch.cuda.synchronize()
    abi.check(abi.lib.tb200_check_status())
    assert torch.equal(E2.view(torch.uint8), eg.view(torch.uint8))
    assert torch.equal(P2.view(torch.uint8), pg.view(torch.uint8))
