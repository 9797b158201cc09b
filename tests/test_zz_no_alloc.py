"""GPU test of tb200_viterbi_static, the Viterbi entry point for hosts that cannot
allocate device memory (all memory owned by another allocator, no memory-pool support, or
no tolerance for allocation stalls).  It must return exactly what tb200_viterbi returns,
call after call, although all calls share one built-in scratch array that is never cleared.

Collected last on purpose (file name): a run that stops at the first failure has then
already exercised everything else."""
import numpy as np
import pytest
import torch

import abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _case(B, T, U, V, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    E = torch.empty((B, T, V), device="cuda").normal_(0, 1.0, generator=g)
    E[:, :, 0] += 2.0
    P = torch.empty((B, U, V), device="cuda").normal_(0, 1.0, generator=g)
    il = torch.randint(max(1, T // 2), T + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
    ll = torch.randint(0, U, (B,), generator=g, device="cuda", dtype=torch.int32)
    il[0], ll[0] = T, U - 1
    LN, _, _ = abi.log_norms(E, P, il, ll)
    return E, P, LN, il, ll


def _static(E, P, LN, il, ll, blank=0, fill=-1):
    B, T, U, V = abi.shapes(E, P)
    out = torch.full((B, max(U - 1, 0)), fill, dtype=torch.int32, device="cuda")
    abi.use_torch_stream()
    abi.check(abi.lib.tb200_viterbi_static(abi.ptr(E), abi.ptr(P), abi.ptr(LN), abi.ptr(out),
                                           abi.ptr(il), abi.ptr(ll), B, T, U, V, blank))
    return out


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    # two different problems back to back: the second finds the first one's leftovers in
    # the shared scratch and must not be affected by them
    for B, T, U, V, seed in [(3, 150, 24, 96, 1), (2, 90, 40, 50, 2)]:
        E, P, LN, il, ll = _case(B, T, U, V, seed)
        want = abi.viterbi(E, P, LN, il, ll)
        got = _static(E, P, LN, il, ll)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (B, T, U, V)   # bit-exact, padding entries untouched in both
        # and against the CPU oracle's `viterbi` (transducer/transducer.h:37-49) fed with the
        # same log-normalisers: an independent implementation, not another kernel of this library
        cpu = lambda t: t.cpu().numpy()
        ref = O.viterbi_abi(cpu(E), cpu(P), cpu(LN), cpu(il), cpu(ll))
        assert np.array_equal(cpu(got), ref), (B, T, U, V)
        for b in range(B):
            n = int(ll[b])
            assert (got[b, :n] > 0).all() and (got[b, n:] == -1).all()


def test_sizes_beyond_the_built_in_scratch_are_refused():
    limit = abi.lib.tb200_viterbi_static_max_nodes()
    assert limit == 4 << 20
    B, T, U, V = 64, 1500, 151, 4096          # 14.5 Mi nodes
    assert B * T * U > limit
    rc = abi.lib.tb200_viterbi_static(None, None, None, None, None, None, B, T, U, V, 0)
    assert rc == 3
    msg = abi.lib.tb200_last_error().decode()
    assert "exceeds the built-in scratch" in msg and "tb200_viterbi" in msg
    # an empty problem decodes nothing (it only performs the per-device set-up)
    assert abi.lib.tb200_viterbi_static(None, None, None, None, None, None, 0, 10, 3, 8, 0) == 0
