"""The drop-in boundary proven with the reference's OWN code on a GPU.

oracle/Makefile compiles, unmodified, (1) the reference's pybind shim transducer/_transducer.cpp
against this repository's include/transducer.h and links it to libtransducer_b200.so, next to
build-time copies of the reference's transducer/__init__.py and torch_binding.py, and (2) the
reference's CUDA test program transducer/test_cuda.cu against include/transducer.h and
include/transducer_cuda.h.  Here the reference's own TransducerLoss runs on CUDA tensors on top of
that shim -- i.e. the three C++-linkage functions forward / backward / viterbi with useCuda=true --
and must reproduce the reference's known answers (the CUDA halves of torch_test.py:41-158, at
its CUDA tolerance allclose(1e-3, 1e-3)); and the test program's device-only groups must pass.
Its stressTest (test_cuda.cu:323-378) needs the CPU backend for its comparison
(useCuda=false, :363), which this library refuses; test_parity_gpu.py restates that sweep
against the oracle instead."""
import glob
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, kat_arrays

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(ROOT, "oracle", "_ref")
HAVE_SHIM = bool(glob.glob(os.path.join(REF_DIR, "transducer", "_transducer*.so"))) and \
    os.path.exists(os.path.join(REF_DIR, "transducer", "torch_binding.py"))
HAVE_TEST = os.path.exists(os.path.join(REF_DIR, "ref_test_cuda"))


@pytest.fixture(scope="module")
def ref_package():
    if not HAVE_SHIM:
        pytest.skip("reference shim was not built (needs the reference sources at build time)")
    sys.path.insert(0, REF_DIR)
    # The reference's wrapper was written for PyTorch 1.9 and calls torch.cuda.get_device()
    # (transducer/torch_binding.py:15), which current PyTorch no longer has: with any CUDA tensor
    # it raises AttributeError before reaching native code, whatever library is underneath.  The
    # test lends it the present-day name of that function; the reference's files stay untouched.
    lent = not hasattr(torch.cuda, "get_device")
    if lent:
        torch.cuda.get_device = torch.cuda.current_device
    try:
        import transducer  # the reference's package: its torch_binding.py + its shim on our library
        yield transducer
    finally:
        sys.path.remove(REF_DIR)
        if lent:
            del torch.cuda.get_device


def _run(ref_package, k):
    E = torch.tensor(k["E"], device="cuda", requires_grad=True)
    P = torch.tensor(k["P"], device="cuda", requires_grad=True)
    labels = torch.tensor(k["labels"], dtype=torch.int32, device="cuda")
    il = torch.tensor(k["in_lens"], dtype=torch.int32, device="cuda")
    ll = torch.tensor(k["lab_lens"], dtype=torch.int32, device="cuda")
    costs = ref_package.TransducerLoss()(E, P, labels, il, ll)
    torch.sum(costs).backward()
    return costs.detach().cpu(), E.grad.cpu(), P.grad.cpu()


@pytest.mark.parametrize("name", ["small", "big"])
def test_reference_wrapper_known_answers_on_cuda(ref_package, kats, name):
    k = kat_arrays(kats[name])
    costs, eg, pg = _run(ref_package, k)
    assert torch.allclose(costs, torch.tensor(k["costs"]), 1e-3, 1e-3)
    assert torch.allclose(eg, torch.tensor(k["egrads"]), 1e-3, 1e-3)
    assert torch.allclose(pg, torch.tensor(k["pgrads"]), 1e-3, 1e-3)


def test_reference_wrapper_viterbi_on_cuda(ref_package, kats):
    v = kats["viterbi"][3]
    E = torch.tensor(v["emissions"], device="cuda").reshape(1, 3, 3)
    P = torch.tensor(v["predictions"], device="cuda").reshape(1, 3, 3)
    il = torch.tensor([3], dtype=torch.int32, device="cuda")
    ll = torch.tensor([2], dtype=torch.int32, device="cuda")
    labels = ref_package.TransducerLoss().viterbi(E, P, il, ll)
    assert labels.cpu().tolist() == [v["labels"]]


def test_reference_wrapper_matches_this_librarys_wrapper(ref_package):
    """Same random batch through the reference's wrapper (torch-op log-normalisers and dense
    gradients around our forward/backward) and through transducer_b200.TransducerLoss."""
    from transducer_b200 import TransducerLoss
    g = torch.Generator(device="cuda").manual_seed(3)
    B, T, U1, V = 3, 60, 9, 40
    E = torch.empty((B, T, V), device="cuda").normal_(0, 1, generator=g)
    P = torch.empty((B, U1, V), device="cuda").normal_(0, 1, generator=g)
    labels = torch.randint(1, V, (B, U1 - 1), generator=g, device="cuda", dtype=torch.int32)
    il = torch.tensor([T, T - 7, T // 2], dtype=torch.int32, device="cuda")
    ll = torch.tensor([U1 - 1, 3, 5], dtype=torch.int32, device="cuda")
    outs = []
    for crit in (ref_package.TransducerLoss(), TransducerLoss()):
        e = E.clone().requires_grad_(True)
        p = P.clone().requires_grad_(True)
        c = crit(e, p, labels, il, ll)
        c.sum().backward()
        outs.append((c.detach(), e.grad, p.grad))
    assert torch.allclose(outs[0][0], outs[1][0], rtol=1e-4)
    for a, b in zip(outs[0][1:], outs[1][1:]):
        assert float((a - b).abs().max()) <= 1e-3 * float(a.abs().max())


@pytest.mark.skipif(not HAVE_TEST, reason="reference CUDA test program was not built")
def test_reference_cuda_test_program_device_groups():
    r = subprocess.run([os.path.join(REF_DIR, "ref_test_cuda")], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    for name in ("tinyTest", "smallTest", "bigTest", "viterbiTest"):
        assert name + " passed" in r.stdout, r.stdout
