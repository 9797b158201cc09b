"""CPU tests of the drop-in boundary: the shared library loads without a GPU and
exports every symbol the headers declare; the pybind module and the Python surface
carry the reference's names, keywords, checks and error messages.  No compute call
is made here."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from transducer_b200 import _lib, _transducer, TransducerLoss
from transducer_b200 import torch_binding as tb


def declared_functions():
    src = open(os.path.join(ROOT, "include", "transducer_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(_lib.lib, n), n
        assert n in _lib.SIGNATURES, "ctypes signature missing for " + n


def test_reference_cpp_symbols_exported():
    # Itanium manglings of transducer/transducer.h:3-49 (global namespace, C++ linkage)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for sym in ("_Z7forwardPKfS0_PfS1_S0_PKiS3_S3_iiiiib",
                "_Z8backwardPKfS0_PfS1_S1_S0_S0_PKiS3_S3_iiiiib",
                "_Z7viterbiPKfS0_S0_PiPKiS3_iiiiib"):
        assert getattr(lib, sym) is not None


def test_reference_cuda_namespace_exported():
    # transducer/transducer_cuda.h:7-59: cuda::cudaCheck (behind the CUDA_CHECK macro that the
    # reference's test_cuda.cu / benchmark_cuda.cu use) and cuda::forward/backward/viterbi
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for sym in ("_ZN4cuda9cudaCheckE9cudaErrorPKci",
                "_ZN4cuda7forwardEPKfS1_PfS2_S1_PKiS4_S4_iiiii",
                "_ZN4cuda8backwardEPKfS1_PfS2_S2_S1_S1_PKiS4_S4_iiiii",
                "_ZN4cuda7viterbiEPKfS1_S1_PiPKiS4_iiiii"):
        assert getattr(lib, sym) is not None
    hdr = open(os.path.join(ROOT, "include", "transducer_cuda.h")).read()
    assert "#define CUDA_CHECK(err)" in hdr and "namespace cuda" in hdr


def test_package_import_does_not_load_the_native_library():
    """Helper modules (workloads, distributed, errors) must be importable by a process that
    must not load the CUDA library: bench.py's CPU reference arm is such a process."""
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); import transducer_b200; "
            "from transducer_b200 import workloads, distributed, errors; "
            "bad = [m for m in sys.modules if m.endswith('_transducer') or m.endswith('._lib')]; "
            "assert not bad, bad" % ROOT)
    subprocess.run([sys.executable, "-c", code], check=True)


def test_version_and_options_roundtrip():
    assert _lib.lib.tb200_version() >= 100
    v = ctypes.c_int(-1)
    assert _lib.lib.tb200_get_option(b"grad_passes", ctypes.byref(v)) == 0 and v.value in (1, 2, 3)
    assert _lib.lib.tb200_set_option(b"no_such_key", 1) == 1
    assert b"no_such_key" in _lib.lib.tb200_last_error()


def test_pybind_module_surface():
    for fn in ("forward", "backward", "viterbi", "loss_forward", "loss_backward",
               "viterbi_decode", "log_norms", "set_stream"):
        assert callable(getattr(_transducer, fn))
    assert isinstance(_transducer.__version__, str)
    # keyword names of the reference's shim (transducer/_transducer.cpp:41-54,137-148)
    doc = _transducer.forward.__doc__
    for kw in ("emissions", "predictions", "costs", "alphas", "logNorms", "labels", "input_lengths",
               "label_lengths", "batch_size", "max_input_length", "max_label_length",
               "alphabet_size", "blank", "use_cuda"):
        assert kw in doc
    assert "log_norms" in _transducer.viterbi.__doc__


def test_cpu_backend_is_refused_not_emulated():
    # useCuda=false: std::invalid_argument -> ValueError, as transducer/transducer.cpp:41
    with pytest.raises(ValueError):
        _transducer.forward(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 2, 0, False)
    E = torch.zeros(1, 2, 3)
    P = torch.zeros(1, 2, 3)
    lab = torch.zeros(1, 1, dtype=torch.int32)
    n = torch.tensor([2], dtype=torch.int32)
    m = torch.tensor([1], dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA tensors only"):
        TransducerLoss()(E, P, lab, n, m)


def _args(B=2, T=5, U=3, V=4):
    return [torch.zeros(B, T, V), torch.zeros(B, U, V), torch.zeros(B, U - 1, dtype=torch.int32),
            torch.full((B,), T, dtype=torch.int32), torch.full((B,), U - 1, dtype=torch.int32)]


def test_certify_inputs_messages():
    # transducer/torch_binding.py:180-229
    tb.certify_inputs(*_args())
    a = _args(); a[0] = a[0].double()
    with pytest.raises(TypeError, match="emissions must be torch.float32"):
        tb.certify_inputs(*a)
    a = _args(); a[2] = a[2].long()
    with pytest.raises(TypeError, match="labels must be torch.int32"):
        tb.certify_inputs(*a)
    a = _args(); a[1] = torch.zeros(2, 3, 5)
    with pytest.raises(ValueError, match="vocab size mismatch."):
        tb.certify_inputs(*a)
    a = _args(); a[3] = a[3][:1]
    with pytest.raises(ValueError, match="must have a length per example."):
        tb.certify_inputs(*a)
    a = _args(); a[4] = a[4][:1]
    with pytest.raises(ValueError, match="must have a label length per example."):
        tb.certify_inputs(*a)
    a = _args(); a[2] = torch.zeros(2, 5, dtype=torch.int32)
    with pytest.raises(ValueError, match="labels must be padded to maximum label length."):
        tb.certify_inputs(*a)
    a = _args(); a[2] = torch.zeros(4, 2, dtype=torch.int32)[::2]
    with pytest.raises(ValueError, match="labels must be contiguous"):
        tb.certify_inputs(*a)
    a = _args(); a[3] = a[3] + 1
    with pytest.raises(ValueError, match="Input length mismatch"):
        tb.certify_inputs(*a)
    a = _args(); a[4] = a[4] + 1
    with pytest.raises(ValueError, match="Output length mismatch"):
        tb.certify_inputs(*a)
    a = _args(); a[0] = a[0][0]
    with pytest.raises(ValueError, match="emissions must be 3D"):
        tb.certify_inputs(*a)


def test_workspace_queries_are_pure_and_monotone():
    f = _lib.lib.tb200_loss_backward_workspace_bytes
    assert f(0, 0, 1, 8) >= 0
    assert f(2, 50, 11, 30) <= f(4, 50, 11, 30) <= f(4, 100, 11, 30)
    assert _lib.lib.tb200_viterbi_decode_workspace_bytes(2, 50, 11, 30) > 0


def test_host_pipeline_needs_a_gpu_and_host_tensors():
    """The host-buffer pipeline is part of the product path: no CUDA device, no result."""
    import torch
    from transducer_b200 import HostLossPipeline
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            HostLossPipeline()
