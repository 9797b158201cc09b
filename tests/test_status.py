"""Device-side failure detection: a bounded wait that runs out inside a kernel must reach the
host as TB200_ERR_DEVICE_STATUS / DeviceStatusError, with the CUDA context still usable.

The failure is produced the only permitted way: a self-test kernel waits, with a limit of a few
microseconds, on a barrier that nothing ever completes, and returns normally.  Nothing here
faults, traps or hangs a GPU.  The code -> exception mapping is tested without a GPU."""
import pytest
import torch

from transducer_b200 import errors


def test_return_codes_map_to_exceptions():
    errors.raise_for_status(0, "")
    with pytest.raises(ValueError, match="workspace too small"):
        errors.raise_for_status(errors.TB200_ERR_WORKSPACE, "workspace too small: need 8 bytes, got 0")
    with pytest.raises(ValueError):
        errors.raise_for_status(errors.TB200_ERR_INVALID_ARGUMENT, "blank outside [0, alphabetSize)")
    # a status value as tb200_check_status reports it, injected on the host
    msg = "device status 3: an MMA completion was never signalled within the time limit"
    with pytest.raises(errors.DeviceStatusError, match="device status 3"):
        errors.raise_for_status(errors.TB200_ERR_DEVICE_STATUS, msg)
    assert issubclass(errors.DeviceStatusError, RuntimeError)
    with pytest.raises(errors.Tb200Error, match="tb200 error 2"):
        errors.raise_for_status(errors.TB200_ERR_CUDA, "[file:1] CUDA error: out of memory")


def test_status_names_without_a_gpu():
    from transducer_b200 import _lib
    names = [_lib.lib.tb200_status_name(c).decode() for c in range(0, 8)]
    assert names[0] == "ok" and "copy never landed" in names[1] and "peer" in names[6]
    assert "unknown" in names[7]
    assert len(set(names[:7])) == 7


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    import abi
    lib = abi.lib
    abi.use_torch_stream()
    assert lib.tb200_check_status() == 0                      # clean to begin with
    abi.check(lib.tb200_selftest_wait_timeout(20))            # 20 microseconds, then gives up
    rc = lib.tb200_check_status()
    assert rc == errors.TB200_ERR_DEVICE_STATUS == 5
    msg = lib.tb200_last_error().decode()
    assert "device status 5" in msg and "self-test" in msg
    assert lib.tb200_check_status() == 0                      # reading the word clears it
    # the context is alive: a real kernel of the library runs and gives the right answer
    E = torch.zeros((1, 2, 32), device="cuda")
    P = torch.zeros((1, 1, 32), device="cuda")
    il = torch.tensor([2], dtype=torch.int32, device="cuda")
    ll = torch.tensor([0], dtype=torch.int32, device="cuda")
    LN, _, _ = abi.log_norms(E, P, il, ll)
    torch.cuda.synchronize()
    assert torch.allclose(LN[0, :, 0].cpu(), torch.full((2,), 3.4657359))   # log(32)
    assert lib.tb200_check_status() == 0


@pytest.mark.gpu
def test_python_surface_raises_device_status_error():
    import abi
    from transducer_b200 import DeviceStatusError, TransducerLoss, torch_binding
    abi.use_torch_stream()
    abi.check(abi.lib.tb200_selftest_wait_timeout(20))
    with pytest.raises(DeviceStatusError, match="self-test"):
        torch_binding.check_device_status()
    torch_binding.check_device_status()                       # cleared
    # the reference-style call (validate_lengths=True) checks by itself
    abi.check(abi.lib.tb200_selftest_wait_timeout(20))
    E = torch.randn((1, 4, 32), device="cuda")
    P = torch.randn((1, 2, 32), device="cuda")
    lab = torch.ones((1, 1), dtype=torch.int32, device="cuda")
    il = torch.tensor([4], dtype=torch.int32, device="cuda")
    ll = torch.tensor([1], dtype=torch.int32, device="cuda")
    with pytest.raises(DeviceStatusError):
        TransducerLoss()(E, P, lab, il, ll)
    costs = TransducerLoss()(E, P, lab, il, ll)               # next call is clean
    assert torch.isfinite(costs).all()
