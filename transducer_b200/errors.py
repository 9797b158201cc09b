"""Exception types of the library and the mapping from C-ABI return codes
(include/transducer_b200.h, TB200_ERR_*) to them.  Pure Python: importable without the
native library."""

TB200_OK = 0
TB200_ERR_INVALID_ARGUMENT = 1
TB200_ERR_CUDA = 2
TB200_ERR_WORKSPACE = 3
TB200_ERR_UNSUPPORTED = 4
TB200_ERR_DEVICE_STATUS = 5


class Tb200Error(RuntimeError):
    """A call into the native library failed (CUDA error, unsupported shape)."""


class DeviceStatusError(Tb200Error):
    """A bounded wait inside a kernel ran out (TB200_ERR_DEVICE_STATUS): the kernel recorded
    which one in the device status word, returned early and poisoned its outputs (NaN costs
    and gradients, labels of -1).  The CUDA context is still usable."""


def raise_for_status(rc, message=""):
    """Raise the exception that belongs to the C-ABI return code `rc` (nothing for 0).
    Invalid arguments and short workspaces are ValueError, as pybind11 maps the reference's
    std::invalid_argument (transducer/transducer.cpp:41)."""
    if rc == TB200_OK:
        return
    if rc in (TB200_ERR_INVALID_ARGUMENT, TB200_ERR_WORKSPACE):
        raise ValueError(message)
    if rc == TB200_ERR_DEVICE_STATUS:
        raise DeviceStatusError(message)
    raise Tb200Error("tb200 error %d: %s" % (rc, message))
