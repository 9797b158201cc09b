"""ctypes view of the C ABI declared in include/transducer_b200.h.

The product path never falls back to anything else: if the shared library has not
been built, importing this module raises."""
import ctypes
import os

from .errors import DeviceStatusError, Tb200Error, raise_for_status  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtransducer_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "transducer_b200: native library missing (%s). Build it with "
        "`python -m transducer_b200.build`; there is no CPU or PyTorch fallback." % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

_p = ctypes.c_void_p
_i = ctypes.c_int
_z = ctypes.c_size_t

# name -> (restype, argtypes); one entry per declaration in transducer_b200.h
SIGNATURES = {
    "tb200_version": (_i, []),
    "tb200_last_error": (ctypes.c_char_p, []),
    "tb200_set_stream": (_i, [_p]),
    "tb200_get_stream": (_p, []),
    "tb200_set_option": (_i, [ctypes.c_char_p, _i]),
    "tb200_get_option": (_i, [ctypes.c_char_p, ctypes.POINTER(_i)]),
    "tb200_launch_count": (ctypes.c_longlong, []),
    "tb200_profile_enable": (_i, [_i]),
    "tb200_profile_reset": (_i, []),
    "tb200_profile_report": (_z, [ctypes.c_char_p, _z]),
    "tb200_check_status": (_i, []),
    "tb200_status_name": (ctypes.c_char_p, [_i]),
    "tb200_selftest_wait_timeout": (_i, [ctypes.c_uint]),
    "tb200_forward": (_i, [_p] * 8 + [_i] * 5),
    "tb200_backward": (_i, [_p] * 10 + [_i] * 5),
    "tb200_viterbi": (_i, [_p] * 6 + [_i] * 5),
    "tb200_viterbi_static_max_nodes": (_z, []),
    "tb200_viterbi_static": (_i, [_p] * 6 + [_i] * 5),
    "tb200_log_norms_workspace_bytes": (_z, [_i] * 4),
    "tb200_log_norms": (_i, [_p] * 7 + [_i] * 4 + [_p, _z]),
    "tb200_loss_forward_workspace_bytes": (_z, [_i] * 4),
    "tb200_loss_saved_bytes": (_z, [_i] * 4),
    "tb200_loss_forward": (_i, [_p] * 8 + [_z] + [_i] * 5 + [_p, _z]),
    "tb200_loss_forward_bf16": (_i, [_p] * 8 + [_z] + [_i] * 5 + [_p, _z]),
    "tb200_loss_backward_bf16": (_i, [_p] * 6 + [_z] + [_p] * 3 + [_i] * 5 + [_p, _z]),
    "tb200_loss_backward_workspace_bytes": (_z, [_i] * 4),
    "tb200_loss_backward": (_i, [_p] * 6 + [_z] + [_p] * 3 + [_i] * 5 + [_p, _z]),
    "tb200_label_arc_scores_workspace_bytes": (_z, [_i] * 4),
    "tb200_label_arc_scores": (_i, [_p] * 5 + [_i] * 5 + [_p, _z]),
    "tb200_viterbi_decode_workspace_bytes": (_z, [_i] * 4),
    "tb200_viterbi_decode": (_i, [_p] * 5 + [_i] * 5 + [_p, _z]),
    "tb200_peer_slots_bytes": (_z, []),
    "tb200_peer_alloc": (_i, [ctypes.POINTER(_p)]),
    "tb200_peer_free": (_i, [_p]),
    "tb200_peer_export": (_i, [_p, _p]),
    "tb200_peer_import": (_i, [_p, ctypes.POINTER(_p)]),
    "tb200_peer_close": (_i, [_p]),
    "tb200_loss_sum_exchange": (_i, [_p, _p, _i, _i, ctypes.c_uint, _p, ctypes.c_uint]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def check(rc):
    """Raise with the library's message when a C-ABI call did not return 0."""
    if rc != 0:
        raise_for_status(rc, lib.tb200_last_error().decode())


def profile_report():
    """Per-kernel device time recorded since the last reset: {name: (launches, total_ms)}."""
    buf = ctypes.create_string_buffer(1 << 16)
    lib.tb200_profile_report(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out
