import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(GOLDEN, "reference_kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def reference_runs():
    """name -> dict of arrays produced by the reference's CPU path (see make_golden.py)."""
    z = np.load(os.path.join(GOLDEN, "reference_runs.npz"))
    out = {}
    for key in z.files:
        case, field = key.split("/")
        out.setdefault(case, {})[field] = z[key]
    return out


def kat_arrays(k):
    """Reshape one forward/backward known-answer group into batched arrays."""
    V = k["V"]
    il = np.asarray(k["input_lengths"], np.int32)
    ll = np.asarray(k["label_lengths"], np.int32)
    B, T, U = len(il), int(il.max()), int(ll.max()) + 1
    E = np.asarray(k["emissions"], np.float32).reshape(B, T, V)
    P = np.asarray(k["predictions"], np.float32).reshape(B, U, V)
    labels = np.asarray(k["labels"], np.int32).reshape(B, U - 1)
    return dict(E=E, P=P, labels=labels, in_lens=il, lab_lens=ll,
                costs=np.asarray(k["costs"], np.float32),
                egrads=np.asarray(k["egrads"], np.float32).reshape(B, T, V),
                pgrads=np.asarray(k["pgrads"], np.float32).reshape(B, U, V))
