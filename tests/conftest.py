import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def load_golden(name):
    """npz -> dict of torch tensors; keys ending in __bf16 are decoded to torch.bfloat16."""
    import torch
    z = np.load(os.path.join(GOLDEN, name))
    out = {}
    for k in z.files:
        a = z[k]
        if k.endswith("__bf16"):
            out[k[:-6]] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        elif a.dtype.kind in "fiub":
            out[k] = torch.from_numpy(np.ascontiguousarray(a)) if a.ndim else a
        else:
            out[k] = a
    return out


@pytest.fixture(scope="session")
def golden():
    cache = {}

    def get(name):
        if name not in cache:
            cache[name] = load_golden(name)
        return cache[name]
    return get


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def reference():
    """The reference package itself, from oracle/_ref (placed there by `python oracle/make_ref.py`; it ships
    with the working tree but is never committed).  Tests that need it are skipped when it is absent."""
    from oracle import make_ref
    try:
        return make_ref.import_reference()
    except ImportError as ex:
        pytest.skip(str(ex))
