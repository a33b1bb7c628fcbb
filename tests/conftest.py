import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    """Load a fixture; `*_bf16` entries (raw bit patterns) come back as torch bf16
    tensors without the suffix, the rest as torch tensors of their own dtype."""
    data = np.load(GOLDEN / f"{name}.npz")
    out = {}
    for key in data.files:
        array = data[key]
        if key.endswith("_bf16"):
            out[key[:-5]] = torch.from_numpy(array.copy()).view(torch.bfloat16)
        elif array.shape == ():
            out[key] = float(array)
        else:
            out[key] = torch.from_numpy(array.copy())
    return out


def rel_l2(actual, expected):
    actual, expected = actual.double(), expected.double()
    return float((actual - expected).norm() / expected.norm().clamp_min(1e-30))


def max_err_ratio(actual, expected):
    """max|err| / max|ref| -- the forward-output bar (<= 1e-2)."""
    actual, expected = actual.double(), expected.double()
    return float((actual - expected).abs().max() / expected.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="session")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from dscuda_b200 import mla
    yield torch.device("cuda:0")
    # every GPU test module must leave the kernels' status word clean
    assert mla.device_status(reset=True) == 0, "a kernel reported a bounded-wait timeout"
