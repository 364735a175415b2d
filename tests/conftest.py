import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "golden_v1.npz")
    return dict(np.load(path))


def random_coords(rng, n_per_batch, shape, batch=1):
    """Unique int32 (b,x,y,z) rows, uniformly sampled without replacement per batch item."""
    out = []
    for b in range(batch):
        lin = rng.choice(int(np.prod(shape)), n_per_batch, replace=False)
        xyz = np.stack(np.unravel_index(lin, shape), axis=1)
        out.append(np.concatenate([np.full((n_per_batch, 1), b), xyz], axis=1))
    return np.concatenate(out).astype(np.int32)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(autouse=True)
def _check_kernel_status(request):
    """GPU tests read back the status word of every tensor-core launch (bounded waits report there)."""
    if request.node.get_closest_marker("gpu") is None:
        yield
        return
    from torchsparse_b200 import backend, backends
    old = backend.check_kernel_status
    old_tf32 = backends.allow_tf32
    backend.check_kernel_status = True
    backends.allow_tf32 = False      # fp32 parity is exact fp32; the TF32 tests switch it on themselves
    yield
    backend.check_kernel_status = old
    backends.allow_tf32 = old_tf32
