import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: torch.from_numpy(z[k]) if z[k].shape != () else (float(z[k]) if z[k].dtype.kind == 'f' else int(z[k]))
                for k in z.files}


def unpack_had(bits, K):
    """+-1 fp32 matrix from the bit-packed fixture (1 bit per entry, set = +1)."""
    b = np.unpackbits(np.asarray(bits, dtype=np.uint8))[: K * K].reshape(K, K)
    return torch.from_numpy(b.astype(np.float32) * 2 - 1)


def rel_to_norm(y, ref):
    """max|y - ref| / ||ref||_2 : the error measure of the fp16 output tolerance."""
    return ((y.double() - ref.double()).abs().max() / ref.double().norm().clamp_min(1e-30)).item()
