import glob
import os
import sys

import numpy as np
import pytest

os.environ.setdefault("MVPA_CHECK_STATUS", "1")  # tests read the kernels' status word back

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "multi-variate-parallel-transformer_b200")
for p in (PKG, os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def golden_op_cases():
    return sorted(os.path.basename(f)[3:-4] for f in glob.glob(os.path.join(GOLDEN, "op_*.npz")))


def load_golden(name, kind="op"):
    return dict(np.load(os.path.join(GOLDEN, f"{kind}_{name}.npz")))


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
