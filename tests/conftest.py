import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return {name[:-4]: np.load(os.path.join(GOLDEN, name)) for name in os.listdir(GOLDEN) if name.endswith(".npz")}


@pytest.fixture(scope="session")
def oracle_c():
    """The C restatement, built on demand with the committed Makefile."""
    import ctypes
    import subprocess

    odir = os.path.join(ROOT, "oracle")
    so = os.path.join(odir, "libdmm_oracle.so")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(odir, "dmm_oracle.c")):
        subprocess.run(["make", "-C", odir], check=True, capture_output=True)
    return ctypes.CDLL(so)
