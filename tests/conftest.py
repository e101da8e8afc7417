"""Shared pytest configuration: the `gpu` marker, import paths and fixture loading."""
from __future__ import annotations

import glob
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


def golden_cases():
    return sorted(glob.glob(os.path.join(GOLDEN, "case_*.npz")))


def load_case(path):
    z = np.load(path)
    d = {k: z[k] for k in z.files}
    for k in ("M", "N", "r", "T", "G"):
        d[k] = int(d[k])
    d["packed"] = {k: d[k] for k in ("U_codes", "U_scale", "U_zero", "Vt_codes", "Vt_scale", "Vt_zero")}
    return d


@pytest.fixture(params=golden_cases(), ids=lambda p: os.path.basename(p)[5:-4])
def case(request):
    return load_case(request.param)
