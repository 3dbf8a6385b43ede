"""Shared fixtures: markers, library loaders, seeded inputs."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GL_P = 0xFFFFFFFF00000001


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import pyoracle
    return pyoracle.load()


@pytest.fixture(scope="session")
def hostcheck():
    """Host build of the library's own field / hash / transcript code."""
    out = os.path.join(ROOT, "tests", "csrc", "_build", "libhost_check.so")
    src = os.path.join(ROOT, "tests", "csrc", "host_check.cu")
    csrc = os.path.join(ROOT, "matrix_b200", "csrc")
    deps = [src] + [os.path.join(dp, f) for dp, _, fs in os.walk(csrc) for f in fs if f.endswith((".cuh", ".hpp"))]
    if not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps):
        os.makedirs(os.path.dirname(out), exist_ok=True)
        subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
                               "-ccbin", "g++", "-I", csrc, "-o", out, src])
    return ctypes.CDLL(out)


from matrix_b200.inputs import splitmix64, field_elems  # noqa: E402,F401
