import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cpu_harness():
    """g++ build of the per-edge arithmetic headers (tests/cpu_harness.cpp), loaded with ctypes."""
    import ctypes

    build = os.path.join(ROOT, "tests", "_build")
    os.makedirs(build, exist_ok=True)
    so = os.path.join(build, "libcpu_harness.so")
    src = os.path.join(ROOT, "tests", "cpu_harness.cpp")
    deps = [src] + [os.path.join(ROOT, "tace_b200", "csrc", f) for f in ("tace_math.cuh", "tp_gen.cuh", "tace_common.cuh")]
    if not os.path.exists(so) or any(os.path.getmtime(d) > os.path.getmtime(so) for d in deps):
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-o", so, src])
    return ctypes.CDLL(so)
