import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def golden():
    return json.loads((ROOT / "tests" / "golden" / "reference_vectors.json").read_text())


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def built_lib():
    """The CUDA library, built in-tree if it is not there yet (nvcc cross-compiles without a GPU)."""
    from webllm_b200 import build
    return build.build()


@pytest.fixture(scope="module")
def gpu(built_lib):
    """A fresh context per test module. Fails (does not skip) when the library or the GPU is missing:
    a silent fallback would hide that the CUDA path did not run."""
    from webllm_b200 import Gpu
    g = Gpu(0, weight_bytes=2 << 30, act_bytes=1 << 30)
    yield g
    g.close()


def bits_to_f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)
