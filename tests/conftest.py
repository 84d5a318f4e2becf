import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def lib():
    # building is cheap when the library is current; it needs nvcc, not a GPU
    import importlib

    build = importlib.import_module("neurips26-tris-moe_b200.build")
    build.build()
    import trismoe_b200

    return trismoe_b200._native.load()


_RUNTIME_SWITCHES = ("TRIS_GROUPED_EXPERTS", "OLMOE_GROUPED_EXPERTS", "TRIS_DEPLOYMENT_ONLY", "OLMOE_DEPLOYMENT_ONLY",
                     "TRIS_COMPACT3_BLOCK_GR", "TRIS_GROUPED_QGMAP_CPU_STAGING", "OLMOE_GROUPED_QGMAP_CPU_STAGING",
                     "MIXTRAL_GROUPED_QGMAP_CPU_STAGING", "TRIS_PACKED4_BACKBONE")


@pytest.fixture(autouse=True)
def default_runtime_switches(monkeypatch):
    """The tests describe the default behaviour: environment switches a shell may carry are taken out
    (tests of the switches set them themselves)."""
    for name in _RUNTIME_SWITCHES:
        monkeypatch.delenv(name, raising=False)
