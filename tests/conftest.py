import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLD = os.path.join(ROOT, "tests", "golden")
SCENES = os.path.join(GOLD, "scenes")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_sessionstart(session):
    """Builds the library when it is missing or older than one of its sources (nvcc
    cross-compiles without a GPU), so that no test runs against a stale binary."""
    from bps_nav_b200 import build as _build
    try:
        _build.build()
    except Exception as e:  # the tests that need the library will say so themselves
        sys.stderr.write(f"could not build libbpsn.so: {e}\n")


def scene_path(name):
    return os.path.join(SCENES, f"{name}.navmesh")


def load_scene(name):
    import numpy as np
    from bps_nav_b200.dataset import Scene
    return Scene(scene_path(name), np.load(os.path.join(SCENES, f"{name}.episodes.npy")), f"{name}.glb")


@pytest.fixture(scope="session")
def gold():
    return GOLD
