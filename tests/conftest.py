import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "3d-deformable-attention_b200")
for p in (PKG_DIR, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests"),
          os.path.join(ROOT, "tests", "golden"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib_built():
    """Make sure libdfa3d_b200.so exists (nvcc cross-compiles without a GPU)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("dfa3d_build", os.path.join(PKG_DIR, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def pytest_sessionfinish(session, exitstatus):
    """With DFA3D_TOL_STATS=<file>: dump what helpers.assert_close recorded about its tolerances."""
    path = os.environ.get("DFA3D_TOL_STATS")
    if path:
        import json
        import helpers
        with open(path, "w") as f:
            json.dump(helpers.TOL_STATS, f, indent=1)
