import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "oracle") not in sys.path:
    sys.path.insert(0, str(ROOT / "oracle"))   # oracle_lib: the CPU checker's bindings


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _native_built():
    """Build whatever is out of date once per session (seconds; nvcc cross-compiles without a GPU)."""
    from dphpc_b200 import build as pkg_build

    sys.path.insert(0, str(ROOT / "oracle"))
    import importlib.util

    spec = importlib.util.spec_from_file_location("oracle_build", ROOT / "oracle" / "build.py")
    ob = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ob)
    ob.build_oracle()
    ob.build_ref()
    pkg_build.build_datasets()
    pkg_build.build_engine()
    ob.build_ref_harness()   # (needs the engine library; only where the reference checkout is present)
    yield


@pytest.fixture(scope="session")
def oracle():
    import oracle_lib

    return oracle_lib.Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU path (oracle/_ref); skipped where it was never built."""
    import oracle_lib

    r = oracle_lib.Reference.try_load()
    if r is None:
        pytest.skip("oracle/_ref/libsddmm_ref.so not built (reference checkout absent)")
    return r


def has_gpu() -> bool:
    try:
        from dphpc_b200 import device_count

        return device_count() > 0
    except Exception:
        return False
