import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return entry.package()


@pytest.fixture(scope="session")
def syn(pkg):
    return pkg.synth


@pytest.fixture(scope="session")
def orc_mod():
    mod = entry.oracle_module()
    mod.build(ref=True)
    return mod


@pytest.fixture(scope="session")
def orc(orc_mod):
    return orc_mod.Oracle()


@pytest.fixture(scope="session")
def ref(orc_mod):
    """The reference's own dequantisers, where oracle/_ref could be built."""
    if not orc_mod.Reference.available():
        pytest.skip("reference header not found - restated oracle only")
    return orc_mod.Reference()


@pytest.fixture(scope="session")
def ref_layer(orc_mod):
    """The reference's own CPU layer loop (moeCpuRef), where oracle/_ref could be built."""
    if not orc_mod.ReferenceLayer.available():
        pytest.skip("reference source not found - restated layer loop only")
    return orc_mod.ReferenceLayer()


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name))
    return load


def has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
