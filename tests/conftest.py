import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "colabfold-cuda-kernels_b200")
for p in (PKG, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def oracle_lib():
    """The CPU oracle (test infrastructure). Built on demand from oracle/oracle.cpp."""
    from mkharness import driver

    if not os.path.isfile(driver.ORACLE_LIB):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), driver.ORACLE_LIB], check=True)
    return driver.Oracle()


@pytest.fixture(scope="session")
def product_lib_path():
    """The CUDA library. Built on demand (nvcc cross-compiles without a GPU)."""
    from mkharness import driver

    if not os.path.isfile(driver.PRODUCT_LIB):
        import build as cck_build

        cck_build.build()
    return driver.PRODUCT_LIB


_inputs_cache = {}


@pytest.fixture(scope="session")
def make_case():
    """Seeded synthetic inputs, cached per configuration for the session."""
    from mkharness import synth

    def get(n_tok, samples, steps, tiny, seed=0, flags=0, churn=0.0):
        key = (n_tok, samples, steps, tiny, seed, flags, churn)
        if key not in _inputs_cache:
            _inputs_cache[key] = synth.make_inputs(n_tok, samples=samples, steps=steps, seed=seed, tiny=tiny, flags=flags, churn=churn)
        return _inputs_cache[key]

    return get
