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
    """The CUDA library, rebuilt whenever a source is newer than it (nvcc cross-compiles without a
    GPU), so that the tests never run a binary that is older than the code they are meant to hold."""
    import shutil

    from mkharness import driver

    import build as cck_build

    if shutil.which("nvcc"):
        cck_build.build()  # does nothing when the library is up to date
    assert os.path.isfile(driver.PRODUCT_LIB), "libcolabfold_cuda_kernels.so is not built and nvcc is not on PATH"
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
