"""The kernel lookup table, as the reference's tests/test_package.py pins it, for the B200 build."""
import ctypes
import os
import subprocess

import pytest

import colabfold_cuda_kernels as cck


def test_diffusion_needs_compute_capability_10_0():
    assert cck.symbol("diffusion", 100) == "MkSample"
    for cc in (80, 90, 103, 120):  # sm_100a machine code runs on 10.0 only
        with pytest.raises(FileNotFoundError):
            cck.symbol("diffusion", cc)
        assert not cck.available(cc, "diffusion")


def test_unknown_kernel():
    with pytest.raises(KeyError):
        cck.library_path("nope", 100)
    assert not cck.available(100, "nope")


def test_second_kernel_is_known_but_not_built():
    """A caller of the reference handles a kernel the package cannot serve by catching
    FileNotFoundError (its contract for a too old GPU): the same here for fp8_contract."""
    assert cck.KERNELS == ("diffusion", "fp8_contract")
    for f in (cck.symbol, cck.library_path):
        with pytest.raises(FileNotFoundError):
            f("fp8_contract", 100)
    assert not cck.available(100, "fp8_contract")
    assert not cck.available(100)  # "all kernels"
    assert set(cck.__all__) == {"KERNELS", "available", "library_path", "symbol"}


def test_library_name_and_c_abi(product_lib_path):
    path = cck.library_path("diffusion", 100)
    assert os.path.basename(path) == "libcolabfold_cuda_kernels.so"
    assert os.path.samefile(path, product_lib_path)
    lib = ctypes.CDLL(path)
    for kernel, entry in cck.C_ABI.items():
        assert cck.available(100, kernel)
        getattr(lib, entry)


def test_library_needs_libc_only(product_lib_path):
    """The reference links its library against libc alone (static CUDA and C++ runtimes,
    src/CMakeLists.txt:76-89) and its CI checks that with ldd: the same here."""
    out = subprocess.run(["ldd", product_lib_path], capture_output=True, text=True).stdout
    needed = {line.split()[0].split(".so")[0] for line in out.splitlines() if "=>" in line}
    assert needed <= {"libc", "libm", "libdl", "libpthread", "librt"}, out
