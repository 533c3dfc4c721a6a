"""The kernel lookup table, as the reference's tests/test_package.py pins it, for the B200 build."""
import ctypes
import os

import pytest

import colabfold_cuda_kernels as cck


def test_diffusion_needs_blackwell():
    assert cck.symbol("diffusion", 100) == "MkSample"
    assert cck.symbol("diffusion", 103) == "MkSample"
    with pytest.raises(FileNotFoundError):
        cck.symbol("diffusion", 90)
    assert not cck.available(90)


def test_unknown_kernel():
    with pytest.raises(KeyError):
        cck.library_path("nope", 120)
    assert not cck.available(120, "nope")


def test_kernels_tuple():
    assert cck.KERNELS == ("diffusion",)
    assert set(cck.__all__) == {"KERNELS", "available", "library_path", "symbol"}


def test_library_name_and_c_abi(product_lib_path):
    path = cck.library_path("diffusion", 100)
    assert os.path.basename(path) == "libcolabfold_cuda_kernels.so"
    assert os.path.samefile(path, product_lib_path)
    lib = ctypes.CDLL(path)
    for kernel in cck.KERNELS:
        getattr(lib, cck.C_ABI[kernel])
