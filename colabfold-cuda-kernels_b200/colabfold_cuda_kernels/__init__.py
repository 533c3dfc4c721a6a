"""Kernel lookup for the B200 build of colabfold-cuda-kernels.

Same four names and the same behaviour as the reference package
(python/colabfold_cuda_kernels/__init__.py:18-58): callers ask for a kernel by name and compute
capability and get the shared library's path and the XLA FFI target name to register. This build
carries sm_100a code for the diffusion sampler only, so every lookup below compute capability 100
fails the way the reference fails below its own minimum.
"""
import os

__all__ = ["KERNELS", "available", "library_path", "symbol"]
__version__ = "0.2.1+b200"

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBRARY = os.path.join(_HERE, "libcolabfold_cuda_kernels.so")

# name -> (lowest compute capability served, XLA FFI target name)
_KERNEL_TABLE = {"diffusion": (100, "MkSample")}
KERNELS = tuple(_KERNEL_TABLE)

# plain C entry point behind each FFI target, for callers without XLA
C_ABI = {"diffusion": "cck_mk_sample"}


def symbol(kernel, cc):
    """XLA FFI target name of `kernel`; KeyError for an unknown kernel, FileNotFoundError when the
    compute capability is too old."""
    try:
        lowest, name = _KERNEL_TABLE[kernel]
    except KeyError:
        raise KeyError("unknown kernel %r, expected one of %s" % (kernel, ", ".join(KERNELS))) from None
    if int(cc) < lowest:
        raise FileNotFoundError("no %s kernel for compute capability %d (needs %d+)" % (kernel, int(cc), lowest))
    return name


def library_path(kernel, cc):
    """Path of the shared library that holds `kernel`."""
    symbol(kernel, cc)
    if not os.path.isfile(_LIBRARY):
        raise FileNotFoundError("%s is not in this package" % _LIBRARY)
    return _LIBRARY


def available(cc, kernel=None):
    """True if the library is present and serves `kernel` (all kernels when None) at `cc`."""
    for name in KERNELS if kernel is None else (kernel,):
        try:
            library_path(name, cc)
        except (FileNotFoundError, KeyError):
            return False
    return True
