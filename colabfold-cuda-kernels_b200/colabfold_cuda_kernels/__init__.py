"""Kernel lookup for the B200 build of colabfold-cuda-kernels.

The four names and their behaviour are the reference package's
(python/colabfold_cuda_kernels/__init__.py:18-58): a caller names a kernel and a compute capability
and gets the shared library's path and the XLA FFI target to register; KeyError for a name the
package has never heard of, FileNotFoundError for a kernel it knows but cannot serve. This build
holds sm_100a machine code for the diffusion sampler and nothing else: such code runs on compute
capability 10.0 only (no PTX travels with it), so every other capability is refused, and the
reference's second kernel, fp8_contract, is known by name but not built.
"""
import os

__all__ = ["KERNELS", "available", "library_path", "symbol"]
__version__ = "0.2.1+b200"

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBRARY = os.path.join(_HERE, "libcolabfold_cuda_kernels.so")

# name -> (compute capabilities served, XLA FFI target name); the names and targets are the reference's
_KERNEL_TABLE = {
    "diffusion": ((100,), "MkSample"),
    "fp8_contract": ((), "CckFp8Contract"),
}
KERNELS = tuple(_KERNEL_TABLE)

# plain C entry point behind each FFI target that is built, for callers without XLA
C_ABI = {"diffusion": "cck_mk_sample"}


def symbol(kernel, cc):
    """XLA FFI target name of `kernel` at compute capability `cc` (major * 10 + minor)."""
    if kernel not in _KERNEL_TABLE:
        raise KeyError("unknown kernel %r, expected one of %s" % (kernel, ", ".join(KERNELS)))
    served, name = _KERNEL_TABLE[kernel]
    if not served:
        raise FileNotFoundError("%s is not built in the B200 library" % kernel)
    if int(cc) not in served:
        raise FileNotFoundError("no %s kernel for compute capability %d: this build holds sm_100a code (compute capability %s)"
                                % (kernel, int(cc), ", ".join(str(c) for c in served)))
    return name


def library_path(kernel, cc):
    """Path of the shared library that holds `kernel`."""
    symbol(kernel, cc)
    if not os.path.isfile(_LIBRARY):
        raise FileNotFoundError("%s is not in this package" % _LIBRARY)
    return _LIBRARY


def available(cc, kernel=None):
    """True if the library is present and serves `kernel` at `cc`; with kernel=None, every kernel of
    KERNELS (False here, since fp8_contract is not built: ask for "diffusion")."""
    for name in KERNELS if kernel is None else (kernel,):
        try:
            library_path(name, cc)
        except (FileNotFoundError, KeyError):
            return False
    return True
