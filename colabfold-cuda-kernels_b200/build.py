"""Builds libcolabfold_cuda_kernels.so for sm_100a in-tree, next to the Python lookup package.

    python colabfold-cuda-kernels_b200/build.py [--force]
    python colabfold-cuda-kernels_b200/build.py --diag CCK_TRACE=1 [--diag CCK_STAGE_REC=1] -o PATH

The second form builds a diagnostics variant of the same sources somewhere else (event trace of one CTA,
stage records): never the library that the lookup package hands out.

Set CCK_FFI_INCLUDE_DIR to a directory holding xla/ffi/api/ffi.h to also compile the XLA FFI handler
`MkSample` (csrc/ffi_handler.cu); without it the library exports the plain C ABI only.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "colabfold_cuda_kernels", "libcolabfold_cuda_kernels.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    """Everything the library is built from: an edit to any of it makes the built library stale."""
    src = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh")))
    return src + [os.path.join(os.path.dirname(HERE), "include", "cck_b200.h"), os.path.abspath(__file__)]


def up_to_date():
    if not os.path.isfile(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(s) <= t for s in sources())


def build(force=False, verbose=False, out=None, defines=()):
    if out is None and defines:
        raise ValueError("a diagnostics variant needs a path of its own")
    if out is None and not force and up_to_date():
        return OUT
    OUT_ = out or OUT
    cmd = ["nvcc", "-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr"] + ARCH + ["-D" + d for d in defines]
    # libc and libm only at run time, as the reference's library (its CI audits that with ldd): the CUDA
    # runtime is linked statically by nvcc's default, the C++ runtime and libgcc by these flags
    cmd += ["-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-static-libstdc++", "-Xcompiler", "-static-libgcc"]
    cmd += ["-o", OUT_, os.path.join(CSRC, "cck_b200.cu")]
    ffi = os.environ.get("CCK_FFI_INCLUDE_DIR")
    if ffi:
        cmd += ["-DCCK_FFI", "-I", ffi, os.path.join(CSRC, "ffi_handler.cu")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    subprocess.run(cmd, check=True, cwd=CSRC)
    return OUT_


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", dest="verbose", action="store_true")
    ap.add_argument("--diag", action="append", default=[], metavar="NAME=VALUE")
    ap.add_argument("-o", dest="out", default=None)
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, out=os.path.abspath(a.out) if a.out else None, defines=a.diag))
