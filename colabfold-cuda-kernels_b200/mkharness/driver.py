"""ctypes drivers: the sampler library's debug C ABI (mk_*) and, for tests and baselines only, the
CPU oracle's matching C ABI (orc_*).

`MkLib` speaks the interface the reference exports for stand-alone driving
(src/diffusion/host.cuh:376-499), so the same class drives this repository's library and a build of
the reference kernel. One library instance holds one global state, as in the reference.
"""
import ctypes
import os

import numpy as np

from . import synth

_HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(_HERE))
PRODUCT_LIB = os.path.join(os.path.dirname(_HERE), "colabfold_cuda_kernels", "libcolabfold_cuda_kernels.so")
ORACLE_LIB = os.path.join(ROOT, "oracle", "liboracle.so")
REFERENCE_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_sm100.so")

BF16_BUFS = {"SCT", "SCLN0", "SCBF", "SCH", "MODS", "AO", "ABF", "AQG", "AKV", "TX", "TX2", "QKVG", "TO", "TC", "PLG"}


def _ptr_array(arrays):
    ptrs = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    sizes = (ctypes.c_size_t * len(arrays))(*[a.nbytes for a in arrays])
    return ptrs, sizes


class MkLib:
    """The mk_* debug API of a sampler library (this repository's, or the reference's)."""

    def __init__(self, path=PRODUCT_LIB):
        if not os.path.isfile(path):
            raise FileNotFoundError("%s is not built" % path)
        self.path = path
        lib = self.lib = ctypes.CDLL(path)
        lib.mk_setup.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p, ctypes.c_void_p]
        lib.mk_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p,
                               ctypes.c_float, ctypes.POINTER(ctypes.c_float), ctypes.c_void_p]
        lib.mk_read.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t]
        lib.mk_buf_id.argtypes = [ctypes.c_char_p]
        lib.mk_buf_bytes.argtypes = [ctypes.c_int]
        lib.mk_buf_bytes.restype = ctypes.c_size_t
        lib.mk_workspace_bytes.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p]
        lib.mk_workspace_bytes.restype = ctypes.c_size_t
        lib.mk_timing_names.restype = ctypes.c_char_p
        lib.mk_gemm_test.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 4
        lib.mk_teardown.restype = None
        self.meta = None

    def setup(self, inputs, meta):
        self._keep = inputs
        ptrs, sizes = _ptr_array(inputs)
        rc = self.lib.mk_setup(meta["S"], meta["N"], meta["A"], meta["NS"], meta["steps"], ptrs, sizes)
        if rc != 0:
            raise RuntimeError("mk_setup failed (%d)" % rc)
        self.meta = meta

    def set_extent(self, n_tokens, n_subsets):
        """Real extents of the next runs inside the bucket given to setup (this library only)."""
        if self.lib.mk_set_extent(n_tokens, n_subsets) != 0:
            raise RuntimeError("mk_set_extent refused (%d, %d)" % (n_tokens, n_subsets))

    def set_flow(self, on):
        """Token-block chains on completion counters (True, the default) or on grid barriers (this
        library only). Returns the previous setting."""
        return bool(self.lib.mk_set_flow(1 if on else 0))

    def workspace_bytes(self, inputs, meta, nsteps, flags=0):
        _, sizes = _ptr_array(inputs)
        return self.lib.mk_workspace_bytes(meta["S"], meta["N"], meta["NS"], nsteps, flags, sizes)

    def run(self, mode=0, nsteps=0, dbg_stop=0, seed=0, xn=None, t=0.0, timing=False):
        """Returns the event-timed milliseconds of the launch; with timing=True, also a dict
        kind -> (wall ms, phases) of the library's per-phase-kind record."""
        ms = ctypes.c_float(0)
        xp = None
        if xn is not None:
            xn = np.ascontiguousarray(xn, dtype=np.float32)
            xp = xn.ctypes.data
        names = [n for n in self.lib.mk_timing_names().decode().split(",") if n]
        words = np.zeros(max(3 * len(names), 1), dtype=np.uint64)
        rc = self.lib.mk_run(mode, nsteps, dbg_stop, ctypes.c_uint64(seed), xp, ctypes.c_float(t), ctypes.byref(ms),
                             words.ctypes.data if timing else None)
        if rc != 0:
            raise RuntimeError("mk_run failed (%d)" % rc)
        if timing:
            return ms.value, {n: (words[2 * i] * 1e-6, int(words[2 * i + 1])) for i, n in enumerate(names)}
        return ms.value

    def read(self, name):
        """A scratch buffer as float32 (bf16 buffers are widened)."""
        bid = self.lib.mk_buf_id(name.encode())
        if bid < 0:
            raise KeyError(name)
        nbytes = self.lib.mk_buf_bytes(bid)
        raw = np.empty(nbytes, dtype=np.uint8)
        if self.lib.mk_read(bid, raw.ctypes.data, nbytes) != 0:
            raise RuntimeError("mk_read(%s) failed" % name)
        if name in BF16_BUFS:
            return synth.from_bf16(raw.view(np.uint16))
        return raw.view(np.float32)

    def gemm_test(self, a_bf, w_bf, tile=0):
        M, K = a_bf.shape
        N = w_bf.shape[0]
        c = np.empty((M, N), dtype=np.float32)
        a_bf = np.ascontiguousarray(a_bf)
        w_bf = np.ascontiguousarray(w_bf)
        rc = self.lib.mk_gemm_test(a_bf.ctypes.data, w_bf.ctypes.data, c.ctypes.data, M, N, K, tile)
        if rc != 0:
            raise RuntimeError("mk_gemm_test failed (%d)" % rc)
        return c

    def teardown(self):
        self.lib.mk_teardown()


class Oracle:
    """The CPU restatement. Test infrastructure: never imported by the product path."""

    def __init__(self, path=ORACLE_LIB):
        if not os.path.isfile(path):
            raise FileNotFoundError("%s is not built (make -C oracle)" % path)
        lib = self.lib = ctypes.CDLL(path)
        lib.orc_setup.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p, ctypes.c_void_p]
        lib.orc_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p,
                                ctypes.c_float, ctypes.c_int]
        lib.orc_buf_count.argtypes = [ctypes.c_char_p]
        lib.orc_buf_count.restype = ctypes.c_size_t
        lib.orc_read.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t]
        lib.orc_read_pair.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.orc_philox.argtypes = [ctypes.c_uint32] * 4 + [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
        lib.orc_rigid.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
        lib.orc_to_bf.argtypes = [ctypes.c_float]
        lib.orc_to_bf.restype = ctypes.c_uint16
        lib.orc_gemm.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3
        lib.orc_apl_index.argtypes = [ctypes.c_int] * 7
        lib.orc_apl_index.restype = ctypes.c_size_t
        lib.orc_teardown.restype = None
        lib.orc_set_threads.argtypes = [ctypes.c_int]
        lib.orc_set_threads.restype = None
        lib.orc_snapshot.argtypes = [ctypes.c_int, ctypes.c_char_p]
        lib.orc_snapshot.restype = None
        self.meta = None

    def set_threads(self, n=0):
        """OpenMP threads of the following calls (0: all processors); returns what is in effect."""
        self.lib.orc_set_threads(int(n))
        return self.lib.orc_threads()

    def snapshot(self, phase, name):
        """Keep buffer `name` as it is when phase `phase` ends; read it back as "name@phase"."""
        self.lib.orc_snapshot(phase, name.encode())

    def clear_snapshots(self):
        self.lib.orc_snapshot(-1, b"")

    def setup(self, inputs, meta):
        ptrs, sizes = _ptr_array(inputs)
        rc = self.lib.orc_setup(meta["S"], meta["N"], meta["A"], meta["NS"], meta["steps"], ptrs, sizes)
        if rc != 0:
            raise RuntimeError("orc_setup failed")
        self.meta = meta

    def run(self, mode=0, nsteps=0, dbg_stop=0, seed=0, xn=None, t=0.0, precise=False):
        xp = None
        if xn is not None:
            xn = np.ascontiguousarray(xn, dtype=np.float32)
            xp = xn.ctypes.data
        rc = self.lib.orc_run(mode, nsteps, dbg_stop, ctypes.c_uint64(seed), xp, ctypes.c_float(t), int(precise))
        if rc != 0:
            raise RuntimeError("orc_run failed")

    def read(self, name):
        n = self.lib.orc_buf_count(name.encode())
        if n == 0:
            raise KeyError(name)
        out = np.empty(n, dtype=np.float32)
        if self.lib.orc_read(name.encode(), out.ctypes.data, n) != 0:
            raise RuntimeError("orc_read(%s) failed" % name)
        return out

    def read_pair(self, b, head):
        N = self.meta["N"]
        out = np.empty((N, N), dtype=np.float32)
        self.lib.orc_read_pair(b, head, out.ctypes.data)
        return out

    def philox(self, idx, step, sample, stream, seed):
        w = np.empty(4, dtype=np.uint32)
        z = np.empty(4, dtype=np.float32)
        self.lib.orc_philox(idx, step, sample, stream, ctypes.c_uint64(seed), w.ctypes.data, z.ctypes.data)
        return w, z

    def gemm(self, a_bf, w_bf):
        M, K = a_bf.shape
        N = w_bf.shape[0]
        c = np.empty((M, N), dtype=np.float32)
        a_bf = np.ascontiguousarray(a_bf)
        w_bf = np.ascontiguousarray(w_bf)
        self.lib.orc_gemm(a_bf.ctypes.data, w_bf.ctypes.data, c.ctypes.data, M, N, K)
        return c

    def teardown(self):
        self.lib.orc_teardown()


def max_rel_err(a, b):
    """max |a - b| over max |b|: the error measure of the parity gates."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def rms_rel_err(a, b):
    """RMS(a - b) over RMS(b): a second figure beside the global maximum, which a few large entries of
    a buffer cannot dominate the way they dominate max |b|."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.sqrt(np.mean((a - b) ** 2)) / max(np.sqrt(np.mean(b ** 2)), 1e-30))
