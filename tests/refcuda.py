"""Loaders for the reference's own CUDA wrappers, compiled test-only.

`make -C oracle refcuda` compiles goldilocks-cuda-rs/cuda/wrapper.cu and
almost-goldilocks-cuda-rs/cuda/wrapper.cu (with the header trees they include)
for sm_100a into oracle/_ref/. They export the same symbol names as this
package's libraries, so each is opened in its own namespace (RTLD_LOCAL) and
bound with the same signature tables. Test infrastructure only: nothing in
the package or in a timed region loads them.
"""
import ctypes
import os

import numpy as np
import pytest

from matrix_b200 import ffi

HERE = os.path.dirname(os.path.abspath(__file__))
REFDIR = os.path.join(os.path.dirname(HERE), "oracle", "_ref")

GL_P = 0xFFFFFFFF00000001
AGL_Q = 0xFFFFFFFEFFFFFFE1  # 2^64 - 2^32 - 31

_cache = {}


def _open(name, sigs):
    if name in _cache:
        return _cache[name]
    path = os.path.join(REFDIR, name)
    if not os.path.exists(path):
        pytest.skip("%s not built (make -C oracle refcuda needs the reference tree)" % name)
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    for fn_name, (res, args) in sigs.items():
        try:
            fn = getattr(lib, fn_name)
        except AttributeError:
            continue  # an addition of this package: not in the reference
        fn.restype = res
        fn.argtypes = args
    _cache[name] = lib
    return lib


def ref_gl():
    """The reference's Goldilocks wrapper, initialised (field, Poseidon2 and Monolith constants)."""
    lib = _open("libgl_ref_cuda.so", ffi.gl_signatures())
    assert lib.goldilocks_cuda_init() == 0
    assert lib.poseidon2_cuda_init() == 0
    assert lib.monolith_cuda_init() == 0
    return lib


def ref_agl():
    """The reference's almost-Goldilocks wrapper, initialised."""
    sigs = ffi.agl_signatures()
    gl = ffi.gl_signatures()
    for name in ("cuda_malloc", "cuda_free", "cuda_memcpy_htod", "cuda_memcpy_dtoh", "cuda_memcpy_dtod",
                 "cuda_device_synchronize", "cuda_get_last_error", "cuda_set_device"):
        sigs[name] = gl[name]
    lib = _open("libagl_ref_cuda.so", sigs)
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


class Buf:
    """Device memory from a library's own cuda_malloc; synchronises the device around copies because the
    reference's entry points return without waiting for their kernels."""

    def __init__(self, lib, nbytes):
        self.lib = lib
        self.nbytes = max(int(nbytes), 8)
        p = ctypes.c_void_p()
        assert lib.cuda_malloc(ctypes.byref(p), self.nbytes) == 0
        self.ptr = p.value
        zero = np.zeros(self.nbytes, dtype=np.uint8)
        assert lib.cuda_memcpy_htod(self.ptr, zero.ctypes.data, self.nbytes) == 0

    @classmethod
    def of(cls, lib, arr):
        arr = np.ascontiguousarray(arr)
        b = cls(lib, arr.nbytes)
        if arr.nbytes:
            assert lib.cuda_memcpy_htod(b.ptr, arr.ctypes.data, arr.nbytes) == 0
        return b

    def get(self, dtype=np.uint64, count=None):
        assert self.lib.cuda_device_synchronize() == 0
        dt = np.dtype(dtype)
        if count is None:
            count = self.nbytes // dt.itemsize
        out = np.empty(count, dtype=dt)
        assert self.lib.cuda_memcpy_dtoh(out.ctypes.data, self.ptr, out.nbytes) == 0
        return out

    def __del__(self):
        try:
            if self.ptr:
                self.lib.cuda_device_synchronize()
                self.lib.cuda_free(self.ptr)
                self.ptr = 0
        except Exception:
            pass


def canon(arr, mod):
    """Words as canonical residues: the reference leaves values anywhere in [0, 2^64)."""
    a = np.asarray(arr, dtype=np.uint64)
    return np.where(a >= np.uint64(mod), a - np.uint64(mod), a)


def sum_rows(partials, rows, width, mod):
    """Adds per-block partial rows on the host, as the reference's Rust drivers do."""
    part = np.asarray(partials[:rows * width], dtype=np.uint64).reshape(rows, width)
    return np.array([sum(int(x) for x in part[:, k]) % mod for k in range(width)], dtype=np.uint64)
