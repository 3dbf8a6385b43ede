"""The block cache behind cuda_malloc / cuda_free (contract of the reference's allocator,
almost-goldilocks-cuda-rs/cuda/wrapper.cu:118-235): reuse of a freed block by a request that fits,
no reuse by a much smaller request, release on flush and on cuda_pool_trim, plain behaviour with
AGL_ALLOC_CACHE=0, and data integrity across reuse."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

from matrix_b200.ffi import load_agl, load_gl

pytestmark = pytest.mark.gpu
MiB = 1 << 20


def _malloc(lib, n):
    p = ctypes.c_void_p()
    assert lib.cuda_malloc(ctypes.byref(p), n) == 0
    return p.value


@pytest.mark.parametrize("loader", [load_gl, load_agl], ids=["gl", "agl"])
def test_reuse_fit_rule_and_flush(loader):
    lib = loader()
    assert lib.mb_alloc_cache_flush() == 0
    base = lib.mb_alloc_cache_bytes()
    assert base == 0
    a = _malloc(lib, 64 * MiB)
    data = np.arange(1 << 16, dtype=np.uint64)
    assert lib.cuda_memcpy_htod(a, data.ctypes.data, data.nbytes) == 0
    assert lib.cuda_free(a) == 0
    assert lib.mb_alloc_cache_bytes() == 64 * MiB
    small = _malloc(lib, 1 * MiB)            # 64 MiB is more than 25 % + 2 MiB above the request: not taken
    assert small != a and lib.mb_alloc_cache_bytes() == 64 * MiB
    b = _malloc(lib, 60 * MiB)               # fits: the cached block comes back
    assert b == a and lib.mb_alloc_cache_bytes() == 0
    back = np.zeros_like(data)
    data2 = data[::-1].copy()
    assert lib.cuda_memcpy_htod(b, data2.ctypes.data, data2.nbytes) == 0
    assert lib.cuda_memcpy_dtoh(back.ctypes.data, b, back.nbytes) == 0
    assert np.array_equal(back, data2)
    assert lib.cuda_free(b) == 0 and lib.cuda_free(small) == 0
    assert lib.mb_alloc_cache_bytes() == 65 * MiB
    assert lib.mb_alloc_cache_flush() == 0 and lib.mb_alloc_cache_bytes() == 0
    # the empty buffer and the null pointer
    z = ctypes.c_void_p()
    assert lib.cuda_malloc(ctypes.byref(z), 0) == 0 and lib.cuda_free(z) == 0 and lib.cuda_free(None) == 0
    assert lib.mb_alloc_cache_flush() == 0


def test_pool_trim_releases_the_cache():
    lib = load_agl()
    p = _malloc(lib, 8 * MiB)
    assert lib.cuda_free(p) == 0 and lib.mb_alloc_cache_bytes() >= 8 * MiB
    assert lib.cuda_pool_trim(0) == 0 and lib.mb_alloc_cache_bytes() == 0


def test_many_small_buffers_cycle_without_growth():
    lib = load_agl()
    lib.mb_alloc_cache_flush()
    seen = set()
    for i in range(200):
        ps = [_malloc(lib, 4096 * (1 + (i + k) % 3)) for k in range(4)]
        seen.update(ps)
        for p in ps:
            assert lib.cuda_free(p) == 0
    assert len(seen) <= 12 and lib.mb_alloc_cache_bytes() <= 12 * 3 * 4096
    lib.mb_alloc_cache_flush()


def test_switch_restores_plain_allocation():
    code = ("import ctypes\nfrom matrix_b200.ffi import load_agl\nlib = load_agl()\np = ctypes.c_void_p()\n"
            "assert lib.cuda_malloc(ctypes.byref(p), 1 << 20) == 0\nassert lib.cuda_free(p) == 0\n"
            "assert lib.mb_alloc_cache_bytes() == 0\nprint('plain')\n")
    env = dict(os.environ, AGL_ALLOC_CACHE="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "plain" in out.stdout, out.stderr


def test_concurrent_threads_never_share_a_block():
    """The reference's callers are rayon workers: several host threads allocate and drop buffers at once. Each
    thread writes its own pattern into every buffer it holds and reads it back after the others had time to
    allocate: a block handed to two owners would show the wrong pattern."""
    import threading
    lib = load_agl()
    errors = []

    def worker(tid):
        try:
            lib.cuda_set_device(0)
            rng = np.random.default_rng(tid)
            for it in range(60):
                sizes = [int(rng.integers(1, 64)) * 4096 for _ in range(3)]
                held = []
                for k, n in enumerate(sizes):
                    p = _malloc(lib, n)
                    pat = np.full(n // 8, (tid << 32) | (it << 8) | k, dtype=np.uint64)
                    assert lib.cuda_memcpy_htod(p, pat.ctypes.data, pat.nbytes) == 0
                    held.append((p, pat))
                for p, pat in held:
                    back = np.empty_like(pat)
                    assert lib.cuda_memcpy_dtoh(back.ctypes.data, p, back.nbytes) == 0
                    assert np.array_equal(back, pat)
                    assert lib.cuda_free(p) == 0
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(t + 1,)) for t in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert lib.mb_alloc_cache_flush() == 0
