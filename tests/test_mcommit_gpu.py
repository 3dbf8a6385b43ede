"""GPU parity of the exact module commitment (transform-domain key cache, partial, add, finish)
against the CPU oracle's schoolbook integers, through the C-ABI. Bit-exact.
Shapes follow zk-torch-4/src/morpheus/commit_gpu.rs:104-168."""
import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from oracle import pyoracle as po

pytestmark = pytest.mark.gpu
N = 4096
Q = 2**64 - 2**32 - 31


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def _cache(lib, seed, kind, rows, col0, ncols, k):
    key = DeviceBuffer(lib, k * ncols * rows * N * 4)
    s = np.asarray(seed, dtype=np.uint32)
    assert lib.agl_mcommit_keygen(s.ctypes.data, kind, rows, col0, ncols, k, key.ptr) == 0
    return key


def _partial(lib, key, kcols, rows, k, x, V, C, idx=None, vstride=0):
    dx = DeviceBuffer.from_numpy(lib, x)
    di = None if idx is None else DeviceBuffer.from_numpy(lib, np.asarray(idx, dtype=np.uint32))
    acc = DeviceBuffer(lib, V * k * rows * N * 4)
    rc = lib.agl_mcommit_partial(key.ptr, kcols, rows, k, dx.ptr, x.dtype.itemsize, V, C, vstride, di.ptr if di else None, acc.ptr)
    assert rc == 0
    return acc


def _finish(lib, acc, V, k, rows, err=None):
    de = None if err is None else DeviceBuffer.from_numpy(lib, np.asarray(err, dtype=np.int64))
    out = DeviceBuffer(lib, V * rows * N * 8)
    assert lib.agl_mcommit_finish(acc.ptr, V, k, rows, de.ptr if de else None, out.ptr) == 0
    return out.to_numpy().reshape(V, rows, N)


def _ternary(rng, shape):
    return rng.integers(-1, 2, size=shape, dtype=np.int8)


@pytest.mark.parametrize("rows,payload,hiding", [(2, 4, 2), (16, 6, 5), (5, 3, 1)])
def test_ternary_commit_with_skipped_column_and_error(lib, rows, payload, hiding):
    """Payload column 1 is absent, hiding columns follow the payload columns, identity error added."""
    seed = [4, 4, 2, 2, 1, 1, 0, 9]
    rng = np.random.default_rng(8 + rows)
    total = payload + hiding
    key = _cache(lib, seed, 1, rows, 0, total, 3)
    idx = [c for c in range(payload) if c != 1] + [payload + h for h in range(hiding)]
    x = _ternary(rng, (len(idx), N))
    err = _ternary(rng, (rows, N)).astype(np.int64)
    acc = _partial(lib, key, total, rows, 3, x, 1, len(idx), idx)
    got = _finish(lib, acc, 1, 3, rows, err)[0]
    want = po.mcommit_commit(seed, 1, rows, idx, x.astype(np.int64), err)
    assert np.array_equal(got, want)


def test_wide_inputs_two_vectors_and_column_shards(lib):
    """|x| < 2^36, five primes, columns split in two shards whose accumulators are added."""
    seed = [7] * 8
    rows, cols = 16, 5
    rng = np.random.default_rng(9)
    x = rng.integers(-(1 << 36), 1 << 36, size=(2, cols, N), dtype=np.int64)
    key = _cache(lib, seed, 2, rows, 0, cols, 5)
    split = 2
    a = _partial(lib, key, cols, rows, 5, np.ascontiguousarray(x[:, :split]), 2, split, list(range(split)))
    b = _partial(lib, key, cols, rows, 5, np.ascontiguousarray(x[:, split:]), 2, cols - split, list(range(split, cols)))
    assert lib.agl_mcommit_add(a.ptr, b.ptr, 2, 5, rows) == 0
    got = _finish(lib, a, 2, 5, rows)
    for v in range(2):
        assert np.array_equal(got[v], po.mcommit_commit(seed, 2, rows, list(range(cols)), x[v]))
    # finishing twice gives the same result: the accumulator is not consumed
    assert np.array_equal(_finish(lib, a, 2, 5, rows), got)


@pytest.mark.parametrize("V,rows,C", [(3, 3, 4), (5, 16, 2), (8, 7, 3), (1, 1, 1)])
def test_vector_counts_strides_and_a_prefix_of_the_cache(lib, V, rows, C):
    """Several vectors per pass with a vector stride larger than the packed one; cache built with five
    primes at a column offset, used with four (a prefix of the prime-major layout)."""
    seed = [3, 1, 4, 1, 5, 9, 2, 6]
    rng = np.random.default_rng(100 * V + C)
    col0, kc = 2**33 + 7, 4
    key = _cache(lib, seed, 3, rows, col0, C + 2, 5)
    vstride = C * N + 640
    x = np.zeros(V * vstride, dtype=np.int64)
    cols = rng.integers(-(1 << 30), 1 << 30, size=(V, C, N), dtype=np.int64)
    for v in range(V):
        x[v * vstride:v * vstride + C * N] = cols[v].reshape(-1)
    idx = [(c * 2 + 1) % (C + 2) for c in range(C)]
    acc = _partial(lib, key, C + 2, rows, kc, x, V, C, idx, vstride)
    got = _finish(lib, acc, V, kc, rows)
    for v in range(V):
        assert np.array_equal(got[v], po.mcommit_commit(seed, 3, rows, [col0 + i for i in idx], cols[v]))


def test_many_columns_in_chunks_and_int8_extremes(lib):
    """Enough columns for several column chunks; int8 values over the whole range; identity column map."""
    seed = [11, 12, 13, 14, 15, 16, 17, 18]
    rows, C = 2, 20
    rng = np.random.default_rng(3)
    x = rng.integers(-128, 128, size=(C, N), dtype=np.int8)
    x[0, :4] = [-128, 127, 0, -1]
    key = _cache(lib, seed, 1, rows, 5, C, 3)
    acc = _partial(lib, key, C, rows, 3, x, 1, C)
    got = _finish(lib, acc, 1, 3, rows)[0]
    assert np.array_equal(got, po.mcommit_commit(seed, 1, rows, [5 + c for c in range(C)], x.astype(np.int64)))


def test_no_columns_and_argument_errors(lib):
    rows, k = 3, 3
    acc = DeviceBuffer(lib, k * rows * N * 4)
    assert lib.agl_mcommit_partial(None, 0, rows, k, None, 1, 1, 0, 0, None, acc.ptr) == 0
    err = np.arange(rows * N, dtype=np.int64) - 6000
    got = _finish(lib, acc, 1, k, rows, err)[0]
    assert np.array_equal(got.reshape(-1), np.array([int(e) % Q for e in err], dtype=np.uint64))
    s = np.zeros(8, dtype=np.uint32)
    key = DeviceBuffer(lib, 4 * N * 4)
    assert lib.agl_mcommit_keygen(s.ctypes.data, 1, 17, 0, 1, 1, key.ptr) == -2
    assert lib.agl_mcommit_keygen(s.ctypes.data, 1, 1, 0, 1, 6, key.ptr) == -2
    assert lib.agl_mcommit_partial(key.ptr, 1, 1, 1, key.ptr, 4, 1, 1, 0, None, acc.ptr) == -2
    assert lib.agl_mcommit_partial(key.ptr, 1, 1, 1, key.ptr, 1, 9, 1, 0, None, acc.ptr) == -2
    assert lib.agl_mcommit_finish(acc.ptr, 1, 0, rows, None, acc.ptr) == -2


def test_linearity_at_a_larger_size(lib):
    """256 columns, 16 rows: commit(x1) + commit(x2) = commit(x1 + x2) mod q (no oracle at this size)."""
    seed = [2, 7, 1, 8, 2, 8, 1, 8]
    rows, C = 16, 256
    rng = np.random.default_rng(12)
    x1, x2 = _ternary(rng, (C, N)), _ternary(rng, (C, N))
    key = _cache(lib, seed, 1, rows, 0, C, 3)
    outs = []
    for x in (x1, x2, (x1 + x2).astype(np.int8)):
        outs.append(_finish(lib, _partial(lib, key, C, rows, 3, x, 1, C), 1, 3, rows)[0])
    s = (outs[0].astype(object) + outs[1].astype(object)) % Q
    assert np.array_equal(s.astype(np.uint64), outs[2])
