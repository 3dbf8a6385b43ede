"""The allocation-free round message against the ordinary entry point and the CPU oracle.

Collected last on purpose (pytest orders files by name): if it fails, a run that
stops at the first failure has already run everything else.

The entry point is for hosts that may not allocate through this library: a
prover whose own arena owns all device memory, or a loop that must stay off the
driver's allocation lock. Its scratch is a fixed array in the library image that
all calls share, so consecutive calls on different inputs are checked: a call
must not see anything of the one before it.
"""
import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from .conftest import GL_P, field_elems

pytestmark = pytest.mark.gpu
P = GL_P
MAX_ROWS = 592   # partial rows the fixed array holds: beyond 592 * 256 pairs the rows are grid-strided


def _ordinary_message(lib, d_polys, d, n, half):
    """The existing entry point: per-block partial rows, added up here."""
    num_blocks = min((half + 255) // 256, 256)
    d_part = DeviceBuffer(lib, num_blocks * (d + 1) * 16)
    assert lib.sumcheck_round_message_ext2_ffi(d_polys.ptr, d_part.ptr, d, n, half, num_blocks) == 0
    part = d_part.to_numpy().reshape(num_blocks, 2 * (d + 1))
    return np.array([sum(int(x) for x in part[:, k]) % P for k in range(2 * (d + 1))], dtype=np.uint64)


def test_no_alloc_round_message_matches_ordinary_entry_point_twice():
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    # two calls in a row, different shapes and data: bit-exact both times
    for call, (nv, d, seed) in enumerate([(17, 3, 901), (13, 2, 902)]):
        n = 1 << nv
        polys = field_elems(seed, n * d * 2)
        d_polys = DeviceBuffer.from_numpy(lib, polys)
        d_msg = DeviceBuffer(lib, (d + 1) * 16)
        half = n // 2
        assert lib.sumcheck_round_message_ext2_noalloc_ffi(d_polys.ptr, d_msg.ptr, d, n, half) == 0, "call %d" % call
        got = d_msg.to_numpy()
        exp = _ordinary_message(lib, d_polys, d, n, half)
        assert np.array_equal(got, exp), "call %d differs from sumcheck_round_message_ext2_ffi" % call
    # a later round of the same tables (half smaller than the table) and a tiny case
    assert lib.sumcheck_round_message_ext2_noalloc_ffi(d_polys.ptr, d_msg.ptr, d, n, 4) == 0
    assert np.array_equal(d_msg.to_numpy(), _ordinary_message(lib, d_polys, d, n, 4))


@pytest.mark.parametrize("d", [1, 3, 8])
def test_no_alloc_capped_grid_against_the_oracle(oracle, d):
    """2^19 pairs per table: more than 592 * 256, so the grid is capped at the 592 rows the fixed array holds and
    every block sweeps several times; the last block adds up all 592 rows. Compared with the CPU oracle and with
    the ordinary entry point, twice in a row on different data (the ticket counter and the rows of the previous
    call must not leak into the next one), then once more on the first data."""
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    nv = 20
    n, half = 1 << nv, 1 << (nv - 1)
    assert half > MAX_ROWS * 256
    d_msg = DeviceBuffer(lib, (d + 1) * 16)
    first = None
    for call, seed in enumerate((911, 912)):
        polys = field_elems(seed + d, n * d * 2)
        d_polys = DeviceBuffer.from_numpy(lib, polys)
        assert lib.sumcheck_round_message_ext2_noalloc_ffi(d_polys.ptr, d_msg.ptr, d, n, half) == 0, "call %d" % call
        got = d_msg.to_numpy()
        exp = np.zeros(2 * (d + 1), dtype=np.uint64)
        oracle.oracle_gl_round_message_ext2(polys.ctypes.data, d, n, half, exp.ctypes.data)
        assert np.array_equal(got, exp), "call %d differs from the CPU oracle" % call
        assert np.array_equal(got, _ordinary_message(lib, d_polys, d, n, half)), "call %d" % call
        if first is None:
            first = (d_polys, got.copy())
    assert lib.sumcheck_round_message_ext2_noalloc_ffi(first[0].ptr, d_msg.ptr, d, n, half) == 0
    assert np.array_equal(d_msg.to_numpy(), first[1])


def test_no_alloc_rejects_sizes_beyond_its_maximum():
    lib = load_gl()
    d_a = DeviceBuffer(lib, 4096)
    assert lib.sumcheck_round_message_ext2_noalloc_ffi(d_a.ptr, d_a.ptr, 2, 1 << 32, (1 << 30) + 1) == -3
    assert lib.sumcheck_round_message_ext2_noalloc_ffi(d_a.ptr, d_a.ptr, 9, 16, 8) == -2
    assert lib.sumcheck_round_message_ext2_noalloc_ffi(0, d_a.ptr, 2, 16, 8) == -2
