"""GPU parity of the Ajtai commitment against the CPU oracle (itself pinned to the
reference's CPU code), through the C-ABI. Bit-exact."""
import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from matrix_b200.inputs import AGL_Q, field_elems

pytestmark = pytest.mark.gpu
Q = AGL_Q
KEY = np.arange(1, 9, dtype=np.uint32)


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def test_reference_regression_vector(lib):
    # key 1..8, z = {0x123456789abcdef0, ~0, 0, 1}: values produced by the reference's cpu_ajtai_commit
    z = np.array([0x123456789abcdef0, 0xFFFFFFFFFFFFFFFF, 0, 1], dtype=np.uint64)
    d_k, d_z, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, z), DeviceBuffer(lib, 42 * 64 * 8)
    assert lib.ajtai_commit_dense_batched_ffi(d_k.ptr, d_z.ptr, 4, 1, 64, d_o.ptr) == 0
    out = d_o.to_numpy()
    assert int(out[0]) == 0x0d35295c35dc119b and int(out[41 * 64 + 63]) == 0x233af51a4cee11e2


@pytest.mark.parametrize("n,b,off", [(1, 1, 0), (5, 2, 0), (37, 4, 11), (64, 8, 1 << 33), (300, 16, 5), (1500, 1, 0)])
def test_dense_planes_match_oracle(lib, n, b, off):
    from oracle import pyoracle
    rng = np.random.default_rng(n + b)
    z = rng.integers(0, 2**63, size=n * b, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=n * b, dtype=np.uint64)
    z[::7] = 0  # empty ring elements are skipped
    d_k, d_z, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, z), DeviceBuffer(lib, b * 42 * 64 * 8)
    assert lib.ajtai_commit_dense_batched_at_ffi(d_k.ptr, d_z.ptr, n, b, 256, off, d_o.ptr) == 0
    assert np.array_equal(d_o.to_numpy(), pyoracle.ajtai_commit(KEY, z, 0, n, b, off))


def test_column_shards_sum_to_the_whole(lib):
    # the reference's test_multi_gpu_split_simulation (tests/ajtai_integration.rs:296-328): j-range shards add up
    n = 96
    rng = np.random.default_rng(1)
    z = rng.integers(0, 2**63, size=n, dtype=np.uint64)
    d_k, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer(lib, 42 * 64 * 8)
    d_z = DeviceBuffer.from_numpy(lib, z)
    assert lib.ajtai_commit_dense_batched_ffi(d_k.ptr, d_z.ptr, n, 1, 64, d_o.ptr) == 0
    whole = d_o.to_numpy()
    acc = np.zeros(42 * 64, dtype=object)
    for lo, hi in ((0, 32), (32, 80), (80, 96)):
        d_s = DeviceBuffer.from_numpy(lib, z[lo:hi].copy())
        assert lib.ajtai_commit_dense_batched_at_ffi(d_k.ptr, d_s.ptr, hi - lo, 1, 64, lo, d_o.ptr) == 0
        acc = (acc + d_o.to_numpy().astype(object)) % Q
    assert [int(x) for x in acc] == [int(x) for x in whole]


@pytest.mark.parametrize("n,planes,off", [(1, 1, 0), (9, 3, 2), (70, 8, 0), (200, 3, 77)])
def test_signed_digits_match_oracle(lib, n, planes, off):
    from oracle import pyoracle
    rng = np.random.default_rng(n * 3 + planes)
    dig = rng.integers(-128, 128, size=planes * n * 64, dtype=np.int8)
    dig[:64] = 127
    dig[64:128] = -128
    d_k, d_z = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, dig)
    d_o = DeviceBuffer(lib, planes * 42 * 64 * 8)
    assert lib.ajtai_commit_s8_scalar_ffi(d_k.ptr, d_z.ptr, n, planes, off, d_o.ptr) == 0
    assert np.array_equal(d_o.to_numpy(), pyoracle.ajtai_commit(KEY, dig, 1, n, planes, off))


@pytest.mark.parametrize("n,planes,off", [(1, 1, 0), (4, 1, 0), (5, 3, 9), (70, 4, 0), (130, 8, 3), (600, 3, 1 << 20)])
def test_tensor_core_digits_match_oracle(lib, n, planes, off):
    # tcgen05 path: exact integer accumulation, so the result must equal the CPU oracle bit for bit;
    # planes = 8 runs two plane groups. Witnesses this short are cut into narrow column chunks (a CTA gets
    # 32 columns); the full 512-column chunk has its own test below.
    from oracle import pyoracle
    rng = np.random.default_rng(n * 5 + planes)
    dig = rng.integers(-127, 128, size=planes * n * 64, dtype=np.int8)
    dig[:64] = 127
    dig[-64:] = -127
    d_k, d_z = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, dig)
    d_o = DeviceBuffer(lib, planes * 42 * 64 * 8)
    assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, n, planes, off, d_o.ptr) == 0
    got = d_o.to_numpy()
    exp = pyoracle.ajtai_commit(KEY, dig, 1, n, planes, off)
    bad = np.nonzero(got != exp)[0]
    assert len(bad) == 0, "%d of %d words differ, first at %d" % (len(bad), len(exp), bad[0])


def test_tensor_core_full_width_chunks_with_worst_case_sums(lib):
    """50 688 ring columns: the smallest witness whose column chunks are the full 512 columns wide, the width the
    2^18-column configuration runs at. Every digit of chunk 0 is +127 and every digit of chunk 1 is -127, the
    largest magnitude a 32-bit accumulator sees before it is drained (255 * 127 * 64 * 512 < 2^31); the rest is
    random. All 42 x 64 output words against the scalar kernel (itself pinned to the CPU oracle), and rows 0 and
    41 against the reference's own host code (ring elements from its ChaCha8 expansion, products by its
    cpu_ring_mul), summed here."""
    from oracle import pyoracle
    n, planes = 50688, 2
    rng = np.random.default_rng(99)
    dig = rng.integers(-127, 128, size=planes * n * 64, dtype=np.int8)
    dig[:512 * 64] = 127
    dig[512 * 64:1024 * 64] = -127
    dig[n * 64 + 1024 * 64:n * 64 + 1536 * 64] = 127          # plane 1: a different chunk
    d_k, d_z = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, dig)
    d_a, d_b = DeviceBuffer(lib, planes * 42 * 64 * 8), DeviceBuffer(lib, planes * 42 * 64 * 8)
    assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, n, planes, 0, d_a.ptr) == 0
    assert lib.ajtai_commit_s8_scalar_ffi(d_k.ptr, d_z.ptr, n, planes, 0, d_b.ptr) == 0
    got = d_a.to_numpy()
    assert np.array_equal(got, d_b.to_numpy())
    ref = pyoracle.load_ref("libajtai_ref.so")
    if ref is None:
        pytest.skip("oracle/_ref/libajtai_ref.so not built")
    z = np.where(dig[:n * 64] < 0, np.uint64(Q) - (-dig[:n * 64].astype(np.int64)).astype(np.uint64),
                 dig[:n * 64].astype(np.int64).astype(np.uint64)).reshape(n, 64)
    z = np.ascontiguousarray(z)
    for row in (0, 41):
        acc = np.zeros(64, dtype=object)
        m, prod = np.zeros(64, dtype=np.uint64), np.zeros(64, dtype=np.uint64)
        part = np.zeros(64, dtype=object)
        for j in range(n):
            ref.ref_ajtai_ring_elem(KEY.ctypes.data, row, j, m.ctypes.data)
            ref.ref_ring_mul(m.ctypes.data, z[j].ctypes.data, prod.ctypes.data)
            part += prod.astype(object)
            if j % 4096 == 4095:
                acc = (acc + part) % Q
                part = np.zeros(64, dtype=object)
        acc = (acc + part) % Q
        assert [int(x) for x in got[row * 64:(row + 1) * 64]] == [int(x) for x in acc], "row %d" % row


def test_tensor_core_rejects_minus_128(lib):
    dig = np.zeros(64, dtype=np.int8)
    dig[5] = -128
    d_k, d_z, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, dig), DeviceBuffer(lib, 42 * 64 * 8)
    assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, 1, 1, 0, d_o.ptr) == -3


@pytest.mark.parametrize("n,off", [(1, 0), (20, 3), (130, 0)])
def test_wide_matches_oracle(lib, n, off):
    from oracle import pyoracle
    w = field_elems(50 + n, n * 64, Q)
    w[:3] = [0, Q - 1, 1]
    d_k, d_z, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, w), DeviceBuffer(lib, 42 * 64 * 8)
    assert lib.ajtai_commit_wide_ffi(d_k.ptr, d_z.ptr, n, off, 128, d_o.ptr) == 0
    assert np.array_equal(d_o.to_numpy(), pyoracle.ajtai_commit(KEY, w, 2, n, 1, off))


def test_materialised_matrix_and_argument_checks(lib):
    n = 3
    d_k, d_m = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer(lib, n * 42 * 64 * 8)
    assert lib.ajtai_materialize_m_ffi(d_k.ptr, d_m.ptr, n) == 0
    m = d_m.to_numpy().reshape(n, 42, 64)
    from oracle import pyoracle
    o = pyoracle.load()
    for (j, i) in ((0, 0), (2, 41), (1, 17)):
        e = np.zeros(64, dtype=np.uint64)
        o.oracle_ajtai_ring_elem(KEY.ctypes.data, i, j, e.ctypes.data)
        assert np.array_equal(m[j, i], e)
    d_z, d_o = DeviceBuffer(lib, 64), DeviceBuffer(lib, 16 * 42 * 64 * 8)
    assert lib.ajtai_commit_dense_batched_ffi(d_k.ptr, d_z.ptr, 1, 3, 64, d_o.ptr) == -2   # B not a power of two <= 16
    assert lib.ajtai_commit_dense_batched_ffi(d_k.ptr, d_z.ptr, 1, 1, 100, d_o.ptr) == -3  # unsupported chunk


def _ternary_planes(rng, n_ring, planes=13):
    """Random disjoint pos / neg masks [planes][n_ring] and the digits they stand for."""
    pos = rng.integers(0, 2**63, size=planes * n_ring, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=planes * n_ring, dtype=np.uint64)
    neg = rng.integers(0, 2**63, size=planes * n_ring, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=planes * n_ring, dtype=np.uint64)
    neg &= ~pos
    pos[::5] = 0
    neg[1::7] = 0
    shifts = np.arange(64, dtype=np.uint64)
    digits = (((pos[:, None] >> shifts) & np.uint64(1)).astype(np.int8) - ((neg[:, None] >> shifts) & np.uint64(1)).astype(np.int8))
    return pos, neg, np.ascontiguousarray(digits.reshape(-1))


@pytest.mark.parametrize("n_ring", [1, 3, 70, 260])
def test_ternary_commit_matches_oracle(lib, n_ring):
    from oracle import pyoracle
    pos, neg, digits = _ternary_planes(np.random.default_rng(40 + n_ring), n_ring)
    exp = pyoracle.ajtai_commit(KEY, digits, 1, n_ring, 13)
    d_k, d_p, d_n = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, pos), DeviceBuffer.from_numpy(lib, neg)
    d_o = DeviceBuffer(lib, 13 * 42 * 64 * 8)
    assert lib.ajtai_commit_ternary_ffi(d_k.ptr, d_p.ptr, d_n.ptr, n_ring, 256, d_o.ptr) == 0
    assert np.array_equal(d_o.to_numpy(), exp)
    # against a materialised matrix
    d_m = DeviceBuffer(lib, 8 * 42 * 64 * n_ring)
    assert lib.ajtai_materialize_m_ffi(d_k.ptr, d_m.ptr, n_ring) == 0
    d_o2 = DeviceBuffer(lib, 13 * 42 * 64 * 8)
    assert lib.ajtai_commit_ternary_premat_ffi(d_m.ptr, d_p.ptr, d_n.ptr, n_ring, 64, d_o2.ptr) == 0
    assert np.array_equal(d_o2.to_numpy(), exp)
    assert lib.ajtai_commit_ternary_ffi(d_k.ptr, d_p.ptr, d_n.ptr, n_ring, 100, d_o.ptr) == -3
    assert lib.ajtai_commit_ternary_ffi(d_k.ptr, d_p.ptr, d_n.ptr, 0, 64, d_o.ptr) == 0
    assert not d_o.to_numpy().any()


@pytest.mark.parametrize("n_ring,planes", [(1, 1), (5, 3), (513, 4), (1100, 6), (700, 8), (130, 13)])
def test_signed_digits_against_a_materialised_matrix(lib, n_ring, planes):
    """The tensor-core kernel streaming the materialised matrix equals the one regenerating it (and the oracle)."""
    from oracle import pyoracle
    rng = np.random.default_rng(70 + n_ring)
    digits = rng.integers(-127, 128, size=planes * n_ring * 64, dtype=np.int8)
    d_k, d_z = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, digits)
    d_m = DeviceBuffer(lib, 8 * 42 * 64 * n_ring)
    assert lib.ajtai_materialize_m_ffi(d_k.ptr, d_m.ptr, n_ring) == 0
    d_a, d_b = DeviceBuffer(lib, planes * 42 * 64 * 8), DeviceBuffer(lib, planes * 42 * 64 * 8)
    assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, n_ring, planes, 0, d_a.ptr) == 0
    assert lib.ajtai_commit_s8_premat_ffi(d_m.ptr, d_z.ptr, n_ring, planes, d_b.ptr) == 0
    assert np.array_equal(d_a.to_numpy(), d_b.to_numpy())
    if n_ring <= 16:
        assert np.array_equal(d_b.to_numpy(), pyoracle.ajtai_commit(KEY, digits, 1, n_ring, planes))
    assert lib.ajtai_commit_s8_premat_ffi(None, d_z.ptr, n_ring, planes, d_b.ptr) == -2
    # byte planes in operand order
    d_t = DeviceBuffer(lib, lib.ajtai_tc_matrix_bytes(n_ring))
    assert lib.ajtai_tc_matrix_bytes(n_ring) == ((n_ring + 3) // 4) * 3 * 28672
    assert lib.ajtai_materialize_tc_ffi(d_k.ptr, d_t.ptr, n_ring, 0) == 0
    d_c = DeviceBuffer(lib, planes * 42 * 64 * 8)
    assert lib.ajtai_commit_s8_tiled_ffi(d_t.ptr, d_z.ptr, n_ring, planes, d_c.ptr) == 0
    assert np.array_equal(d_a.to_numpy(), d_c.to_numpy())


@pytest.mark.parametrize("n_ring,k_chunks", [(1, 13), (50, 13), (300, 8), (64, 16)])
def test_wide_to_ternary_and_back(lib, n_ring, k_chunks):
    """Planes recombine to the coefficients (sum_i 2^i (pos_i - neg_i)); a coefficient that needs more bits
    raises the flag; committing the planes and recombining equals the commit of the signed coefficients."""
    from oracle import pyoracle
    rng = np.random.default_rng(n_ring)
    lim = min(2**k_chunks - 1, 32767)
    wide = rng.integers(-lim, lim + 1, size=n_ring * 64, dtype=np.int16)
    wide[:4] = [lim, -lim, 0, 1]
    d_w = DeviceBuffer.from_numpy(lib, wide)
    d_p, d_n = DeviceBuffer(lib, 8 * k_chunks * n_ring), DeviceBuffer(lib, 8 * k_chunks * n_ring)
    d_e = DeviceBuffer.from_numpy(lib, np.zeros(1, dtype=np.int32))
    assert lib.aext2_wide_to_ternary_ffi(d_w.ptr, d_p.ptr, d_n.ptr, d_e.ptr, n_ring, k_chunks) == 0
    lib.cuda_device_synchronize()
    pos, neg = d_p.to_numpy().reshape(k_chunks, n_ring), d_n.to_numpy().reshape(k_chunks, n_ring)
    assert int(d_e.to_numpy(dtype="int32")[0]) == 0
    assert not (pos & neg).any()
    shifts = np.arange(64, dtype=np.uint64)
    rec = np.zeros((n_ring, 64), dtype=np.int64)
    for i in range(k_chunks):
        rec += (((pos[i][:, None] >> shifts) & np.uint64(1)).astype(np.int64) - ((neg[i][:, None] >> shifts) & np.uint64(1)).astype(np.int64)) << i
    assert np.array_equal(rec.reshape(-1), wide.astype(np.int64))
    if k_chunks < 15:
        wide[7] = 2**k_chunks
        d_w2 = DeviceBuffer.from_numpy(lib, wide)
        assert lib.aext2_wide_to_ternary_ffi(d_w2.ptr, d_p.ptr, d_n.ptr, d_e.ptr, n_ring, k_chunks) == 0
        lib.cuda_device_synchronize()
        assert int(d_e.to_numpy(dtype="int32")[0]) == 1
    assert lib.aext2_wide_to_ternary_ffi(d_w.ptr, d_p.ptr, d_n.ptr, d_e.ptr, n_ring, 17) == -1


@pytest.mark.parametrize("k,cols", [(1, 1), (200, 40), (5000, 300), (3000, 5)])
def test_sparse_commit_matches_oracle(lib, k, cols):
    from oracle import pyoracle
    rng = np.random.default_rng(k)
    pos = rng.integers(0, 64 * cols, size=k, dtype=np.uint64)
    if k > 100:
        pos[: k // 2] = np.sort(pos[: k // 2])  # runs that reuse a column, then arbitrary order
    exp = np.zeros(42 * 64, dtype=np.uint64)
    pyoracle.load().oracle_ajtai_commit_sparse(KEY.ctypes.data, pos.ctypes.data, k, exp.ctypes.data)
    d_k, d_p, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, pos), DeviceBuffer(lib, 42 * 64 * 8)
    assert lib.ajtai_commit_sparse_ffi(d_k.ptr, d_p.ptr, k, 1024, d_o.ptr) == 0
    assert np.array_equal(d_o.to_numpy(), exp)
    assert lib.ajtai_commit_sparse_ffi(d_k.ptr, d_p.ptr, 0, 64, d_o.ptr) == 0
    assert not d_o.to_numpy().any()
    assert lib.ajtai_commit_sparse_ffi(d_k.ptr, d_p.ptr, k, 7, d_o.ptr) == -3


def test_sparse_commit_reference_vector(lib):
    """The position list whose commitment the reference's cpu_ajtai_commit_sparse produced (tests/golden/ajtai_ref.json)."""
    import hashlib, json, os
    from .conftest import ROOT
    sp = json.load(open(os.path.join(ROOT, "tests", "golden", "ajtai_ref.json")))["sparse"]
    pos = np.array(sp["positions"], dtype=np.uint64)
    d_k, d_p, d_o = DeviceBuffer.from_numpy(lib, KEY), DeviceBuffer.from_numpy(lib, pos), DeviceBuffer(lib, 42 * 64 * 8)
    assert lib.ajtai_commit_sparse_ffi(d_k.ptr, d_p.ptr, len(pos), 256, d_o.ptr) == 0
    out = d_o.to_numpy()
    assert int(out[0]) == sp["first"] and int(out[-1]) == sp["last"]
    assert hashlib.sha256(out.tobytes()).hexdigest() == sp["sha256"]
