"""GPU parity of the Goldilocks sumcheck path against the CPU oracle, through
the C-ABI. Bit-exact: every compared word must be equal."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from .conftest import GL_P, field_elems

pytestmark = pytest.mark.gpu
P = GL_P


@pytest.fixture(scope="module")
def lib():
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    assert lib.poseidon2_cuda_init() == 0
    return lib


def _sum_partials(partials, rows, width):
    out = []
    part = partials.reshape(rows, width)
    for k in range(width):
        out.append(sum(int(x) for x in part[:, k]) % P)
    return out


@pytest.mark.parametrize("nv,d", [(1, 1), (1, 2), (2, 2), (4, 2), (3, 3), (9, 1), (10, 4), (12, 3), (13, 8), (16, 2),
                                  (18, 1), (19, 4)])   # one table, and five or more, beyond 2^16 pairs: 256-thread blocks
def test_base_round_and_fold_dropin(lib, oracle, nv, d):
    n = 1 << nv
    polys = field_elems(1000 + nv * 10 + d, n * d)
    if nv == 12 and d == 3:  # inputs of the reference's test_gpu_sumcheck_vs_cpu_large
        polys = np.array([(i * m + k) % P for (m, k) in ((37, 1), (53, 7), (71, 13)) for i in range(n)], dtype=np.uint64)
    cur = polys.copy()
    d_a = DeviceBuffer.from_numpy(lib, cur)
    d_b = DeviceBuffer(lib, cur.nbytes)
    size = n
    for rnd in range(nv):
        half = size // 2
        num_blocks = min((half + 255) // 256, 256)
        d_part = DeviceBuffer(lib, num_blocks * (d + 1) * 8)
        assert lib.sumcheck_round_message_ffi(d_a.ptr, d_part.ptr, d, n, half, num_blocks) == 0
        got = _sum_partials(d_part.to_numpy(), num_blocks, d + 1)
        exp = np.zeros(d + 1, dtype=np.uint64)
        oracle.oracle_gl_round_message(cur.ctypes.data, d, n, half, exp.ctypes.data)
        assert got == [int(x) for x in exp], "round %d" % rnd
        assert int(d_part.to_numpy().max()) < P
        r = (rnd * 11 + 5) if rnd % 2 == 0 else int(field_elems(rnd, 1)[0])
        assert lib.sumcheck_fold_ffi(d_a.ptr, d_b.ptr, r, d, n, half) == 0
        nxt = cur.copy()
        oracle.oracle_gl_fold(cur.ctypes.data, nxt.ctypes.data, r, d, n, half)
        out = d_b.to_numpy()
        for i in range(d):
            assert np.array_equal(out[i * n:i * n + half], nxt[i * n:i * n + half])
        cur = nxt
        d_a, d_b = d_b, d_a
        size = half


@pytest.mark.parametrize("nv,d", [(1, 1), (2, 2), (5, 3), (11, 2), (12, 5), (14, 8), (16, 3), (18, 1)])
def test_ext2_round_and_fold_dropin(lib, oracle, nv, d):
    n = 1 << nv
    cur = field_elems(2000 + nv * 10 + d, n * d * 2)
    d_a = DeviceBuffer.from_numpy(lib, cur)
    d_b = DeviceBuffer(lib, cur.nbytes)
    size = n
    for rnd in range(nv):
        half = size // 2
        num_blocks = min((half + 255) // 256, 256)
        d_part = DeviceBuffer(lib, num_blocks * (d + 1) * 16)
        assert lib.sumcheck_round_message_ext2_ffi(d_a.ptr, d_part.ptr, d, n, half, num_blocks) == 0
        got = _sum_partials(d_part.to_numpy(), num_blocks, 2 * (d + 1))
        exp = np.zeros(2 * (d + 1), dtype=np.uint64)
        oracle.oracle_gl_round_message_ext2(cur.ctypes.data, d, n, half, exp.ctypes.data)
        assert got == [int(x) for x in exp], "round %d" % rnd
        r = field_elems(3000 + rnd, 2)
        assert lib.sumcheck_fold_ext2_ffi(d_a.ptr, d_b.ptr, int(r[0]), int(r[1]), d, n, half) == 0
        nxt = cur.copy()
        oracle.oracle_gl_fold_ext2(cur.ctypes.data, nxt.ctypes.data, int(r[0]), int(r[1]), d, n, half)
        out = d_b.to_numpy()
        for i in range(d):
            assert np.array_equal(out[2 * i * n:2 * (i * n + half)], nxt[2 * i * n:2 * (i * n + half)])
        cur = nxt
        d_a, d_b = d_b, d_a
        size = half


def test_noncanonical_inputs_give_canonical_outputs(lib, oracle):
    # Inputs at or above p are other names of the same residues.
    nv, d = 8, 2
    n = 1 << nv
    canon = field_elems(77, n * d)
    loose = canon.copy()
    small = canon < np.uint64(2**32 - 1)
    loose[small] = loose[small] + np.uint64(P)
    loose[0] = np.uint64(P)  # zero
    canon[0] = 0
    d_a = DeviceBuffer.from_numpy(lib, loose)
    d_part = DeviceBuffer(lib, (d + 1) * 8)
    assert lib.sumcheck_round_message_ffi(d_a.ptr, d_part.ptr, d, n, n // 2, 1) == 0
    exp = np.zeros(d + 1, dtype=np.uint64)
    oracle.oracle_gl_round_message(canon.ctypes.data, d, n, n // 2, exp.ctypes.data)
    assert np.array_equal(d_part.to_numpy(), exp)


@pytest.mark.parametrize("nv,d,base", [(1, 1, True), (1, 2, False), (2, 2, True), (3, 3, False), (6, 2, True),
                                       (10, 3, True), (12, 2, False), (15, 4, True), (18, 2, True), (20, 2, True),
                                       (19, 1, True), (19, 1, False)])
def test_whole_proof_matches_oracle(lib, nv, d, base):
    # (20, 2, True) is the 2^20 configuration: f, g uniform with seeds 1 and 2,
    # transcript label "bench"; every round polynomial, challenge and the final
    # claim must equal the CPU prover's, word for word.
    from oracle import pyoracle
    n = 1 << nv
    w = 1 if base else 2
    if nv == 20:
        polys = np.concatenate([field_elems(1, n), field_elems(2, n)])
    else:
        polys = field_elems(4000 + nv * 10 + d, n * d * w)
    exp = pyoracle.sumcheck_prove(polys, d, nv, base, b"bench")
    rm = np.zeros((nv, d + 1, 2), dtype=np.uint64)
    ch = np.zeros((nv, 2), dtype=np.uint64)
    fes = np.zeros((d, 2), dtype=np.uint64)
    fe = np.zeros(2, dtype=np.uint64)
    st = np.zeros(8, dtype=np.uint64)
    rc = lib.gl_sumcheck_prove_host_ffi(polys.ctypes.data, d, nv, 1 if base else 0, b"bench", 5, rm.ctypes.data,
                                        ch.ctypes.data, fes.ctypes.data, fe.ctypes.data, st.ctypes.data)
    assert rc == 0
    assert np.array_equal(rm, exp["round_msgs"])
    assert np.array_equal(ch, exp["challenges"])
    assert np.array_equal(fes, exp["final_evals"])
    assert np.array_equal(fe, exp["final_eval"])
    assert np.array_equal(st, exp["state"])


def test_bad_arguments_are_rejected(lib):
    d_a = DeviceBuffer(lib, 1024)
    assert lib.sumcheck_round_message_ffi(d_a.ptr, d_a.ptr, 0, 16, 8, 1) == -2
    assert lib.sumcheck_round_message_ffi(d_a.ptr, d_a.ptr, 9, 16, 8, 1) == -2
    assert lib.sumcheck_round_message_ffi(d_a.ptr, d_a.ptr, 2, 16, 0, 1) == -2
    assert lib.sumcheck_fold_ffi(0, d_a.ptr, 1, 2, 16, 8) == -2
