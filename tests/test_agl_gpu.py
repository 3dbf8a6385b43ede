"""GPU parity of the almost-Goldilocks entry points (field batches, sumcheck,
eq tables, partial evaluation) and of the Goldilocks partial evaluation against
the CPU oracle, through the C-ABI. Bit-exact."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl, load_gl
from matrix_b200.inputs import AGL_Q
from .conftest import GL_P, field_elems

pytestmark = pytest.mark.gpu
Q = AGL_Q


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def aelems(seed, n):
    return field_elems(seed, n, Q)


def test_field_batches_match_python_integers(lib):
    n = 4096
    a, b = field_elems(1, n, 2**64 - 1), field_elems(2, n, 2**64 - 1)  # loose inputs
    a[:6] = [0, 1, Q - 1, Q, 2**64 - 1, 2**32 + 31]
    b[:6] = [0, Q - 1, Q - 1, Q + 5, 2**64 - 1, 2**32 + 31]
    d_a, d_b, d_r = DeviceBuffer.from_numpy(lib, a), DeviceBuffer.from_numpy(lib, b), DeviceBuffer(lib, 8 * n)
    for fn, op in ((lib.agl_batch_add_ffi, lambda x, y: (x + y) % Q), (lib.agl_batch_sub_ffi, lambda x, y: (x - y) % Q),
                   (lib.agl_batch_mul_ffi, lambda x, y: (x * y) % Q)):
        assert fn(d_a.ptr, d_b.ptr, d_r.ptr, n) == 0
        got = d_r.to_numpy()
        assert all(int(g) == op(int(x), int(y)) for g, x, y in zip(got, a, b))
    assert lib.agl_batch_inverse_ffi(d_a.ptr, d_r.ptr, 64) == 0
    got = d_r.to_numpy()[:64]
    assert all((int(g) * int(x)) % Q == (1 if int(x) % Q else 0) and int(g) < Q for g, x in zip(got, a))
    # (1 + 2X)(3 + 4X) = 27 + 10X (almost-goldilocks-cuda-rs/tests/integration.rs:141-146)
    x, y = np.array([1, 2], dtype=np.uint64), np.array([3, 4], dtype=np.uint64)
    d_x, d_y, d_o = DeviceBuffer.from_numpy(lib, x), DeviceBuffer.from_numpy(lib, y), DeviceBuffer(lib, 16)
    assert lib.aext2_batch_mul_ffi(d_x.ptr, d_y.ptr, d_o.ptr, 1) == 0
    assert list(d_o.to_numpy()) == [27, 10]
    assert lib.aext2_batch_inverse_ffi(d_x.ptr, d_o.ptr, 1) == 0
    inv = d_o.to_numpy()
    assert ((int(inv[0]) + 2 * 3 * int(inv[1])) % Q, (2 * int(inv[0]) + int(inv[1])) % Q) == (1, 0)


def _sum_rows(buf, rows, width):
    part = buf.to_numpy().reshape(rows, width)
    return [sum(int(x) for x in part[:, k]) % Q for k in range(width)]


@pytest.mark.parametrize("nv,d", [(1, 1), (4, 2), (9, 3), (12, 3), (14, 8), (16, 2), (18, 1)])
def test_base_sumcheck_dropin(lib, oracle, nv, d):
    n = 1 << nv
    cur = aelems(100 + nv + d, n * d)
    d_a, d_b = DeviceBuffer.from_numpy(lib, cur), DeviceBuffer(lib, cur.nbytes)
    size = n
    for rnd in range(nv):
        half = size // 2
        nb = min((half + 255) // 256, 256)
        d_p = DeviceBuffer(lib, nb * (d + 1) * 8)
        assert lib.agl_sumcheck_round_message_ffi(d_a.ptr, d_p.ptr, d, n, half, nb) == 0
        exp = np.zeros(d + 1, dtype=np.uint64)
        oracle.oracle_agl_round_message(cur.ctypes.data, d, n, half, exp.ctypes.data)
        assert _sum_rows(d_p, nb, d + 1) == [int(x) for x in exp]
        r = rnd * 11 + 5 if rnd % 2 == 0 else int(aelems(rnd, 1)[0])
        assert lib.agl_sumcheck_fold_ffi(d_a.ptr, d_b.ptr, r, d, n, half) == 0
        nxt = cur.copy()
        oracle.oracle_agl_fold(cur.ctypes.data, nxt.ctypes.data, r, d, n, half)
        out = d_b.to_numpy()
        for i in range(d):
            assert np.array_equal(out[i * n:i * n + half], nxt[i * n:i * n + half])
        cur, size = nxt, half
        d_a, d_b = d_b, d_a


@pytest.mark.parametrize("nv,d", [(1, 1), (5, 2), (11, 3), (13, 5), (16, 3), (18, 1)])
def test_ext2_sumcheck_dropin_and_fused(lib, oracle, nv, d):
    n = 1 << nv
    cur = aelems(200 + nv + d, n * d * 2)
    d_a, d_b = DeviceBuffer.from_numpy(lib, cur), DeviceBuffer(lib, cur.nbytes)
    size = n
    fused_msg = None
    for rnd in range(nv):
        half = size // 2
        nb = min((half + 255) // 256, 256)
        d_p = DeviceBuffer(lib, nb * (d + 1) * 16)
        assert lib.aext2_sumcheck_round_message_ffi(d_a.ptr, d_p.ptr, d, n, half, nb) == 0
        exp = np.zeros(2 * (d + 1), dtype=np.uint64)
        oracle.oracle_aext2_round_message(cur.ctypes.data, d, n, half, exp.ctypes.data)
        assert _sum_rows(d_p, nb, 2 * (d + 1)) == [int(x) for x in exp]
        if fused_msg is not None:
            assert fused_msg == [int(x) for x in exp], "fused fold+message differs at round %d" % rnd
        r = aelems(300 + rnd, 2)
        nxt = cur.copy()
        oracle.oracle_aext2_fold(cur.ctypes.data, nxt.ctypes.data, int(r[0]), int(r[1]), d, n, half)
        if half >= 2 and rnd % 2 == 0:
            quarter = half // 2
            nbq = min((quarter + 255) // 256, 64)
            d_q = DeviceBuffer(lib, nbq * (d + 1) * 16)
            assert lib.aext2_sumcheck_fold_round_ffi(d_a.ptr, d_b.ptr, int(r[0]), int(r[1]), d, n, quarter, d_q.ptr, nbq) == 0
            fused_msg = _sum_rows(d_q, nbq, 2 * (d + 1))
        else:
            assert lib.aext2_sumcheck_fold_ffi(d_a.ptr, d_b.ptr, int(r[0]), int(r[1]), d, n, half) == 0
            fused_msg = None
        out = d_b.to_numpy()
        for i in range(d):
            assert np.array_equal(out[2 * i * n:2 * (i * n + half)], nxt[2 * i * n:2 * (i * n + half)])
        cur, size = nxt, half
        d_a, d_b = d_b, d_a


def test_mixed_fused_first_round(lib, oracle):
    nv, d = 12, 2
    n = 1 << nv
    base = aelems(400, n * d)
    r = aelems(401, 2)
    d_in = DeviceBuffer.from_numpy(lib, base)
    d_out = DeviceBuffer(lib, 16 * n * d)
    quarter = n // 4
    nb = 8
    d_p = DeviceBuffer(lib, nb * (d + 1) * 16)
    assert lib.aext2_sumcheck_fold_round_mixed_ffi(d_in.ptr, d_out.ptr, int(r[0]), int(r[1]), d, n, quarter, d_p.ptr, nb) == 0
    folded = np.zeros(2 * n * d, dtype=np.uint64)
    oracle.oracle_aext2_fold_mixed(base.ctypes.data, folded.ctypes.data, int(r[0]), int(r[1]), d, n, n, n // 2)
    out = d_out.to_numpy()
    for i in range(d):
        assert np.array_equal(out[2 * i * n:2 * i * n + n], folded[2 * i * n:2 * i * n + n])
    exp = np.zeros(2 * (d + 1), dtype=np.uint64)
    oracle.oracle_aext2_round_message(folded.ctypes.data, d, n, quarter, exp.ctypes.data)
    assert _sum_rows(d_p, nb, 2 * (d + 1)) == [int(x) for x in exp]


@pytest.mark.parametrize("log_n", [0, 1, 3, 12, 13, 17])
def test_eq_tables(lib, oracle, log_n):
    n = 1 << log_n
    for words, fn, ofn in ((1, lib.agl_eq_dp_all_ffi, oracle.oracle_agl_eq_base), (2, lib.aext2_eq_dp_all_ffi, oracle.oracle_agl_eq_ext2)):
        r = aelems(500 + log_n, max(1, log_n) * words)
        d_r = DeviceBuffer.from_numpy(lib, r)
        d_a, d_b = DeviceBuffer(lib, 8 * n * words), DeviceBuffer(lib, 8 * n * words)
        res = ctypes.c_void_p()
        assert fn(d_r.ptr, d_a.ptr, d_b.ptr, log_n, ctypes.byref(res)) == 0
        got = np.empty(n * words, dtype=np.uint64)
        assert lib.cuda_memcpy_dtoh(got.ctypes.data, res.value, got.nbytes) == 0
        exp = np.zeros(n * words, dtype=np.uint64)
        ofn(r.ctypes.data, log_n, exp.ctypes.data)
        assert np.array_equal(got, exp)


@pytest.mark.parametrize("log_n,m", [(1, 1), (4, 0), (6, 3), (10, 4), (12, 5), (13, 9), (16, 16), (18, 7)])
def test_partial_eval_both_fields(lib, oracle, log_n, m):
    n = 1 << log_n
    gl = load_gl()
    for field, L, mod, pe, pex, ope, opex in (
            ("agl", lib, Q, lib.agl_partial_eval_ffi, lib.agl_partial_eval_ext2_from_base_ffi,
             oracle.oracle_agl_partial_eval, oracle.oracle_agl_partial_eval_ext2_from_base),
            ("gl", gl, GL_P, gl.partial_eval_gl_ffi, gl.partial_eval_ext2_from_gl_ffi,
             oracle.oracle_gl_partial_eval, oracle.oracle_gl_partial_eval_ext2_from_base)):
        data = field_elems(600 + log_n, n, mod)
        r = field_elems(601 + m, 2 * max(m, 1), mod)
        d_data = DeviceBuffer.from_numpy(L, data)
        d_r = DeviceBuffer.from_numpy(L, r)
        assert pe(d_data.ptr, d_r.ptr, log_n, m) == 0
        exp = np.zeros(n >> m, dtype=np.uint64)
        ope(data.ctypes.data, exp.ctypes.data, r.ctypes.data, log_n, m)
        assert np.array_equal(d_data.to_numpy()[:n >> m], exp), field
        if m >= 1:
            d_in = DeviceBuffer.from_numpy(L, data)
            d_out = DeviceBuffer(L, 16 * max(n // 2, 1))
            assert pex(d_in.ptr, d_out.ptr, d_r.ptr, log_n, m) == 0
            exp2 = np.zeros(2 * (n >> m), dtype=np.uint64)
            opex(data.ctypes.data, exp2.ctypes.data, r.ctypes.data, log_n, m)
            assert np.array_equal(d_out.to_numpy()[:2 * (n >> m)], exp2), field


def _split_luts(n, new_var_order, half):
    # almost-goldilocks-cuda-rs/src/partial_eval.rs:283-321
    inv = list(new_var_order)  # new position -> old variable
    lo = np.zeros(1 << half, dtype=np.uint32)
    for x in range(1 << half):
        lo[x] = sum(1 << inv[bit] for bit in range(half) if x >> bit & 1)
    hi = np.zeros(1 << (n - half), dtype=np.uint32)
    for x in range(1 << (n - half)):
        hi[x] = sum(1 << inv[half + bit] for bit in range(n - half) if x >> bit & 1)
    return lo, hi


@pytest.mark.parametrize("n,m,half", [(4, 2, 2), (10, 4, 5), (13, 6, 6), (16, 9, 8), (17, 0, 9)])
def test_fused_permute_partial_eval_both_fields(lib, oracle, n, m, half):
    gl = load_gl()
    rng = np.random.default_rng(n)
    order = list(rng.permutation(n))
    lo, hi = _split_luts(n, order, half)
    perm = np.array([int(lo[x & ((1 << half) - 1)]) | int(hi[x >> half]) for x in range(1 << n)], dtype=np.int64)
    for L, mod, fn, eqfn, pex in (
            (lib, Q, lib.agl_fused_permute_partial_eval_ffi, oracle.oracle_agl_eq_ext2, oracle.oracle_agl_partial_eval_ext2_from_base),
            (gl, GL_P, gl.fused_permute_partial_eval_ffi, oracle.oracle_gl_eq_ext2, oracle.oracle_gl_partial_eval_ext2_from_base)):
        evals = field_elems(900 + n, 1 << n, mod)
        r = field_elems(901 + n, 2 * max(m, 1), mod)
        eq = np.zeros(2 << m, dtype=np.uint64)
        eqfn(r.ctypes.data, m, eq.ctypes.data)
        out_size = 1 << (n - m)
        d_e, d_q = DeviceBuffer.from_numpy(L, evals), DeviceBuffer.from_numpy(L, eq)
        d_lo, d_hi = DeviceBuffer.from_numpy(L, lo), DeviceBuffer.from_numpy(L, hi)
        d_o = DeviceBuffer(L, 16 * out_size)
        assert fn(d_e.ptr, d_o.ptr, d_q.ptr, d_lo.ptr, d_hi.ptr, n, m, half, out_size, 0) == 0
        # expected: permute on the host, then the oracle's partial evaluation of the m low variables
        permuted = evals[perm]
        exp = np.zeros(2 * out_size, dtype=np.uint64)
        if m == 0:
            exp[0::2] = permuted
        else:
            pex(permuted.ctypes.data, exp.ctypes.data, r.ctypes.data, n, m)
        assert np.array_equal(d_o.to_numpy(), exp)


def test_fused_permute_partial_eval_tables_of_exactly_48k(lib, oracle):
    """n = 25, half = 12: the two index tables take exactly 48 KB of dynamic shared memory, which together with
    the kernel's static shared memory is above the default limit (the launch has to opt in)."""
    n, m, half = 25, 12, 12
    order = list(range(n - m, n)) + list(range(n - m))   # the m high variables become the low ones
    lo, hi = _split_luts(n, order, half)
    x = np.arange(1 << n, dtype=np.int64)
    perm = lo[x & ((1 << half) - 1)].astype(np.int64) | hi[x >> half].astype(np.int64)
    evals = field_elems(925, 1 << n, Q)
    r = field_elems(926, 2 * m, Q)
    eq = np.zeros(2 << m, dtype=np.uint64)
    oracle.oracle_agl_eq_ext2(r.ctypes.data, m, eq.ctypes.data)
    out_size = 1 << (n - m)
    d_e, d_q = DeviceBuffer.from_numpy(lib, evals), DeviceBuffer.from_numpy(lib, eq)
    d_lo, d_hi = DeviceBuffer.from_numpy(lib, lo), DeviceBuffer.from_numpy(lib, hi)
    d_o = DeviceBuffer(lib, 16 * out_size)
    assert lib.agl_fused_permute_partial_eval_ffi(d_e.ptr, d_o.ptr, d_q.ptr, d_lo.ptr, d_hi.ptr, n, m, half, out_size, 0) == 0
    permuted = np.ascontiguousarray(evals[perm])
    exp = np.zeros(2 * out_size, dtype=np.uint64)
    oracle.oracle_agl_partial_eval_ext2_from_base(permuted.ctypes.data, exp.ctypes.data, r.ctypes.data, n, m)
    assert np.array_equal(d_o.to_numpy(), exp)
    # a few fixed variables on the same table: groups of lanes instead of a block per output
    for m2 in (1, 3, 6):
        order2 = list(range(n - m2, n)) + list(range(n - m2))
        lo2, hi2 = _split_luts(n, order2, half)
        perm2 = lo2[x & ((1 << half) - 1)].astype(np.int64) | hi2[x >> half].astype(np.int64)
        oracle.oracle_agl_eq_ext2(r.ctypes.data, m2, eq.ctypes.data)
        d_q2 = DeviceBuffer.from_numpy(lib, eq[:2 << m2])
        d_l2, d_h2 = DeviceBuffer.from_numpy(lib, lo2), DeviceBuffer.from_numpy(lib, hi2)
        d_o2 = DeviceBuffer(lib, 16 << (n - m2))
        assert lib.agl_fused_permute_partial_eval_ffi(d_e.ptr, d_o2.ptr, d_q2.ptr, d_l2.ptr, d_h2.ptr, n, m2, half, 1 << (n - m2), 0) == 0
        permuted = np.ascontiguousarray(evals[perm2])
        exp2 = np.zeros(2 << (n - m2), dtype=np.uint64)
        oracle.oracle_agl_partial_eval_ext2_from_base(permuted.ctypes.data, exp2.ctypes.data, r.ctypes.data, n, m2)
        assert np.array_equal(d_o2.to_numpy(), exp2)


def test_fused_permute_partial_eval_sector_loads_and_unaligned_table(lib, oracle):
    """Fixed variables moved down, the rest in order: four consecutive outputs read one 32-byte sector. The same
    call on a table that starts 8 bytes into its allocation must not use 16-byte loads; one and two outputs
    (no group of four) take the per-output kernels."""
    for n, m, half in ((12, 5, 6), (14, 9, 7), (9, 2, 4), (6, 5, 3), (5, 5, 2)):
        order = list(range(n - m, n)) + list(range(n - m))
        lo, hi = _split_luts(n, order, half)
        x = np.arange(1 << n, dtype=np.int64)
        perm = lo[x & ((1 << half) - 1)].astype(np.int64) | hi[x >> half].astype(np.int64)
        evals = field_elems(930 + n, (1 << n) + 1, Q)
        r = field_elems(931 + n, 2 * m, Q)
        eq = np.zeros(2 << m, dtype=np.uint64)
        oracle.oracle_agl_eq_ext2(r.ctypes.data, m, eq.ctypes.data)
        out_size = 1 << (n - m)
        d_e, d_q = DeviceBuffer.from_numpy(lib, evals), DeviceBuffer.from_numpy(lib, eq)
        d_lo, d_hi = DeviceBuffer.from_numpy(lib, lo), DeviceBuffer.from_numpy(lib, hi)
        d_o = DeviceBuffer(lib, 16 * out_size)
        for shift in (0, 1):
            assert lib.agl_fused_permute_partial_eval_ffi(d_e.ptr + 8 * shift, d_o.ptr, d_q.ptr, d_lo.ptr, d_hi.ptr, n, m, half,
                                                          out_size, 0) == 0
            permuted = np.ascontiguousarray(evals[shift:shift + (1 << n)][perm])
            exp = np.zeros(2 * out_size, dtype=np.uint64)
            oracle.oracle_agl_partial_eval_ext2_from_base(permuted.ctypes.data, exp.ctypes.data, r.ctypes.data, n, m)
            assert np.array_equal(d_o.to_numpy(), exp), (n, m, shift)
