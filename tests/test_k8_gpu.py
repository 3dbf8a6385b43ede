"""GPU parity of the K = F_q[Theta]/(Theta^8 - 3) product sumcheck and its table helpers against
the CPU oracle, through the C-ABI. Bit-exact."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from matrix_b200.inputs import AGL_Q, field_elems, splitmix64
from oracle import pyoracle

pytestmark = pytest.mark.gpu
Q = AGL_Q


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def _tables(seed, ntab, n, raw=False):
    """ntab tables of 2^n elements; raw: any 64-bit words (non-canonical representatives)."""
    gen = (lambda s, w: splitmix64(s, w)) if raw else (lambda s, w: field_elems(s, w, Q))
    return [np.ascontiguousarray(gen(seed + j, 8 << n)) for j in range(ntab)]


def _ptrs(bufs):
    return (ctypes.c_void_p * len(bufs))(*[b.ptr for b in bufs])


@pytest.mark.parametrize("ntab,d,n,raw", [(1, 1, 1, False), (2, 2, 1, False), (2, 2, 5, False), (3, 3, 9, False),
                                         (6, 6, 7, False), (4, 6, 6, True), (3, 2, 12, False), (2, 3, 14, True)])
def test_round_sums_match_oracle(lib, ntab, d, n, raw):
    tabs = _tables(100 + n, ntab, n, raw)
    dev = [DeviceBuffer.from_numpy(lib, t) for t in tabs]
    out = np.zeros((d + 1) * 8, dtype=np.uint64)
    assert lib.agl_mpiop_sc_round(_ptrs(dev), ntab, 1 << n, d, out.ctypes.data) == 0
    assert np.array_equal(out, pyoracle.k8_sc_round(tabs, d))
    # twice in a row: the ticket counter and scratch are left clean
    out2 = np.zeros_like(out)
    assert lib.agl_mpiop_sc_round(_ptrs(dev), ntab, 1 << n, d, out2.ctypes.data) == 0
    assert np.array_equal(out2, out)


def test_round_argument_errors(lib):
    tabs = _tables(7, 2, 3)
    dev = [DeviceBuffer.from_numpy(lib, t) for t in tabs]
    out = np.zeros(64, dtype=np.uint64)
    assert lib.agl_mpiop_sc_round(_ptrs(dev * 4), 8, 8, 2, out.ctypes.data) == -3
    assert lib.agl_mpiop_sc_round(_ptrs(dev), 2, 8, 7, out.ctypes.data) == -3
    assert lib.agl_mpiop_sc_round(_ptrs(dev), 2, 0, 2, out.ctypes.data) != 0
    assert lib.agl_mpiop_sc_fold_round(_ptrs(dev), _ptrs(dev), 2, 2, out.ctypes.data, 2, out.ctypes.data) == -3


@pytest.mark.parametrize("n,raw", [(1, False), (2, True), (6, False), (13, True)])
def test_fold_matches_oracle(lib, n, raw):
    tab = _tables(200 + n, 1, n, raw)[0]
    r = field_elems(9, 8, Q)
    d_in, d_out = DeviceBuffer.from_numpy(lib, tab), DeviceBuffer(lib, 64 << (n - 1))
    assert lib.agl_mpiop_sc_fold(d_in.ptr, d_out.ptr, 1 << n, r.ctypes.data) == 0
    lib.cuda_device_synchronize()
    assert np.array_equal(d_out.to_numpy(), pyoracle.k8_sc_fold(tab, r))


@pytest.mark.parametrize("ntab,d,n", [(2, 2, 2), (3, 3, 8), (6, 6, 6), (2, 4, 13)])
def test_fused_fold_round_matches_oracle(lib, ntab, d, n):
    tabs = _tables(300 + n, ntab, n)
    r = field_elems(11, 8, Q)
    dev = [DeviceBuffer.from_numpy(lib, t) for t in tabs]
    outs = [DeviceBuffer(lib, 64 << (n - 1)) for _ in range(ntab)]
    sums = np.zeros((d + 1) * 8, dtype=np.uint64)
    assert lib.agl_mpiop_sc_fold_round(_ptrs(dev), _ptrs(outs), ntab, 1 << n, r.ctypes.data, d, sums.ctypes.data) == 0
    folded = [pyoracle.k8_sc_fold(t, r) for t in tabs]
    for o, f in zip(outs, folded):
        assert np.array_equal(o.to_numpy(), f)
    assert np.array_equal(sums, pyoracle.k8_sc_round(folded, d))


def test_whole_sumcheck_round_trip(lib):
    """Rounds chained the way zk-torch-4/src/morpheus/piop/mod.rs:785-840 drives them: round sums, then
    fused fold + next sums, down to length 2; every round satisfies s(0) + s(1) = claim with the claim
    interpolated in the oracle's arithmetic."""
    ntab, n = 3, 10
    tabs = _tables(400, ntab, n)
    cur = [DeviceBuffer.from_numpy(lib, t) for t in tabs]
    host = tabs
    sums = np.zeros((ntab + 1) * 8, dtype=np.uint64)
    assert lib.agl_mpiop_sc_round(_ptrs(cur), ntab, 1 << n, ntab, sums.ctypes.data) == 0
    length = 1 << n
    for i in range(n - 1):
        assert np.array_equal(sums, pyoracle.k8_sc_round(host, ntab))
        r = field_elems(500 + i, 8, Q)
        nxt = [DeviceBuffer(lib, 64 * (length // 2)) for _ in range(ntab)]
        assert lib.agl_mpiop_sc_fold_round(_ptrs(cur), _ptrs(nxt), ntab, length, r.ctypes.data, ntab, sums.ctypes.data) == 0
        host = [pyoracle.k8_sc_fold(t, r) for t in host]
        cur, length = nxt, length // 2
    assert length == 2 and np.array_equal(sums, pyoracle.k8_sc_round(host, ntab))


@pytest.mark.parametrize("n", [0, 1, 2, 7, 12])
def test_eq_table_matches_oracle(lib, n):
    point = field_elems(600 + n, 8 * max(n, 1), Q)
    d_out = DeviceBuffer(lib, 64 << n)
    assert lib.agl_mpiop_eq(point.ctypes.data, n, d_out.ptr) == 0
    lib.cuda_device_synchronize()
    exp = np.zeros(8 << n, dtype=np.uint64)
    pyoracle.load().oracle_k8_eq_table(point.ctypes.data, n, exp.ctypes.data)
    assert np.array_equal(d_out.to_numpy(), exp)


def test_eq_outer_axpy_lift(lib):
    oracle = pyoracle.load()
    nlo, nhi = 5, 4
    plo, phi = field_elems(21, 8 * nlo, Q), field_elems(22, 8 * nhi, Q)
    d_lo, d_hi, d_out = DeviceBuffer(lib, 64 << nlo), DeviceBuffer(lib, 64 << nhi), DeviceBuffer(lib, 64 << (nlo + nhi))
    assert lib.agl_mpiop_eq(plo.ctypes.data, nlo, d_lo.ptr) == 0
    assert lib.agl_mpiop_eq(phi.ctypes.data, nhi, d_hi.ptr) == 0
    assert lib.agl_mpiop_eq_outer(d_lo.ptr, nlo, d_hi.ptr, nhi, d_out.ptr) == 0
    lib.cuda_device_synchronize()
    full = np.zeros(8 << (nlo + nhi), dtype=np.uint64)
    oracle.oracle_k8_eq_table(np.concatenate([plo, phi]).ctypes.data, nlo + nhi, full.ctypes.data)
    assert np.array_equal(d_out.to_numpy(), full)
    # axpy
    n = 777
    a, b, c = splitmix64(31, 8 * n), field_elems(32, 8 * n, Q), field_elems(33, 8, Q)
    d_a, d_b = DeviceBuffer.from_numpy(lib, a), DeviceBuffer.from_numpy(lib, b)
    assert lib.agl_mpiop_axpy(d_a.ptr, d_b.ptr, n, c.ctypes.data) == 0
    lib.cuda_device_synchronize()
    exp = a.copy()
    oracle.oracle_k8_axpy(exp.ctypes.data, b.ctypes.data, n, c.ctypes.data)
    assert np.array_equal(d_a.to_numpy(), exp)
    # lift
    base = splitmix64(34, n)
    d_base, d_k = DeviceBuffer.from_numpy(lib, base), DeviceBuffer(lib, 64 * n)
    assert lib.agl_mpiop_lift(d_base.ptr, n, d_k.ptr) == 0
    lib.cuda_device_synchronize()
    got = d_k.to_numpy().reshape(n, 8)
    assert np.array_equal(got[:, 0], base % np.uint64(Q)) and not got[:, 1:].any()


def _py_kmul_base(e, v):
    return [(int(x) * int(v)) % Q for x in e]


def test_partial_eval_mle_gather_lookup(lib):
    oracle = pyoracle.load()
    rng = np.random.default_rng(3)
    # partial evaluation over a permuted split of 9 variables: 4 stay, 5 are bound
    n = 9
    perm = rng.permutation(n)
    rest_pos, fix_pos = np.array(perm[:4], dtype=np.int32), np.array(perm[4:], dtype=np.int32)
    vals = field_elems(50, 1 << n, Q)
    vals[::3] = 0
    vals[1::5] = 1
    point = field_elems(51, 8 * 5, Q)
    e = np.zeros(8 << 5, dtype=np.uint64)
    oracle.oracle_k8_eq_table(point.ctypes.data, 5, e.ctypes.data)
    d_v, d_e, d_o = DeviceBuffer.from_numpy(lib, vals), DeviceBuffer.from_numpy(lib, e), DeviceBuffer(lib, 64 << 4)
    assert lib.agl_mpiop_pe(d_v.ptr, rest_pos.ctypes.data, 4, fix_pos.ctypes.data, 5, d_e.ptr, d_o.ptr) == 0
    lib.cuda_device_synchronize()
    got = d_o.to_numpy().reshape(16, 8)
    dep = lambda x, pos: sum(((x >> j) & 1) << int(pos[j]) for j in range(len(pos)))
    for r in range(16):
        acc = [0] * 8
        for f in range(32):
            v = int(vals[dep(r, rest_pos) | dep(f, fix_pos)])
            acc = [(a + int(x) * v) % Q for a, x in zip(acc, e[8 * f:8 * f + 8])]
        assert [int(x) for x in got[r]] == acc
    # multilinear extension at a K point, several sizes (n = 0, odd, even)
    for nn in (0, 1, 7, 12):
        vv = field_elems(60 + nn, 1 << nn, Q)
        pt = field_elems(70 + nn, 8 * max(nn, 1), Q)
        table = np.zeros(8 << nn, dtype=np.uint64)
        oracle.oracle_k8_eq_table(pt.ctypes.data, nn, table.ctypes.data)
        exp = [0] * 8
        for x in range(1 << nn):
            exp = [(a + int(t) * int(vv[x])) % Q for a, t in zip(exp, table[8 * x:8 * x + 8])]
        d_vv = DeviceBuffer.from_numpy(lib, vv)
        out = np.zeros(8, dtype=np.uint64)
        assert lib.agl_mpiop_mle(d_vv.ptr, pt.ctypes.data, nn, out.ctypes.data) == 0
        assert [int(x) for x in out] == exp
    # gather and selector lookup
    src = field_elems(80, 8 << 6, Q)
    pos = np.array([5, 0, 9, 3, 7, 2], dtype=np.int32)
    nout = 1 << 10
    d_s, d_g = DeviceBuffer.from_numpy(lib, src), DeviceBuffer(lib, 64 * nout)
    assert lib.agl_mpiop_gather(d_s.ptr, pos.ctypes.data, 6, nout, d_g.ptr) == 0
    lib.cuda_device_synchronize()
    g = d_g.to_numpy().reshape(nout, 8)
    for x in range(0, nout, 37):
        idx = sum(((x >> int(pos[j])) & 1) << j for j in range(6))
        assert np.array_equal(g[x], src[8 * idx:8 * idx + 8])
    sel = rng.integers(0, 2**63, size=500, dtype=np.uint64)
    d_sel, d_l = DeviceBuffer.from_numpy(lib, sel), DeviceBuffer(lib, 64 * 500)
    assert lib.agl_mpiop_sel_lookup(d_sel.ptr, 500, 7, 63, d_s.ptr, d_l.ptr) == 0
    lib.cuda_device_synchronize()
    look = d_l.to_numpy().reshape(500, 8)
    for i in range(0, 500, 13):
        k = (int(sel[i]) >> 7) & 63
        assert np.array_equal(look[i], src[8 * k:8 * k + 8])
