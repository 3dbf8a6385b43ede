"""GPU parity of the batched same-point sumcheck family over almost-Goldilocks Ext2: every entry point against
Python-integer arithmetic following the reference kernels (cuda_almost_goldilocks/almost_sumcheck_prover.cuh:233-1007),
and the three layouts (interleaved, shared eq, factored eq) against each other on a whole sumcheck."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from matrix_b200.inputs import AGL_Q, field_elems
from oracle import pyoracle

pytestmark = pytest.mark.gpu
Q = AGL_Q
W = 3


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def emul(a, b):
    return ((a[0] * b[0] + W * a[1] * b[1]) % Q, (a[0] * b[1] + a[1] * b[0]) % Q)


def eadd(a, b):
    return ((a[0] + b[0]) % Q, (a[1] + b[1]) % Q)


def esub(a, b):
    return ((a[0] - b[0]) % Q, (a[1] - b[1]) % Q)


def pairs(arr):
    return [(int(arr[2 * i]), int(arr[2 * i + 1])) for i in range(len(arr) // 2)]


def message(eq, f, half):
    """m(0), m(1), m(2) of sum_y eq f over pairs (2y, 2y + 1)."""
    m = [(0, 0)] * 3
    for y in range(half):
        e0, e1, f0, f1 = eq[2 * y], eq[2 * y + 1], f[2 * y], f[2 * y + 1]
        m[0] = eadd(m[0], emul(e0, f0))
        m[1] = eadd(m[1], emul(e1, f1))
        m[2] = eadd(m[2], emul(esub(eadd(e1, e1), e0), esub(eadd(f1, f1), f0)))
    return m


def fold(t, r, half):
    return [eadd(t[2 * y], emul(r, esub(t[2 * y + 1], t[2 * y]))) for y in range(half)]


def sum_partials(partial, blocks, leaves, nv):
    p = partial.reshape(blocks, leaves, nv, 2)
    return [[tuple(int(sum(int(p[b, l, c, k]) for b in range(blocks)) % Q) for k in range(2)) for c in range(nv)] for l in range(leaves)]


def packed_bits(rng, leaves, n):
    words = (n + 63) // 64
    arr = rng.integers(0, 2**63, size=leaves * words, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=leaves * words, dtype=np.uint64)
    bits = [[(int(arr[l * words + (i >> 6)]) >> (i & 63)) & 1 for i in range(n)] for l in range(leaves)]
    return arr, bits, words


@pytest.mark.parametrize("log_n,leaves,blocks", [(1, 1, 1), (4, 3, 2), (9, 5, 7)])
def test_interleaved_message_fold_and_binary_round0(lib, log_n, leaves, blocks):
    n, half = 1 << log_n, 1 << (log_n - 1)
    rng = np.random.default_rng(log_n)
    polys = field_elems(10 + log_n, leaves * 4 * n, Q)
    d_polys = DeviceBuffer.from_numpy(lib, polys)
    d_part = DeviceBuffer(lib, 8 * blocks * leaves * 6)
    assert lib.aext2_sumcheck_batched_round_message_ffi(d_polys.ptr, d_part.ptr, n, half, leaves, blocks) == 0
    lib.cuda_device_synchronize()
    got = sum_partials(d_part.to_numpy(), blocks, leaves, 3)
    tabs = [(pairs(polys[l * 4 * n:l * 4 * n + 2 * n]), pairs(polys[l * 4 * n + 2 * n:(l + 1) * 4 * n])) for l in range(leaves)]
    for l in range(leaves):
        assert got[l] == message(tabs[l][0], tabs[l][1], half)
    r = (int(field_elems(77, 1, Q)[0]), int(field_elems(78, 1, Q)[0]))
    d_out = DeviceBuffer(lib, polys.nbytes)
    assert lib.aext2_sumcheck_batched_fold_ffi(d_polys.ptr, d_out.ptr, r[0], r[1], n, half, leaves) == 0
    lib.cuda_device_synchronize()
    out = d_out.to_numpy()
    for l in range(leaves):
        for t in range(2):
            base = l * 4 * n + t * 2 * n
            assert pairs(out[base:base + 2 * half]) == fold(tabs[l][t], r, half)
    # binary f: lift, then round 0 without the lift
    packed, bits, words = packed_bits(rng, leaves, n)
    d_packed = DeviceBuffer.from_numpy(lib, packed)
    assert lib.aext2_batched_lift_binary_ffi(d_packed.ptr, d_polys.ptr, n, leaves, words) == 0
    lib.cuda_device_synchronize()
    lifted = d_polys.to_numpy()
    for l in range(leaves):
        assert pairs(lifted[l * 4 * n + 2 * n:(l + 1) * 4 * n]) == [(b, 0) for b in bits[l]]
        assert np.array_equal(lifted[l * 4 * n:l * 4 * n + 2 * n], polys[l * 4 * n:l * 4 * n + 2 * n])  # eq slot untouched
    assert lib.aext2_sumcheck_batched_round_message_ffi(d_polys.ptr, d_part.ptr, n, half, leaves, blocks) == 0
    lib.cuda_device_synchronize()
    via_lift = sum_partials(d_part.to_numpy(), blocks, leaves, 3)
    d_polys0 = DeviceBuffer.from_numpy(lib, polys)  # f slot holds arbitrary data: it must be ignored
    assert lib.aext2_sumcheck_batched_round0_binary_msg_ffi(d_polys0.ptr, d_packed.ptr, d_part.ptr, n, half, leaves, blocks, words) == 0
    lib.cuda_device_synchronize()
    assert sum_partials(d_part.to_numpy(), blocks, leaves, 3) == via_lift
    assert lib.aext2_sumcheck_batched_fold_ffi(d_polys.ptr, d_out.ptr, r[0], r[1], n, half, leaves) == 0
    lib.cuda_device_synchronize()
    exp = d_out.to_numpy().copy()
    d_out2 = DeviceBuffer(lib, polys.nbytes)
    assert lib.aext2_sumcheck_batched_round0_binary_fold_ffi(d_polys0.ptr, d_packed.ptr, d_out2.ptr, r[0], r[1], n, half, leaves, words) == 0
    lib.cuda_device_synchronize()
    got2 = d_out2.to_numpy()
    for l in range(leaves):
        for t in range(2):
            base = l * 4 * n + t * 2 * n
            assert np.array_equal(got2[base:base + 2 * half], exp[base:base + 2 * half])


def test_lifts_selective_add_and_fu(lib):
    rng = np.random.default_rng(5)
    n, leaves = 300, 6
    packed, bits, words = packed_bits(rng, leaves, n)
    neg_packed, nbits, _ = packed_bits(rng, leaves, n)
    neg_packed &= ~packed
    nbits = [[(int(neg_packed[l * words + (i >> 6)]) >> (i & 63)) & 1 for i in range(n)] for l in range(leaves)]
    d_p, d_n = DeviceBuffer.from_numpy(lib, packed), DeviceBuffer.from_numpy(lib, neg_packed)
    d_f = DeviceBuffer(lib, 16 * n * leaves)
    assert lib.aext2_lift_binary_contig_ffi(d_p.ptr, d_f.ptr, n, leaves, words) == 0
    lib.cuda_device_synchronize()
    f = d_f.to_numpy()
    for l in range(leaves):
        assert pairs(f[l * 2 * n:(l + 1) * 2 * n]) == [(b, 0) for b in bits[l]]
    d_polys = DeviceBuffer.from_numpy(lib, np.zeros(4 * n * leaves, dtype=np.uint64))
    assert lib.aext2_batched_lift_ternary_single_ffi(d_p.ptr, d_n.ptr, d_polys.ptr, n, leaves, words) == 0
    lib.cuda_device_synchronize()
    t = d_polys.to_numpy()
    for l in range(leaves):
        assert pairs(t[l * 4 * n + 2 * n:(l + 1) * 4 * n]) == [((p - m) % Q, 0) for p, m in zip(bits[l], nbits[l])]
    # selective add
    eq = field_elems(9, 2 * n, Q)
    d_eq = DeviceBuffer.from_numpy(lib, eq)
    blocks = 3
    d_part = DeviceBuffer(lib, 8 * blocks * leaves * 2)
    assert lib.aext2_selective_add_batched_planes_ffi(d_eq.ptr, d_p.ptr, d_part.ptr, n, leaves, words, blocks) == 0
    lib.cuda_device_synchronize()
    got = sum_partials(d_part.to_numpy(), blocks, leaves, 1)
    eqp = pairs(eq)
    for l in range(leaves):
        s = (0, 0)
        for i in range(n):
            if bits[l][i]:
                s = eadd(s, eqp[i])
        assert got[l][0] == s
    # F_u: leaves grouped by point
    alphas = field_elems(12, 2 * leaves, Q)
    ap = pairs(alphas)
    order = np.array([4, 0, 2, 5, 1, 3], dtype=np.int32)
    offsets = np.array([0, 2, 2, 6], dtype=np.int32)  # point 1 has no leaves
    d_a, d_o, d_off = DeviceBuffer.from_numpy(lib, alphas), DeviceBuffer.from_numpy(lib, order), DeviceBuffer.from_numpy(lib, offsets)
    d_fu = DeviceBuffer(lib, 16 * n * 3)
    for ternary in (False, True):
        if ternary:
            assert lib.aext2_build_fu_ternary_ffi(d_p.ptr, d_n.ptr, d_a.ptr, d_o.ptr, d_off.ptr, d_fu.ptr, n, 3, words) == 0
        else:
            assert lib.aext2_build_fu_ffi(d_p.ptr, d_a.ptr, d_o.ptr, d_off.ptr, d_fu.ptr, n, 3, words) == 0
        lib.cuda_device_synchronize()
        fu = d_fu.to_numpy()
        for u in range(3):
            exp = []
            for x in range(n):
                acc = (0, 0)
                for s in range(offsets[u], offsets[u + 1]):
                    leaf = int(order[s])
                    if bits[leaf][x]:
                        acc = eadd(acc, ap[leaf])
                    if ternary and nbits[leaf][x]:
                        acc = esub(acc, ap[leaf])
                exp.append(acc)
            assert pairs(fu[u * 2 * n:(u + 1) * 2 * n]) == exp


def test_three_layouts_agree_on_a_whole_sumcheck(lib):
    """One sumcheck of sum_x eq(R_u, x) F_u(x) per point, driven through the shared-eq entry points (message, fold of
    eq and f) and through the factored form (suffix tables, A / B sums, prefix scalar on the host,
    almost_sumcheck_prover.cuh:481-497): identical round messages; eq tables from the batched and the stream builders."""
    log_n, uniq = 7, 2
    n = 1 << log_n
    points = field_elems(31, 2 * log_n * uniq, Q)
    fu = field_elems(32, 2 * n * uniq, Q)
    d_r = DeviceBuffer.from_numpy(lib, points)
    d_a, d_b = DeviceBuffer(lib, 16 * n * uniq), DeviceBuffer(lib, 16 * n * uniq)
    res = ctypes.c_void_p()
    assert lib.aext2_eq_dp_all_batched_ffi(d_r.ptr, d_a.ptr, d_b.ptr, log_n, uniq, n, ctypes.byref(res), None) == 0
    lib.cuda_device_synchronize()
    eq_dev = np.empty(2 * n * uniq, dtype=np.uint64)
    assert lib.cuda_memcpy_dtoh(eq_dev.ctypes.data, res.value, eq_dev.nbytes) == 0
    oracle = pyoracle.load()
    for u in range(uniq):
        exp = np.zeros(2 * n, dtype=np.uint64)
        oracle.oracle_agl_eq_ext2(points[u * 2 * log_n:].ctypes.data, log_n, exp.ctypes.data)
        assert np.array_equal(eq_dev[u * 2 * n:(u + 1) * 2 * n], exp)
    st = ctypes.c_void_p()
    assert lib.cuda_stream_create(ctypes.byref(st)) == 0
    d_c, d_d = DeviceBuffer(lib, 16 * n), DeviceBuffer(lib, 16 * n)
    assert lib.aext2_eq_dp_all_stream_ffi(d_r.ptr, d_c.ptr, d_d.ptr, log_n, ctypes.byref(res), st) == 0
    assert lib.cuda_stream_synchronize(st) == 0
    one = np.empty(2 * n, dtype=np.uint64)
    assert lib.cuda_memcpy_dtoh(one.ctypes.data, res.value, one.nbytes) == 0
    assert np.array_equal(one, eq_dev[:2 * n])
    lib.cuda_stream_destroy(st)

    # suffix tables
    stride = 2 * n
    d_suf = DeviceBuffer(lib, 8 * stride * uniq)
    assert lib.aext2_eq_suffix_dp_ffi(d_r.ptr, d_suf.ptr, log_n, uniq, stride) == 0
    lib.cuda_device_synchronize()
    suf = d_suf.to_numpy()
    pts = [pairs(points[u * 2 * log_n:(u + 1) * 2 * log_n]) for u in range(uniq)]
    for u in range(uniq):
        for t in range(1, log_n + 1):
            size, off = 1 << (log_n - t), (1 << (log_n - t)) - 1
            got = pairs(suf[u * stride + 2 * off:u * stride + 2 * (off + size)])
            for y in range(size):
                e = (1, 0)
                for i in range(t, log_n):
                    bit = (y >> (i - t)) & 1
                    e = emul(e, pts[u][i] if bit else esub((1, 0), pts[u][i]))
                assert got[y] == e

    # rounds: shared-eq path on device tables vs factored path
    leaf_map = np.arange(uniq, dtype=np.int32)
    d_map = DeviceBuffer.from_numpy(lib, leaf_map)
    d_eq, d_eq2 = DeviceBuffer.from_numpy(lib, eq_dev), DeviceBuffer(lib, eq_dev.nbytes)
    d_f, d_f2 = DeviceBuffer.from_numpy(lib, fu), DeviceBuffer(lib, fu.nbytes)
    d_ff, d_ff2 = DeviceBuffer.from_numpy(lib, fu), DeviceBuffer(lib, fu.nbytes)  # f tables of the factored path
    blocks = 4
    d_part = DeviceBuffer(lib, 8 * blocks * uniq * 6)
    prefix = [(1, 0)] * uniq
    half = n // 2
    for t in range(log_n):
        assert lib.aext2_sharedeq_msg_ffi(d_eq.ptr, d_f.ptr, d_map.ptr, d_part.ptr, n, half, uniq, blocks) == 0
        lib.cuda_device_synchronize()
        shared_msgs = sum_partials(d_part.to_numpy()[:blocks * uniq * 6], blocks, uniq, 3)
        off = (1 << (log_n - t - 1)) - 1  # eqsuf_{t+1}
        assert lib.aext2_sharedeq_factored_msg_ffi(d_suf.ptr, d_ff.ptr, d_part.ptr, off, stride, 2 * n, half, uniq, blocks) == 0
        lib.cuda_device_synchronize()
        ab = sum_partials(d_part.to_numpy()[:blocks * uniq * 4], blocks, uniq, 2)
        for u in range(uniq):
            A, B, R, p = ab[u][0], ab[u][1], pts[u][t], prefix[u]
            t0 = emul(emul(p, esub((1, 0), R)), A)
            t1 = emul(emul(p, R), B)
            t2 = emul(emul(p, esub(emul((3, 0), R), (1, 0))), esub(eadd(B, B), A))
            assert shared_msgs[u] == [t0, t1, t2]
        r = (int(field_elems(90 + t, 1, Q)[0]), int(field_elems(190 + t, 1, Q)[0]))
        assert lib.aext2_fold_single_ffi(d_eq.ptr, d_eq2.ptr, r[0], r[1], n, half, uniq) == 0
        assert lib.aext2_fold_single_ffi(d_f.ptr, d_f2.ptr, r[0], r[1], n, half, uniq) == 0
        assert lib.aext2_fold_single_ffi(d_ff.ptr, d_ff2.ptr, r[0], r[1], n, half, uniq) == 0
        d_eq, d_eq2, d_f, d_f2, d_ff, d_ff2 = d_eq2, d_eq, d_f2, d_f, d_ff2, d_ff
        for u in range(uniq):
            R = pts[u][t]
            prefix[u] = emul(prefix[u], eadd(emul(r, R), emul(esub((1, 0), r), esub((1, 0), R))))
        half //= 2
        if half == 0:
            break
