"""The oracle's K = F_q[Theta]/(Theta^8 - 3): the ring identities the reference tests
(zk-torch-4/src/morpheus/field8.rs:193-256) and an independent big-integer product. No GPU."""
import ctypes
import random

import numpy as np

from matrix_b200.inputs import AGL_Q
from oracle import pyoracle

Q = AGL_Q


def _k8(lib, fn, a, b):
    A, B, O = (np.array(x, dtype=np.uint64) for x in (a, b, [0] * 8))
    getattr(lib, fn)(A.ctypes.data, B.ctypes.data, O.ctypes.data)
    return [int(x) for x in O]


def py_mul(a, b):
    out = [0] * 8
    for i in range(8):
        for j in range(8):
            if i + j < 8:
                out[i + j] += a[i] * b[j]
            else:
                out[i + j - 8] += 3 * a[i] * b[j]
    return [x % Q for x in out]


def test_ring_identities_and_product(oracle):
    rnd = random.Random(5)
    el = lambda: [rnd.randrange(Q) for _ in range(8)]
    mul = lambda a, b: _k8(oracle, "oracle_k8_mul", a, b)
    add = lambda a, b: _k8(oracle, "oracle_k8_add", a, b)
    sub = lambda a, b: _k8(oracle, "oracle_k8_sub", a, b)
    for _ in range(40):
        a, b, c = el(), el(), el()
        assert mul(a, b) == py_mul(a, b) == mul(b, a)
        assert mul(a, mul(b, c)) == mul(mul(a, b), c)
        assert mul(a, add(b, c)) == add(mul(a, b), mul(a, c))
        assert sub(a, a) == [0] * 8
    theta = [0, 1, 0, 0, 0, 0, 0, 0]
    p = [1, 0, 0, 0, 0, 0, 0, 0]
    for _ in range(8):
        p = mul(p, theta)
    assert p == [3, 0, 0, 0, 0, 0, 0, 0]
    # extreme words, non-canonical inputs
    big = [2**64 - 1] * 8
    assert mul(big, big) == py_mul([x % Q for x in big], [x % Q for x in big])


def test_eq_table_matches_product(oracle):
    rnd = random.Random(6)
    n = 5
    point = np.array([rnd.randrange(Q) for _ in range(8 * n)], dtype=np.uint64)
    table = np.zeros(8 << n, dtype=np.uint64)
    oracle.oracle_k8_eq_table(point.ctypes.data, n, table.ctypes.data)
    one = [1] + [0] * 7
    total = [0] * 8
    for idx in range(1 << n):
        p = one
        for j in range(n):
            r = [int(x) for x in point[8 * j:8 * j + 8]]
            f = r if (idx >> j) & 1 else [(o - x) % Q for o, x in zip(one, r)]
            p = py_mul(p, f)
        assert [int(x) for x in table[8 * idx:8 * idx + 8]] == p
        total = [(x + y) % Q for x, y in zip(total, p)]
    assert total == one


def test_round_sums_and_fold_are_consistent(oracle):
    """s[0] + s[1] is the sum of the products over the table; folding on r and summing again gives the
    round polynomial at r (degree ntab, interpolated with Python integers)."""
    rnd = random.Random(7)
    ntab, n = 3, 4
    tabs = [np.array([rnd.randrange(Q) for _ in range(8 << n)], dtype=np.uint64) for _ in range(ntab)]
    s = pyoracle.k8_sc_round(tabs, ntab).reshape(ntab + 1, 8)
    total = [0] * 8
    for x in range(1 << n):
        p = [1] + [0] * 7
        for t in tabs:
            p = py_mul(p, [int(v) for v in t[8 * x:8 * x + 8]])
        total = [(a + b) % Q for a, b in zip(total, p)]
    assert [(int(a) + int(b)) % Q for a, b in zip(s[0], s[1])] == total
    r = [rnd.randrange(Q) for _ in range(8)]
    folded = [pyoracle.k8_sc_fold(t, r) for t in tabs]
    s2 = pyoracle.k8_sc_round(folded, ntab).reshape(ntab + 1, 8)
    claim = [(int(a) + int(b)) % Q for a, b in zip(s2[0], s2[1])]
    # Lagrange interpolation of s at r over the nodes 0..ntab, in K
    def k_scale(a, c):
        return [(x * c) % Q for x in a]
    acc = [0] * 8
    for i in range(ntab + 1):
        num, den = [1] + [0] * 7, 1
        for j in range(ntab + 1):
            if j != i:
                num = py_mul(num, [(r[0] - j) % Q] + r[1:])
                den = den * (i - j) % Q
        term = py_mul([int(v) for v in s[i]], k_scale(num, pow(den, Q - 2, Q)))
        acc = [(x + y) % Q for x, y in zip(acc, term)]
    assert acc == claim
