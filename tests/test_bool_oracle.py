"""The sparse boolean-check oracle on CPU: against a dense evaluation of the same sum, and the sumcheck
identities between rounds."""
import numpy as np

from oracle import pyoracle as po
from .bool_cases import ext, fold_eq, make_terms, ones
from .link_cases import Q, e2_add, e2_mul, e2_sub, lagrange_at


def test_rounds_against_dense_tables_and_identities():
    arity, n_terms = 6, 7
    idx, off = make_terms(1, arity, n_terms, 0.2)
    val, w, eq = ones(len(idx)), ext(2, n_terms), ext(3, 1 << arity)
    # dense tables v_t
    size = 1 << arity
    dense = [[(0, 0)] * size for _ in range(n_terms)]
    for t in range(n_terms):
        for i in range(off[t], off[t + 1]):
            dense[t][int(idx[i])] = (1, 0)
    E = lambda a, i: (int(a[2 * i]), int(a[2 * i + 1]))
    prev = None
    for rnd in range(arity):
        flags, gid, msg, total = po.bool_round(idx, val, off, w, eq)
        m = [E(msg, k) for k in range(4)]
        half = size // 2
        want = [(0, 0)] * 4
        for t in range(n_terms):
            for y in range(half):
                for c in range(4):
                    a = e2_add(dense[t][2 * y], e2_mul((c, 0), e2_sub(dense[t][2 * y + 1], dense[t][2 * y])))
                    e = e2_add(E(eq, 2 * y), e2_mul((c, 0), e2_sub(E(eq, 2 * y + 1), E(eq, 2 * y))))
                    want[c] = e2_add(want[c], e2_mul(e2_mul(E(w, t), e2_mul(a, e2_sub(a, (1, 0)))), e))
        assert m == want
        if prev is None:
            assert e2_add(m[0], m[1]) == (0, 0)      # binary tables: the claimed sum is zero
        else:
            assert e2_add(m[0], m[1]) == prev
        r = ext(10 + rnd, 1)
        prev = lagrange_at(m, (int(r[0]), int(r[1])))
        idx, val, off = po.bool_fold(idx, val, flags, gid, off, r, total)
        off = off.copy()
        for t in range(n_terms):
            dense[t] = [e2_add(dense[t][2 * y], e2_mul((int(r[0]), int(r[1])), e2_sub(dense[t][2 * y + 1], dense[t][2 * y])))
                        for y in range(half)]
        eq = fold_eq(eq, r, Q)
        size = half
        # the sparse lists hold exactly the nonzero folded values
        for t in range(n_terms):
            got = {int(idx[i]): E(val, i) for i in range(off[t], off[t + 1])}
            assert all(dense[t][p] == v for p, v in got.items())
            assert all(v == (0, 0) or p in got for p, v in enumerate(dense[t]))
    assert all(off[t + 1] - off[t] <= 1 for t in range(n_terms))
