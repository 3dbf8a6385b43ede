"""The link sumcheck oracle on CPU: its forms against one another, Python integers on a tiny case,
and the sumcheck identity between consecutive rounds."""
import numpy as np

from oracle import pyoracle as po
from .link_cases import Q, e2_add, e2_mul, e2_sub, ext, lagrange_at, random_bits, sparse_ext, support_lists


def _range_poly(u):
    return e2_sub(e2_mul(e2_mul(u, u), u), u)


def test_round_message_against_python_integers():
    half, nc = 4, 2
    w, om = ext(1, nc * 2 * half), ext(2, nc * 2 * half)
    eq, tags = ext(3, half), ext(4, nc)
    got = po.link_round(eq, tags, half, nc, 0, w=w, omega=om, w_stride=2 * half, omega_stride=2 * half)
    E = lambda a, i: (int(a[2 * i]), int(a[2 * i + 1]))
    want = [(0, 0)] * 7
    for e in range(nc):
        acc = [(0, 0)] * 7
        for i in range(half):
            wl, wh = E(w, e * 2 * half + i), E(w, e * 2 * half + half + i)
            ol, oh = E(om, e * 2 * half + i), E(om, e * 2 * half + half + i)
            for k in range(4):
                wk = e2_add(wl, e2_mul((k, 0), e2_sub(wh, wl)))
                acc[k] = e2_add(acc[k], e2_mul(E(eq, i), _range_poly(wk)))
                if k < 3:
                    ok = e2_add(ol, e2_mul((k, 0), e2_sub(oh, ol)))
                    acc[4 + k] = e2_add(acc[4 + k], e2_mul(ok, wk))
        for k in range(7):
            want[k] = e2_add(want[k], e2_mul(E(tags, e), acc[k]) if k < 4 else acc[k])
    assert [E(got, k) for k in range(7)] == want


def test_forms_agree():
    """Bits against their expansion, lists against the dense sweep, first-round shortcut on ternary witnesses."""
    half, nc = 128, 3
    stride = 2 * half
    words, b = random_bits(5, nc * stride, 0.1)
    om, eq, tags = ext(6, nc * stride), ext(7, half), ext(8, nc)
    table = po.link_expand_bits(words)
    assert [int(x) for x in table[0::2]] == [int(x) for x in b] and not table[1::2].any()
    dense = po.link_round(eq, tags, half, nc, 1, w=table, omega=om, w_stride=stride, omega_stride=stride)
    bits = po.link_round(eq, tags, half, nc, 1, bits=words, omega=om, bits_stride_words=stride // 64, omega_stride=stride)
    assert np.array_equal(dense, bits) and not dense[:4].any()
    full = po.link_round(eq, tags, half, nc, 0, w=table, omega=om, w_stride=stride, omega_stride=stride)
    assert np.array_equal(full, dense)   # R vanishes on {0, 1}: the shortcut changes nothing
    pair = b.reshape(nc, 2, half).any(axis=1)
    lists = support_lists(pair, extra_seed=1)
    eq_g = np.concatenate([eq.reshape(half, 2)[lists[0][int(o):int(o) + int(n)]] for o, n in zip(lists[1], lists[2])]).reshape(-1)
    listed = po.link_round(np.ascontiguousarray(eq_g), tags, half, nc, 1, bits=words, omega=om, lists=lists,
                           bits_stride_words=stride // 64, omega_stride=stride)
    assert np.array_equal(listed, dense)
    wt = sparse_ext(9, nc * stride, 0.2, ternary=True)
    a = po.link_round(eq, tags, half, nc, 1, w=wt, omega=om, w_stride=stride, omega_stride=stride)
    c = po.link_round(eq, tags, half, nc, 0, w=wt, omega=om, w_stride=stride, omega_stride=stride)
    assert np.array_equal(a, c)


def test_eval_half_satisfies_the_sumcheck_identity():
    """E_{i+1}(0) + E_{i+1}(1) = E_i(r) after folding both tables with r."""
    half, nc = 64, 2
    stride = 2 * half
    w, om = sparse_ext(10, nc * stride, 0.5), ext(11, nc * stride)
    tags = ext(12, nc)
    for rnd in range(3):
        eq = ext(13 + rnd, half)
        msg = po.link_round(eq, tags, half, nc, 0, w=w, omega=om, w_stride=stride, omega_stride=stride)
        E = [(int(msg[8 + 2 * k]), int(msg[9 + 2 * k])) for k in range(3)]
        r = ext(20 + rnd, 1)
        w = po.link_fold_rows(w, stride, half, nc, r)
        om = po.link_fold_rows(om, stride, half, nc, r)
        half //= 2
        nxt = po.link_round(ext(30, half), tags, half, nc, 0, w=w, omega=om, w_stride=stride, omega_stride=stride)
        s = e2_add((int(nxt[8]), int(nxt[9])), (int(nxt[10]), int(nxt[11])))
        assert s == lagrange_at(E, (int(r[0]), int(r[1])))


def test_eq_table_most_significant_variable_first():
    pt = ext(14, 5)
    table = np.zeros(2 * 32, dtype=np.uint64)
    table[0] = 1
    span = 1
    for k in reversed(range(5)):   # the table is built from the last variable up (pcs/link.rs:199-213)
        table = po.link_eq_expand(table, span, pt[2 * k:2 * k + 2])
        span *= 2
    lst = np.arange(32, dtype=np.uint32)
    assert np.array_equal(table, po.link_eq_gather(pt, 5, lst))
    # index 0b10000 has only the first variable set
    want = (1, 0)
    for k in range(5):
        r = (int(pt[2 * k]), int(pt[2 * k + 1]))
        want = e2_mul(want, r if k == 0 else e2_sub((1, 0), r))
    assert (int(table[32]), int(table[33])) == want
