"""Seeded inputs for the link sumcheck tests (shared by the CPU and GPU files)."""
import numpy as np

from matrix_b200.inputs import AGL_Q, field_elems

Q = AGL_Q


def ext(seed, n):
    """n extension elements as 2n canonical words."""
    return np.ascontiguousarray(field_elems(seed, 2 * n, Q))


def sparse_ext(seed, n, density, ternary=False):
    """n extension elements, most of them zero; ternary: values in {-1, 0, 1} embedded in the base field."""
    rng = np.random.default_rng(seed)
    v = ext(seed + 1000, n).reshape(n, 2)
    keep = rng.random(n) < density
    if ternary:
        t = rng.integers(-1, 2, size=n)
        v[:, 0] = np.where(t < 0, np.uint64(Q - 1), t.astype(np.uint64))
        v[:, 1] = 0
    v[~keep] = 0
    return np.ascontiguousarray(v.reshape(-1))


def random_bits(seed, n_bits, density):
    rng = np.random.default_rng(seed)
    b = (rng.random(n_bits) < density).astype(np.uint8)
    words = np.packbits(b.reshape(-1, 64)[:, ::-1], axis=1).view(">u8").astype(np.uint64).reshape(-1)
    return np.ascontiguousarray(words), b


def support_lists(nonzero_pair, extra_seed=None):
    """nonzero_pair: bool [n_commit][half]; returns (list u32, off u64, len u64), with a few zero pairs added."""
    lists, off, ln = [], [], []
    pos = 0
    rng = np.random.default_rng(extra_seed) if extra_seed is not None else None
    for row in nonzero_pair:
        idx = np.nonzero(row)[0]
        if rng is not None and len(row) > 4:
            idx = np.union1d(idx, rng.integers(0, len(row), size=3))
        lists.append(idx.astype(np.uint32))
        off.append(pos)
        ln.append(len(idx))
        pos += len(idx)
    l = np.concatenate(lists) if pos else np.zeros(1, dtype=np.uint32)
    return np.ascontiguousarray(l.astype(np.uint32)), np.array(off, dtype=np.uint64), np.array(ln, dtype=np.uint64)


def to_int(words):
    return [int(x) for x in words]


def e2_mul(a, b):
    return ((a[0] * b[0] + 3 * a[1] * b[1]) % Q, (a[0] * b[1] + a[1] * b[0]) % Q)


def e2_add(a, b):
    return ((a[0] + b[0]) % Q, (a[1] + b[1]) % Q)


def e2_sub(a, b):
    return ((a[0] - b[0]) % Q, (a[1] - b[1]) % Q)


def lagrange_at(vals, r):
    """Value at r of the polynomial with the given values at 0, 1, ..., len - 1 (extension arithmetic)."""
    n = len(vals)
    acc = (0, 0)
    for i in range(n):
        num, den = (1, 0), 1
        for j in range(n):
            if j != i:
                num = e2_mul(num, e2_sub(r, (j, 0)))
                den = den * (i - j) % Q
        inv = pow(den, Q - 2, Q)
        acc = e2_add(acc, e2_mul(e2_mul(num, (inv, 0)), vals[i]))
    return acc
