"""Seeded inputs for the sparse boolean-check sumcheck tests."""
import numpy as np

from .link_cases import ext


def make_terms(seed, arity, n_terms, density, with_empty=True):
    """Sorted unique positions below 2^arity per term, some terms empty; returns (idx u32, term_off u32)."""
    rng = np.random.default_rng(seed)
    segs = []
    for t in range(n_terms):
        if with_empty and t % 5 == 3:
            segs.append(np.zeros(0, dtype=np.uint32))
            continue
        k = max(1, int(density * (1 << arity)))
        pos = np.unique(rng.integers(0, 1 << arity, size=k, dtype=np.uint64)).astype(np.uint32)
        if t % 3 == 0 and len(pos) > 2:      # force a few adjacent pairs and a pair straddling nothing
            pos = np.unique(np.concatenate([pos, (pos[:len(pos) // 2] ^ np.uint32(1))])).astype(np.uint32)
        segs.append(pos)
    off = np.zeros(n_terms + 1, dtype=np.uint32)
    off[1:] = np.cumsum([len(s) for s in segs])
    idx = np.concatenate(segs) if off[-1] else np.zeros(0, dtype=np.uint32)
    return np.ascontiguousarray(idx.astype(np.uint32)), off


def ones(n):
    v = np.zeros(2 * n, dtype=np.uint64)
    v[0::2] = 1
    return v


def fold_eq(eq, r, q):
    """Adjacent pairs of the eq table folded with r (Python integers)."""
    n = len(eq) // 4
    out = np.zeros(2 * n, dtype=np.uint64)
    r0, r1 = int(r[0]), int(r[1])
    for i in range(n):
        a0, a1, b0, b1 = (int(x) for x in eq[4 * i:4 * i + 4])
        d0, d1 = (b0 - a0) % q, (b1 - a1) % q
        out[2 * i] = (a0 + r0 * d0 + 3 * r1 * d1) % q
        out[2 * i + 1] = (a1 + r0 * d1 + r1 * d0) % q
    return out


__all__ = ["make_terms", "ones", "fold_eq", "ext"]
