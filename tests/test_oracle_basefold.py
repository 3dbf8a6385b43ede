"""CPU tests of the Basefold oracle: table, commit structure, prover -> verifier
round trip, tamper rejection, evaluation claim against direct MLE evaluation."""
import ctypes

import numpy as np
import pytest

from .conftest import GL_P, field_elems

P = GL_P


def test_table_first_entries_follow_xorshift():
    from oracle import pyoracle
    nv, lr = 3, 1
    tab = pyoracle.bf_table(nv, lr, seed=42)
    s = 42
    M = (1 << 64) - 1

    def nxt(s):
        s ^= (s << 13) & M
        s ^= s >> 7
        s ^= (s << 17) & M
        return s
    for k in range(8 + 4 + 2):
        s = nxt(s); x0 = s % P
        s = nxt(s); x1 = s % P
        while x1 == x0:
            s = nxt(s); x1 = s % P
        assert int(tab[2 * k]) == x0
        assert int(tab[2 * k + 1]) * ((x1 - x0) % P) % P == 1
    assert len(tab) == 2 * (8 + 4 + 2)


def _mle_eval_ext2(evals, point):
    # direct evaluation with Python integers; point = list of (c0, c1)
    def mul(a, b):
        return ((a[0] * b[0] + 7 * a[1] * b[1]) % P, (a[0] * b[1] + a[1] * b[0]) % P)
    cur = [(int(v), 0) for v in evals]
    for (r0, r1) in point:
        nxt = []
        for j in range(len(cur) // 2):
            a, b = cur[2 * j], cur[2 * j + 1]
            d = ((b[0] - a[0]) % P, (b[1] - a[1]) % P)
            m = mul((r0, r1), d)
            nxt.append(((a[0] + m[0]) % P, (a[1] + m[1]) % P))
        cur = nxt
    return cur[0]


def test_codeword_is_evaluations_on_pm1_cube_repeated():
    # interpolate + butterflies = the multilinear extension evaluated on {1,-1}^nv;
    # the repetition makes the codeword 2^lr equal blocks after the bit reversal.
    from oracle import pyoracle
    nv, lr = 4, 2
    evals = field_elems(11, 1 << nv)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    n = 1 << nv
    for blk in range(1, 1 << lr):
        assert np.array_equal(cw[:n], cw[blk * n:(blk + 1) * n])

    def rev(x, bits):
        return int(format(x, "0%db" % bits)[::-1], 2)
    for j in range(n):
        pt = [((1, 0) if ((j >> i) & 1) == 0 else (P - 1, 0)) for i in range(nv)]
        assert int(cw[rev(j, nv)]) == _mle_eval_ext2(evals, pt)[0]
    assert np.array_equal(bh[[rev(i, nv) for i in range(n)]], evals)


@pytest.mark.parametrize("nv,lr,nq", [(2, 1, 3), (3, 1, 5), (4, 3, 7), (6, 1, 10), (8, 2, 12)])
def test_open_verifies_and_claims_mle_value(nv, lr, nq):
    from oracle import pyoracle
    evals = field_elems(20 + nv, 1 << nv)
    point = field_elems(30 + nv, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    proof, st = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)
    root = tree[-4:]
    assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) == 0
    ev = _mle_eval_ext2(evals, [(int(point[2 * i]), int(point[2 * i + 1])) for i in range(nv)])
    assert (int(proof[0]), int(proof[1])) == ev
    # Any flipped word must be rejected, except final-codeword entries that no
    # query lands on: the reference's verifier checks that vector only at the
    # queried positions (basefold.rs:1894-1905).
    rng = np.random.default_rng(nv)
    fc_lo = 2 + nv * 6 + (nv - 1) * 4
    fc_hi = fc_lo + (2 << lr)
    candidates = [i for i in range(len(proof)) if not (fc_lo <= i < fc_hi)]
    for pos in rng.choice(candidates, size=min(40, len(candidates)), replace=False):
        bad = proof.copy()
        bad[pos] ^= np.uint64(1)
        assert pyoracle.bf_verify(root, nv, lr, point, table, nq, bad) != 0, "flip at %d accepted" % pos


@pytest.mark.parametrize("hash_id", [0, 1])
def test_host_hashed_tree_top_matches_oracle_tree(hostcheck, hash_id):
    """The provers stop a round's tree on the device at a layer of eight digests and hash the levels above on the
    host (matrix_b200/csrc/host/host_tree_top.hpp). Those host levels must be the oracle tree's own top, with both
    Merkle hashes and for layers of 8, 4, 2 and 1 digests."""
    from oracle import pyoracle
    lib = pyoracle.load()
    u64 = ctypes.c_uint64
    with pyoracle.merkle_hash(hash_id):
        for leaves, ext2 in ((32, 0), (16, 1), (8, 1), (4, 0), (2, 1), (1, 0)):
            cw = field_elems(700 + leaves, leaves * (4 if ext2 else 2))
            tree = np.zeros(4 * (2 * leaves - 1), dtype=np.uint64)
            lib.oracle_bf_merkle_tree(cw.ctypes.data, leaves, ext2, tree.ctypes.data)
            count = min(leaves, 8)
            start = 4 * (2 * leaves - 2 * count)          # the layer of `count` digests
            nodes = np.ascontiguousarray(tree[start:start + 4 * count])
            upper = np.zeros(4 * max(count - 1, 1), dtype=np.uint64)
            root = np.zeros(4, dtype=np.uint64)
            hostcheck.hc_tree_top(hash_id, nodes.ctypes.data_as(ctypes.POINTER(u64)), ctypes.c_size_t(count),
                                  upper.ctypes.data_as(ctypes.POINTER(u64)), root.ctypes.data_as(ctypes.POINTER(u64)))
            assert np.array_equal(root, tree[-4:])
            if count > 1:
                assert np.array_equal(upper[:4 * (count - 1)], tree[start + 4 * count:])


@pytest.mark.parametrize("nv,lr,nq,hash_id", [(2, 1, 3, 0), (2, 0, 0, 0), (5, 1, 0, 1), (2, 2, 1, 0), (3, 0, 4, 0), (4, 3, 7, 1), (6, 1, 10, 0),
                                                    (8, 2, 12, 1), (11, 1, 30, 0)])
def test_library_verifier_with_host_table_agrees_with_oracle_verifier(nv, lr, nq, hash_id):
    """basefold_verify_with_table_host (the library's verifier with the folding table in host memory: no device call,
    so it runs here) on proofs written by the oracle prover: it accepts them, and on every flipped proof word it
    stops at the same check as the oracle's restatement of the reference verifier
    (goldilocks-cuda-rs/src/basefold.rs:1759-1925)."""
    from matrix_b200.ffi import load_gl
    from oracle import pyoracle
    lib = load_gl()
    evals = field_elems(40 + nv, 1 << nv)
    point = field_elems(50 + nv, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    with pyoracle.merkle_hash(hash_id):
        cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
        proof, _ = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)
    root = np.ascontiguousarray(tree[-4:])

    def ours(pr, rt=root, pt=point, label=b"bench", h=hash_id):
        res = ctypes.c_int(777)
        rc = lib.basefold_verify_with_table_host(rt.ctypes.data, nv, lr, pt.ctypes.data, table.ctypes.data, label, len(label), nq, h,
                                                 pr.ctypes.data, ctypes.byref(res))
        assert rc == 0
        return res.value

    def theirs(pr, rt=root, pt=point, label=b"bench"):
        with pyoracle.merkle_hash(hash_id):
            return pyoracle.bf_verify(rt, nv, lr, pt, table, nq, pr, label=label)

    assert theirs(proof) == 0 and ours(proof) == 0
    if nq:
        assert ours(proof, h=1 - hash_id) == -101        # the other hash: the first commitment path fails
    words = len(proof)
    positions = range(words) if words <= 600 else sorted(set(int(x) for x in np.random.default_rng(nv).integers(0, words, 300)))
    for pos in positions:
        bad = proof.copy()
        bad[pos] ^= np.uint64(1)
        assert ours(bad) == theirs(bad), "word %d flipped" % pos
    bad_root = root.copy()
    bad_root[0] ^= np.uint64(1)
    assert ours(proof, rt=bad_root) == theirs(proof, rt=bad_root) != 0
    bad_point = point.copy()
    bad_point[1] ^= np.uint64(1)
    assert ours(proof, pt=bad_point) == theirs(proof, pt=bad_point) != 0
    assert ours(proof, label=b"other") == theirs(proof, label=b"other") != 0
    res = ctypes.c_int(0)
    assert lib.basefold_verify_with_table_host(root.ctypes.data, 0, lr, point.ctypes.data, table.ctypes.data, b"bench", 5, nq, 0,
                                               proof.ctypes.data, ctypes.byref(res)) != 0
