"""GPU parity of the Basefold path (commit, opening, Merkle, eq tables) against
the CPU oracle, through the C-ABI. Bit-exact."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from .conftest import GL_P, field_elems

pytestmark = pytest.mark.gpu
P = GL_P
u64 = ctypes.c_uint64


@pytest.fixture(scope="module")
def lib():
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    return lib


def _dev_read(lib, ptr, words):
    out = np.empty(words, dtype=np.uint64)
    assert lib.cuda_memcpy_dtoh(out.ctypes.data, ptr, out.nbytes) == 0
    return out


# ---- kernels -------------------------------------------------------------------

@pytest.mark.parametrize("nv", [0, 1, 2, 5, 11, 12, 13, 14, 17, 20])
def test_interpolate_matches_oracle(lib, oracle, nv):
    n = 1 << nv
    evals = field_elems(500 + nv, n)
    d_e = DeviceBuffer.from_numpy(lib, evals)
    d_c, d_b = DeviceBuffer(lib, 8 * n), DeviceBuffer(lib, 8 * n)
    assert lib.basefold_bhc_interpolate_ffi(d_e.ptr, d_c.ptr, d_b.ptr, nv) == 0
    c, b = np.zeros(n, dtype=np.uint64), np.zeros(n, dtype=np.uint64)
    oracle.oracle_bf_bhc_interpolate(evals.ctypes.data, c.ctypes.data, b.ctypes.data, nv)
    assert np.array_equal(d_c.to_numpy(), c)
    assert np.array_equal(d_b.to_numpy(), b)


@pytest.mark.parametrize("nv,lr", [(1, 0), (1, 3), (3, 1), (10, 2), (12, 1), (13, 3), (16, 1), (19, 1)])
def test_encode_matches_oracle(lib, oracle, nv, lr):
    n, m = 1 << nv, 1 << (nv + lr)
    coeffs = field_elems(600 + nv, n)
    d_c = DeviceBuffer.from_numpy(lib, coeffs)
    d_w = DeviceBuffer(lib, 8 * m)
    assert lib.basefold_encode_ffi(d_c.ptr, d_w.ptr, nv, lr) == 0
    cw = np.zeros(m, dtype=np.uint64)
    oracle.oracle_bf_encode(coeffs.ctypes.data, cw.ctypes.data, nv, lr)
    assert np.array_equal(d_w.to_numpy(), cw)
    assert np.array_equal(d_c.to_numpy(), coeffs), "encode must not modify its input"


@pytest.mark.parametrize("log_n", [0, 1, 4, 9, 13])
def test_bit_reverse_in_place(lib, oracle, log_n):
    n = 1 << log_n
    for words, fn, ofn in ((1, lib.basefold_bit_reverse_gl_ffi, oracle.oracle_bf_bit_reverse_gl),
                           (2, lib.basefold_bit_reverse_ext2_ffi, oracle.oracle_bf_bit_reverse_ext2)):
        data = field_elems(700 + log_n, n * words)
        d = DeviceBuffer.from_numpy(lib, data)
        assert fn(d.ptr, log_n) == 0
        exp = data.copy()
        ofn(exp.ctypes.data, log_n)
        assert np.array_equal(d.to_numpy(), exp)


@pytest.mark.parametrize("leaves,ext2", [(1, False), (2, True), (8, False), (64, True), (2048, False), (4096, True), (1 << 15, False)])
def test_merkle_tree_matches_oracle(lib, oracle, leaves, ext2):
    words = leaves * (4 if ext2 else 2)
    cw = field_elems(800 + leaves, words)
    d_cw = DeviceBuffer.from_numpy(lib, cw)
    d_t = DeviceBuffer(lib, 32 * (2 * leaves - 1))
    fn = lib.poseidon2_merkle_tree_ext2_ffi if ext2 else lib.poseidon2_merkle_tree_gl_ffi
    assert fn(d_cw.ptr, d_t.ptr, leaves) == 0
    exp = np.zeros(4 * (2 * leaves - 1), dtype=np.uint64)
    oracle.oracle_bf_merkle_tree(cw.ctypes.data, leaves, 1 if ext2 else 0, exp.ctypes.data)
    assert np.array_equal(d_t.to_numpy(), exp)


def test_leaf_digest_small_fixture(lib, oracle):
    # The codeword of the reference's test_gl_leaf_hash_matches_gpu
    # (goldilocks-cuda-rs/src/cpu_poseidon2.rs:239-256).
    data = np.array([100, 200, 300, 400, 500, 600, 700, 800], dtype=np.uint64)
    d_cw = DeviceBuffer.from_numpy(lib, data)
    d_t = DeviceBuffer(lib, 32 * 7)
    assert lib.poseidon2_merkle_tree_gl_ffi(d_cw.ptr, d_t.ptr, 4) == 0
    tree = d_t.to_numpy()
    oracle.gl_hash_gl_leaf.argtypes = [u64, u64, ctypes.c_void_p]
    for i in range(4):
        out = (u64 * 4)()
        oracle.gl_hash_gl_leaf(int(data[2 * i]), int(data[2 * i + 1]), out)
        assert list(tree[4 * i:4 * i + 4]) == list(out)


def test_permute_and_compress_batches(lib, oracle):
    n = 1000
    states = field_elems(900, 8 * n)
    states[:8] = np.arange(8, dtype=np.uint64)
    d_in = DeviceBuffer.from_numpy(lib, states)
    d_out = DeviceBuffer(lib, states.nbytes)
    assert lib.poseidon2_hash_batch_ffi(d_in.ptr, d_out.ptr, n) == 0
    got = d_out.to_numpy().reshape(n, 8)
    for k in (0, 1, 17, n - 1):
        s = (u64 * 8)(*[int(x) for x in states[8 * k:8 * k + 8]])
        oracle.gl_poseidon2_permute(s)
        assert list(got[k]) == list(s)
    # vector produced by the reference's own poseidon2_permute_8 for input 0..7
    assert int(got[0][0]) == 2477790949385295168
    left, right = states[:4 * n].copy(), states[4 * n:].copy()
    d_l, d_r = DeviceBuffer.from_numpy(lib, left), DeviceBuffer.from_numpy(lib, right)
    d_o = DeviceBuffer(lib, 32 * n)
    assert lib.poseidon2_compress_batch_ffi(d_l.ptr, d_r.ptr, d_o.ptr, n) == 0
    got = d_o.to_numpy().reshape(n, 4)
    oracle.gl_compress.argtypes = [ctypes.c_void_p] * 3
    for k in (0, 5, n - 1):
        o = np.zeros(4, dtype=np.uint64)
        oracle.gl_compress(left[4 * k:].ctypes.data, right[4 * k:].ctypes.data, o.ctypes.data)
        assert np.array_equal(got[k], o)
    assert lib.poseidon2_merkle_layer_ffi(d_in.ptr, d_o.ptr, n) == 0
    got = d_o.to_numpy().reshape(n, 4)
    o = np.zeros(4, dtype=np.uint64)
    oracle.gl_compress(states[8 * 3:].ctypes.data, states[8 * 3 + 4:].ctypes.data, o.ctypes.data)
    assert np.array_equal(got[3], o)


@pytest.mark.parametrize("log_n", [0, 1, 2, 7, 12, 13, 16, 19])
def test_eq_tables_match_oracle(lib, oracle, log_n):
    n = 1 << log_n
    for words, fn, ofn in ((1, lib.eq_dp_all_ffi, oracle.oracle_gl_eq_base), (2, lib.ext2_eq_dp_all_ffi, oracle.oracle_gl_eq_ext2)):
        r = field_elems(1000 + log_n, max(1, log_n) * words)
        d_r = DeviceBuffer.from_numpy(lib, r)
        d_a, d_b = DeviceBuffer(lib, 8 * n * words), DeviceBuffer(lib, 8 * n * words)
        res = ctypes.c_void_p()
        assert fn(d_r.ptr, d_a.ptr, d_b.ptr, log_n, ctypes.byref(res)) == 0
        assert res.value in (d_a.ptr, d_b.ptr)
        got = _dev_read(lib, res.value, n * words)
        exp = np.zeros(n * words, dtype=np.uint64)
        ofn(r.ctypes.data, log_n, exp.ctypes.data)
        assert np.array_equal(got, exp)


# ---- table, commit, opening ------------------------------------------------------

def _table(lib, nv, lr, seed=42):
    h = ctypes.c_void_p()
    assert lib.basefold_table_create(nv, lr, nv, seed, ctypes.byref(h)) == 0
    return h


def test_table_matches_oracle(lib):
    from oracle import pyoracle
    for nv, lr in ((3, 1), (8, 2), (14, 1)):
        h = _table(lib, nv, lr)
        total = lib.basefold_table_entries(h)
        got = np.zeros(2 * total, dtype=np.uint64)
        assert lib.basefold_table_download(h, got.ctypes.data) == 0
        assert np.array_equal(got, pyoracle.bf_table(nv, lr))
        lib.basefold_table_destroy(h)


@pytest.mark.parametrize("nv,lr", [(2, 1), (5, 3), (12, 1), (13, 2), (16, 1)])
def test_commit_matches_oracle(lib, nv, lr):
    from oracle import pyoracle
    evals = field_elems(3, 1 << nv)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    c = ctypes.c_void_p()
    root = np.zeros(4, dtype=np.uint64)
    assert lib.basefold_commit_host(evals.ctypes.data, nv, lr, ctypes.byref(c), root.ctypes.data) == 0
    assert np.array_equal(root, tree[-4:])
    assert np.array_equal(_dev_read(lib, lib.basefold_commitment_codeword(c), len(cw)), cw)
    assert np.array_equal(_dev_read(lib, lib.basefold_commitment_bh_evals(c), len(bh)), bh)
    assert np.array_equal(_dev_read(lib, lib.basefold_commitment_tree(c), len(tree)), tree)
    lib.basefold_commitment_destroy(c)


@pytest.mark.parametrize("nv,lr,nq", [(2, 1, 2), (2, 0, 1), (3, 1, 4), (4, 3, 5), (7, 1, 9), (10, 2, 16), (13, 1, 34),
                                      (16, 1, 100), (18, 1, 100)])
def test_commit_open_matches_oracle(lib, nv, lr, nq):
    # (18, 1, 100): rate 1/2, 100 queries, Poseidon2 trees and transcript; evaluations
    # seed 3, table seed 42, point seed 4 -- the 2^24 configuration at a size the
    # CPU oracle finishes in seconds. Every word of the proof must be equal.
    from oracle import pyoracle
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    exp, exp_state = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)
    h = _table(lib, nv, lr)
    words = lib.basefold_proof_words(nv, lr, nq)
    assert words == len(exp)
    proof = np.zeros(words, dtype=np.uint64)
    root = np.zeros(4, dtype=np.uint64)
    c = ctypes.c_void_p()
    assert lib.basefold_commit_host(evals.ctypes.data, nv, lr, ctypes.byref(c), root.ctypes.data) == 0
    st = np.zeros(8, dtype=np.uint64)
    assert lib.basefold_open_ext2(c, point.ctypes.data, h, b"bench", 5, nq, proof.ctypes.data, st.ctypes.data) == 0
    assert np.array_equal(root, tree[-4:])
    bad = np.nonzero(proof != exp)[0]
    assert len(bad) == 0, "first differing proof word: %d of %d" % (bad[0], words)
    assert np.array_equal(st, exp_state)
    assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) == 0
    # one-call form from host buffers
    proof2 = np.zeros(words, dtype=np.uint64)
    root2 = np.zeros(4, dtype=np.uint64)
    assert lib.basefold_prove_host(evals.ctypes.data, nv, lr, point.ctypes.data, h, b"bench", 5, nq,
                                   root2.ctypes.data, proof2.ctypes.data) == 0
    assert np.array_equal(proof2, exp) and np.array_equal(root2, root)
    lib.basefold_commitment_destroy(c)
    lib.basefold_table_destroy(h)


def test_full_size_commit_and_opening_2_24(lib):
    """The benchmarked configuration at its own size: 2^24 evaluations (seed 3), rate 1/2, 100 queries, point
    seed 4, table seed 42, label "bench". The commitment root must equal the root of one full-size commit by the
    CPU oracle, the folding table must equal the oracle's, and the proof must pass the oracle's restatement of
    the reference verifier (goldilocks-cuda-rs/src/basefold.rs:1759-1925). About a minute of CPU work."""
    from oracle import pyoracle
    nv, lr, nq = 24, 1, 100
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    h = _table(lib, nv, lr)
    words = lib.basefold_proof_words(nv, lr, nq)
    proof = np.zeros(words, dtype=np.uint64)
    root = np.zeros(4, dtype=np.uint64)
    assert lib.basefold_prove_host(evals.ctypes.data, nv, lr, point.ctypes.data, h, b"bench", 5, nq,
                                   root.ctypes.data, proof.ctypes.data) == 0
    table = pyoracle.bf_table(nv, lr)
    got_table = np.zeros(2 * lib.basefold_table_entries(h), dtype=np.uint64)
    assert lib.basefold_table_download(h, got_table.ctypes.data) == 0
    assert np.array_equal(got_table, table)
    del got_table
    lib.basefold_table_destroy(h)
    _, _, tree = pyoracle.bf_commit(evals, nv, lr)
    assert np.array_equal(root, tree[-4:]), "commitment root of the 2^24 polynomial"
    del tree
    assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) == 0
    # a flipped word of the first oracle, of a folded root and of a query value must all be caught
    for pos in (2, 2 + 6 * nv + 1, words - 1 - 4 * (nv + lr)):
        bad = proof.copy()
        bad[pos] ^= np.uint64(1)
        assert pyoracle.bf_verify(root, nv, lr, point, table, nq, bad) != 0, "tampered word %d accepted" % pos


def test_reference_call_sequence_through_dropin_entry_points(lib, oracle):
    # Replays open_ext2's own kernel sequence (goldilocks-cuda-rs/src/basefold.rs:578-863:
    # interp / product / eval / fused round / fold / tree, partial sums added on
    # the host) with this library's drop-in entry points; the oracles, roots and
    # final codeword must equal the CPU oracle's.
    from oracle import pyoracle
    nv, lr, nq = 9, 1, 0
    n, cw_len = 1 << nv, 1 << (nv + lr)
    evals = field_elems(3, n)
    point = field_elems(4, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    exp, _ = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)

    class T(ctypes.Structure):
        _fields_ = [("sponge", u64 * 8), ("in_buf", u64 * 4), ("out_buf", u64 * 4),
                    ("in_count", ctypes.c_int), ("out_count", ctypes.c_int), ("perms", u64)]
    t = T()
    oracle.gl_transcript_squeeze.restype = u64
    oracle.gl_transcript_absorb.argtypes = [ctypes.c_void_p, u64]
    oracle.gl_transcript_new(ctypes.byref(t), b"bench", 5)
    absorb = lambda v: oracle.gl_transcript_absorb(ctypes.byref(t), int(v))
    squeeze = lambda: oracle.gl_transcript_squeeze(ctypes.byref(t))

    def add2(a, b):
        return ((a[0] + b[0]) % P, (a[1] + b[1]) % P)

    def reduce3(bufs, blocks):
        out = []
        for b in bufs:
            part = b.to_numpy()[:2 * blocks].reshape(blocks, 2)
            acc = (0, 0)
            for row in part:
                acc = add2(acc, (int(row[0]), int(row[1])))
            out += [acc[0], acc[1]]
        return out

    for v in tree[-4:]:
        absorb(v)
    for v in point:
        absorb(v)
    d_point = DeviceBuffer.from_numpy(lib, point)
    d_eq_a, d_eq_b = DeviceBuffer(lib, 16 * n), DeviceBuffer(lib, 16 * n)
    res = ctypes.c_void_p()
    assert lib.ext2_eq_dp_all_ffi(d_point.ptr, d_eq_a.ptr, d_eq_b.ptr, nv, ctypes.byref(res)) == 0
    if res.value != d_eq_a.ptr:
        d_eq_a, d_eq_b = d_eq_b, d_eq_a
    d_bh_fp = DeviceBuffer.from_numpy(lib, bh)
    assert lib.basefold_bit_reverse_gl_ffi(d_bh_fp.ptr, nv) == 0
    blocks = 4
    d_dp = DeviceBuffer(lib, 16 * blocks)
    assert lib.basefold_dot_product_mixed_ffi(d_bh_fp.ptr, d_eq_a.ptr, d_dp.ptr, n, blocks) == 0
    part = d_dp.to_numpy().reshape(blocks, 2)
    ev = (sum(int(x) for x in part[:, 0]) % P, sum(int(x) for x in part[:, 1]) % P)
    assert ev == (int(exp[0]), int(exp[1]))
    pc = [DeviceBuffer(lib, 16 * 256) for _ in range(3)]
    pair = n // 2
    assert lib.basefold_sumcheck_interp_gl_ffi(d_bh_fp.ptr, pair) == 0
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_eq_a.ptr, pair) == 0
    assert lib.basefold_sumcheck_product_mixed_ffi(d_eq_a.ptr, d_bh_fp.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pair, blocks) == 0
    oracles = [reduce3(pc, blocks)]
    for v in oracles[-1]:
        absorb(v)
    c0, c1 = squeeze(), squeeze()
    d_bh_a, d_bh_b = DeviceBuffer(lib, 16 * n), DeviceBuffer(lib, 16 * n)
    assert lib.basefold_sumcheck_eval_mixed_ffi(d_bh_fp.ptr, c0, c1, d_bh_a.ptr, pair) == 0
    assert lib.basefold_sumcheck_eval_ext2_ffi(d_eq_a.ptr, c0, c1, d_eq_b.ptr, pair) == 0
    pair //= 2
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_eq_b.ptr, pair) == 0
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_bh_a.ptr, pair) == 0
    assert lib.basefold_sumcheck_product_ext2_ffi(d_eq_b.ptr, d_bh_a.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pair, blocks) == 0
    oracles.append(reduce3(pc, blocks))
    for v in oracles[-1]:
        absorb(v)
    d_table = DeviceBuffer.from_numpy(lib, table)
    d_cw = DeviceBuffer.from_numpy(lib, cw)
    cw_pairs = cw_len // 2
    level_off = 0
    folds = [DeviceBuffer(lib, 16 * cw_pairs)]
    assert lib.basefold_fold_mixed_ffi(d_cw.ptr, d_table.ptr, c0, c1, folds[0].ptr, cw_pairs) == 0
    roots = []

    def tree_root(buf, pairs):
        d_t = DeviceBuffer(lib, 32 * (pairs - 1))
        assert lib.poseidon2_merkle_tree_ext2_ffi(buf.ptr, d_t.ptr, pairs // 2) == 0
        return d_t.to_numpy()[-4:]
    roots.append(tree_root(folds[0], cw_pairs))
    for v in roots[-1]:
        absorb(v)
    level_off += 2 * cw_pairs
    cw_pairs //= 2
    eq_cur, eq_oth, bh_cur, bh_oth = d_eq_b, d_eq_a, d_bh_a, d_bh_b
    for rnd in range(1, nv - 1):
        c0, c1 = squeeze(), squeeze()
        product_pairs = pair // 2
        assert lib.fused_sumcheck_round_ext2_ffi(eq_cur.ptr, bh_cur.ptr, c0, c1, eq_oth.ptr, bh_oth.ptr, pc[0].ptr,
                                                 pc[1].ptr, pc[2].ptr, product_pairs, min(blocks, product_pairs)) == 0
        oracles.append(reduce3(pc, min(blocks, product_pairs)))
        eq_cur, eq_oth, bh_cur, bh_oth = eq_oth, eq_cur, bh_oth, bh_cur
        pair //= 2
        for v in oracles[-1]:
            absorb(v)
        folds.append(DeviceBuffer(lib, 16 * cw_pairs))
        assert lib.basefold_fold_ext2_ffi(folds[-2].ptr, d_table.ptr + 8 * level_off, c0, c1, folds[-1].ptr, cw_pairs) == 0
        roots.append(tree_root(folds[-1], cw_pairs))
        for v in roots[-1]:
            absorb(v)
        level_off += 2 * cw_pairs
        cw_pairs //= 2
    c0, c1 = squeeze(), squeeze()
    d_fin = DeviceBuffer(lib, 16 * cw_pairs)
    assert lib.basefold_fold_ext2_ffi(folds[-1].ptr, d_table.ptr + 8 * level_off, c0, c1, d_fin.ptr, cw_pairs) == 0
    got = np.array([x for o in oracles for x in o] + [int(x) for r in roots for x in r] + [int(x) for x in d_fin.to_numpy()],
                   dtype=np.uint64)
    assert np.array_equal(got, exp[2:2 + len(got)])
