"""This library against the reference's own Goldilocks CUDA wrapper, entry point by entry point.

The reference's goldilocks-cuda-rs/cuda/wrapper.cu is compiled unchanged for
sm_100a (oracle/Makefile, target refcuda) and loaded next to this package's
library. Every scenario below is one Python function of `lib`; it runs once
per library on the same seeded inputs, and the outputs must be equal word for
word after bringing the reference's words into [0, p) (its kernels leave
non-canonical residues, goldilocks-cuda-rs/cuda/wrapper.cu:1604-1648). The
last scenario replays the kernel sequence of open_ext2
(goldilocks-cuda-rs/src/basefold.rs:578-863) on the reference library and
compares it with the CPU oracle's proof, which pins the oracle's Basefold
opening to what the reference's kernels compute.

Sizes stay at or below 2^16 elements and every argument is one the reference
accepts (its kernels check no pointer or size).
"""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import load_gl
from .conftest import field_elems
from .refcuda import GL_P, Buf, canon, ref_gl, sum_rows

pytestmark = pytest.mark.gpu
P = GL_P
u64 = ctypes.c_uint64


@pytest.fixture(scope="module")
def libs():
    ours = load_gl()
    assert ours.goldilocks_cuda_init() == 0 and ours.poseidon2_cuda_init() == 0 and ours.monolith_cuda_init() == 0
    return ours, ref_gl()


def both(libs, scenario, *args):
    """Runs `scenario(lib, *args)` on both libraries; returns two lists of canonical word arrays."""
    out = []
    for lib in libs:
        res = scenario(lib, *args)
        assert lib.cuda_device_synchronize() == 0
        out.append([canon(r, P) for r in res])
    ours, ref = out
    assert len(ours) == len(ref)
    for k, (a, b) in enumerate(zip(ours, ref)):
        assert a.shape == b.shape, "output %d" % k
        bad = np.nonzero(a != b)[0]
        assert len(bad) == 0, "output %d differs from the reference at word %d of %d" % (k, bad[0], len(a))
    return ours


# ---- interpolate / encode / bit reversal ------------------------------------------------

def _interp(lib, nv):
    n = 1 << nv
    d_e = Buf.of(lib, field_elems(500 + nv, n))
    d_c, d_b = Buf(lib, 8 * n), Buf(lib, 8 * n)
    assert lib.basefold_bhc_interpolate_ffi(d_e.ptr, d_c.ptr, d_b.ptr, nv) == 0
    return [d_c.get(count=n), d_b.get(count=n)]


@pytest.mark.parametrize("nv", [1, 2, 5, 11, 13, 16])
def test_interpolate(libs, oracle, nv):
    got = both(libs, _interp, nv)
    n = 1 << nv
    evals = field_elems(500 + nv, n)
    c, b = np.zeros(n, dtype=np.uint64), np.zeros(n, dtype=np.uint64)
    oracle.oracle_bf_bhc_interpolate(evals.ctypes.data, c.ctypes.data, b.ctypes.data, nv)
    assert np.array_equal(got[0], c) and np.array_equal(got[1], b)


def _encode(lib, nv, lr):
    n, m = 1 << nv, 1 << (nv + lr)
    d_c = Buf.of(lib, field_elems(600 + nv, n))
    d_w = Buf(lib, 8 * m)
    assert lib.basefold_encode_ffi(d_c.ptr, d_w.ptr, nv, lr) == 0
    return [d_w.get(count=m)]


@pytest.mark.parametrize("nv,lr", [(1, 0), (1, 3), (3, 1), (10, 2), (13, 3), (15, 1)])
def test_encode(libs, oracle, nv, lr):
    got = both(libs, _encode, nv, lr)
    coeffs = field_elems(600 + nv, 1 << nv)
    cw = np.zeros(1 << (nv + lr), dtype=np.uint64)
    oracle.oracle_bf_encode(coeffs.ctypes.data, cw.ctypes.data, nv, lr)
    assert np.array_equal(got[0], cw)


def _bitrev(lib, log_n):
    n = 1 << log_n
    d1 = Buf.of(lib, field_elems(700 + log_n, n))
    d2 = Buf.of(lib, field_elems(701 + log_n, 2 * n))
    assert lib.basefold_bit_reverse_gl_ffi(d1.ptr, log_n) == 0
    assert lib.basefold_bit_reverse_ext2_ffi(d2.ptr, log_n) == 0
    return [d1.get(count=n), d2.get(count=2 * n)]


@pytest.mark.parametrize("log_n", [1, 4, 9, 13])
def test_bit_reverse(libs, log_n):
    both(libs, _bitrev, log_n)


# ---- codeword folds ----------------------------------------------------------------------

def _folds(lib, pairs, table):
    cw = field_elems(41, 2 * pairs)
    cw2 = field_elems(42, 4 * pairs)
    r = field_elems(43, 2)
    d_t = Buf.of(lib, table[:2 * pairs])
    d_cw, d_cw2 = Buf.of(lib, cw), Buf.of(lib, cw2)
    o1, o2, o3 = Buf(lib, 8 * pairs), Buf(lib, 16 * pairs), Buf(lib, 16 * pairs)
    assert lib.basefold_fold_gl_ffi(d_cw.ptr, d_t.ptr, int(r[0]), o1.ptr, pairs) == 0
    assert lib.basefold_fold_mixed_ffi(d_cw.ptr, d_t.ptr, int(r[0]), int(r[1]), o2.ptr, pairs) == 0
    assert lib.basefold_fold_ext2_ffi(d_cw2.ptr, d_t.ptr, int(r[0]), int(r[1]), o3.ptr, pairs) == 0
    return [o1.get(count=pairs), o2.get(count=2 * pairs), o3.get(count=2 * pairs)]


@pytest.mark.parametrize("pairs", [1, 2, 300, 1 << 13])
def test_codeword_folds(libs, pairs):
    from oracle import pyoracle
    table = pyoracle.bf_table(13, 1)   # level 0 has 2^13 (point, weight) entries
    both(libs, _folds, pairs, table)


# ---- inner sumcheck pieces ---------------------------------------------------------------

def _inner_sumcheck(lib, pairs, blocks):
    eq_b, bh_b = field_elems(51, 2 * pairs), field_elems(52, 2 * pairs)
    eq_e, bh_e = field_elems(53, 4 * pairs), field_elems(54, 4 * pairs)
    r = field_elems(55, 2)
    outs = []
    pc = [Buf(lib, 16 * blocks) for _ in range(3)]

    def partials(words):
        return [sum_rows(p.get(), blocks, words, P) for p in pc]

    # base field: interp, product, eval
    d_eq, d_bh = Buf.of(lib, eq_b), Buf.of(lib, bh_b)
    assert lib.basefold_sumcheck_interp_gl_ffi(d_eq.ptr, pairs) == 0
    assert lib.basefold_sumcheck_interp_gl_ffi(d_bh.ptr, pairs) == 0
    outs += [d_eq.get(count=2 * pairs), d_bh.get(count=2 * pairs)]
    assert lib.basefold_sumcheck_product_gl_ffi(d_eq.ptr, d_bh.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pairs, blocks) == 0
    outs += partials(1)
    d_o = Buf(lib, 8 * pairs)
    assert lib.basefold_sumcheck_eval_gl_ffi(d_bh.ptr, int(r[0]), d_o.ptr, pairs) == 0
    outs.append(d_o.get(count=pairs))
    # mixed: extension eq, base bh
    d_eqe = Buf.of(lib, eq_e)
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_eqe.ptr, pairs) == 0
    outs.append(d_eqe.get(count=4 * pairs))
    assert lib.basefold_sumcheck_product_mixed_ffi(d_eqe.ptr, d_bh.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pairs, blocks) == 0
    outs += partials(2)
    d_o2 = Buf(lib, 16 * pairs)
    assert lib.basefold_sumcheck_eval_mixed_ffi(d_bh.ptr, int(r[0]), int(r[1]), d_o2.ptr, pairs) == 0
    outs.append(d_o2.get(count=2 * pairs))
    # extension field
    d_bhe = Buf.of(lib, bh_e)
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_bhe.ptr, pairs) == 0
    assert lib.basefold_sumcheck_product_ext2_ffi(d_eqe.ptr, d_bhe.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pairs, blocks) == 0
    outs += partials(2)
    assert lib.basefold_sumcheck_eval_ext2_ffi(d_bhe.ptr, int(r[0]), int(r[1]), d_o2.ptr, pairs) == 0
    outs.append(d_o2.get(count=2 * pairs))
    # fused round: inputs of 4 * q extension elements each, interpolated form
    if pairs % 2 == 0:
        q = pairs // 2
        fb = min(blocks, q)
        e_out, b_out = Buf(lib, 32 * q), Buf(lib, 32 * q)
        assert lib.fused_sumcheck_round_ext2_ffi(d_eqe.ptr, d_bhe.ptr, int(r[0]), int(r[1]), e_out.ptr, b_out.ptr,
                                                 pc[0].ptr, pc[1].ptr, pc[2].ptr, q, fb) == 0
        outs += [e_out.get(count=4 * q), b_out.get(count=4 * q)]
        outs += [sum_rows(p.get(), fb, 2, P) for p in pc]
    # dot products
    d_a, d_b = Buf.of(lib, eq_b), Buf.of(lib, bh_b)
    d_p = Buf(lib, 16 * blocks)
    assert lib.basefold_dot_product_gl_ffi(d_a.ptr, d_b.ptr, d_p.ptr, 2 * pairs, blocks) == 0
    outs.append(sum_rows(d_p.get(), blocks, 1, P))
    assert lib.basefold_dot_product_mixed_ffi(d_a.ptr, d_eqe.ptr, d_p.ptr, 2 * pairs, blocks) == 0
    outs.append(sum_rows(d_p.get(), blocks, 2, P))
    return outs


@pytest.mark.parametrize("pairs,blocks", [(1, 1), (2, 1), (6, 2), (1000, 3), (1 << 14, 64)])
def test_inner_sumcheck_kernels(libs, pairs, blocks):
    both(libs, _inner_sumcheck, pairs, blocks)


# ---- hashing -----------------------------------------------------------------------------

def _trees(lib, leaves):
    cw1, cw2 = field_elems(800 + leaves, 2 * leaves), field_elems(801 + leaves, 4 * leaves)
    d1, d2 = Buf.of(lib, cw1), Buf.of(lib, cw2)
    words = 4 * (2 * leaves - 1)
    outs = []
    for fn, d in ((lib.poseidon2_merkle_tree_gl_ffi, d1), (lib.poseidon2_merkle_tree_ext2_ffi, d2),
                  (lib.monolith_merkle_tree_gl_ffi, d1), (lib.monolith_merkle_tree_ext2_ffi, d2)):
        t = Buf(lib, 8 * words)
        assert fn(d.ptr, t.ptr, leaves) == 0
        outs.append(t.get(count=words))
    return outs


@pytest.mark.parametrize("leaves", [1, 2, 8, 2048, 1 << 15])
def test_merkle_trees(libs, oracle, leaves):
    from oracle import pyoracle
    got = both(libs, _trees, leaves)
    cw1, cw2 = field_elems(800 + leaves, 2 * leaves), field_elems(801 + leaves, 4 * leaves)
    exp = np.zeros(4 * (2 * leaves - 1), dtype=np.uint64)
    for k, (cw, ext2, mono) in enumerate(((cw1, 0, 0), (cw2, 1, 0), (cw1, 0, 1), (cw2, 1, 1))):
        with pyoracle.merkle_hash(mono):
            oracle.oracle_bf_merkle_tree(cw.ctypes.data, leaves, ext2, exp.ctypes.data)
        assert np.array_equal(got[k], exp), "tree %d against the CPU oracle" % k


def _hash_batches(lib, n):
    states = field_elems(900, 8 * n)
    states[:8] = np.arange(8, dtype=np.uint64)
    d_in, d_out = Buf.of(lib, states), Buf(lib, 64 * n)
    assert lib.poseidon2_hash_batch_ffi(d_in.ptr, d_out.ptr, n) == 0
    outs = [d_out.get(count=8 * n)]
    d_l, d_r = Buf.of(lib, states[:4 * n]), Buf.of(lib, states[4 * n:])
    d_o = Buf(lib, 32 * n)
    assert lib.poseidon2_compress_batch_ffi(d_l.ptr, d_r.ptr, d_o.ptr, n) == 0
    outs.append(d_o.get(count=4 * n))
    assert lib.poseidon2_merkle_layer_ffi(d_in.ptr, d_o.ptr, n) == 0
    outs.append(d_o.get(count=4 * n))
    inp = (u64 * 12)(*range(12))
    out = (u64 * 12)()
    assert lib.monolith_permute_test_ffi(inp, out) == 0
    outs.append(np.array(list(out), dtype=np.uint64))
    return outs


def test_hash_batches(libs):
    both(libs, _hash_batches, 1000)


# ---- linear sumcheck drop-ins -------------------------------------------------------------

def _sumcheck_rounds(lib, nv, d, ext2):
    w = 2 if ext2 else 1
    n = 1 << nv
    d_a = Buf.of(lib, field_elems(2000 + nv * 10 + d, n * d * w))
    d_b = Buf(lib, 8 * n * d * w)
    outs = []
    size = n
    for rnd in range(nv):
        half = size // 2
        nb = min((half + 255) // 256, 256)
        d_part = Buf(lib, nb * (d + 1) * 8 * w)
        r = field_elems(3000 + rnd, 2)
        if ext2:
            assert lib.sumcheck_round_message_ext2_ffi(d_a.ptr, d_part.ptr, d, n, half, nb) == 0
            outs.append(sum_rows(d_part.get(), nb, 2 * (d + 1), P))
            assert lib.sumcheck_fold_ext2_ffi(d_a.ptr, d_b.ptr, int(r[0]), int(r[1]), d, n, half) == 0
        else:
            assert lib.sumcheck_round_message_ffi(d_a.ptr, d_part.ptr, d, n, half, nb) == 0
            outs.append(sum_rows(d_part.get(), nb, d + 1, P))
            assert lib.sumcheck_fold_ffi(d_a.ptr, d_b.ptr, int(r[0]), d, n, half) == 0
        full = d_b.get(count=n * d * w).reshape(d, n * w)
        outs.append(np.ascontiguousarray(full[:, :half * w]).reshape(-1))
        d_a, d_b = d_b, d_a
        size = half
    return outs


@pytest.mark.parametrize("nv,d,ext2", [(1, 1, False), (4, 2, False), (10, 4, False), (13, 8, False), (16, 2, False),
                                       (1, 1, True), (5, 3, True), (12, 5, True), (14, 8, True), (15, 2, True)])
def test_sumcheck_round_and_fold(libs, nv, d, ext2):
    both(libs, _sumcheck_rounds, nv, d, ext2)


# ---- eq tables, partial evaluation --------------------------------------------------------

def _eq_tables(lib, log_n):
    n = 1 << log_n
    outs = []
    for w, fn in ((1, lib.eq_dp_all_ffi), (2, lib.ext2_eq_dp_all_ffi)):
        d_r = Buf.of(lib, field_elems(1000 + log_n, log_n * w))
        d_a, d_b = Buf(lib, 8 * n * w), Buf(lib, 8 * n * w)
        res = ctypes.c_void_p()
        assert fn(d_r.ptr, d_a.ptr, d_b.ptr, log_n, ctypes.byref(res)) == 0
        assert res.value in (d_a.ptr, d_b.ptr)
        outs.append((d_a if res.value == d_a.ptr else d_b).get(count=n * w))
    return outs


@pytest.mark.parametrize("log_n", [1, 2, 7, 12, 16])
def test_eq_tables(libs, log_n):
    both(libs, _eq_tables, log_n)


def _partial_eval(lib, log_n, m):
    n = 1 << log_n
    data = field_elems(600 + log_n, n)
    d_r = Buf.of(lib, field_elems(601 + m, 2 * m))
    d_data = Buf.of(lib, data)
    assert lib.partial_eval_gl_ffi(d_data.ptr, d_r.ptr, log_n, m) == 0
    outs = [d_data.get(count=n >> m)]
    d_in, d_out = Buf.of(lib, data), Buf(lib, 16 * max(n // 2, 1))
    assert lib.partial_eval_ext2_from_gl_ffi(d_in.ptr, d_out.ptr, d_r.ptr, log_n, m) == 0
    outs.append(d_out.get(count=2 * (n >> m)))
    return outs


@pytest.mark.parametrize("log_n,m", [(1, 1), (6, 3), (10, 4), (13, 9), (16, 16)])
def test_partial_eval(libs, log_n, m):
    both(libs, _partial_eval, log_n, m)


def _fused_permute(lib, n, m, half, lo, hi, eq):
    out_size = 1 << (n - m)
    d_e, d_q = Buf.of(lib, field_elems(900 + n, 1 << n)), Buf.of(lib, eq)
    d_lo, d_hi = Buf.of(lib, lo), Buf.of(lib, hi)
    d_o = Buf(lib, 16 * out_size)
    # dynamic shared memory the reference's kernel needs: both index tables, then two words per warp
    # (cuda/fused_permute_peval.cuh:40-52); this library sizes its own and ignores the argument
    smem = ((4 * (len(lo) + len(hi)) + 7) & ~7) + 16 * 32
    assert lib.fused_permute_partial_eval_ffi(d_e.ptr, d_o.ptr, d_q.ptr, d_lo.ptr, d_hi.ptr, n, m, half, out_size, smem) == 0
    return [d_o.get(count=2 * out_size)]


@pytest.mark.parametrize("n,m,half", [(4, 2, 2), (10, 4, 5), (13, 6, 6), (16, 9, 8)])
def test_fused_permute_partial_eval(libs, oracle, n, m, half):
    from .test_agl_gpu import _split_luts
    order = list(np.random.default_rng(n).permutation(n))
    lo, hi = _split_luts(n, order, half)
    r = field_elems(901 + n, 2 * m)
    eq = np.zeros(2 << m, dtype=np.uint64)
    oracle.oracle_gl_eq_ext2(r.ctypes.data, m, eq.ctypes.data)
    both(libs, _fused_permute, n, m, half, lo, hi, eq)


# ---- device challenger --------------------------------------------------------------------

def _challenger(lib, n):
    states = ctypes.c_void_p()
    assert lib.challenger_alloc_states(ctypes.byref(states), n) == 0
    assert lib.challenger_init_states(states, n) == 0
    script = [("obs", 1), ("obs", 5), ("smp", 1), ("smp", 2), ("obs2", 2), ("smp", 5), ("obs", 3), ("smp", 7),
              ("obs", 4), ("smp", 1)]
    outs = []
    for step, (kind, count) in enumerate(script):
        if kind.startswith("obs"):
            d_v = Buf.of(lib, field_elems(700 + step, n * count))
            if kind == "obs2":
                assert lib.challenger_observe_ext2_ffi(states, d_v.ptr, n) == 0
            elif count == 1:
                assert lib.challenger_observe_ffi(states, d_v.ptr, n) == 0
            else:
                assert lib.challenger_observe_slice_ffi(states, d_v.ptr, count, n) == 0
            assert lib.cuda_device_synchronize() == 0
        else:
            d_o = Buf(lib, 8 * n * count)
            fn = {1: lib.challenger_sample_ffi, 2: lib.challenger_sample_ext2_ffi, 5: lib.challenger_sample_ext5_ffi}.get(count)
            if fn is not None:
                assert fn(states, d_o.ptr, n) == 0
            else:
                assert lib.challenger_sample_array_ffi(states, d_o.ptr, count, n) == 0
            outs.append(d_o.get(count=n * count))
    assert lib.cuda_device_synchronize() == 0
    lib.cuda_free(states)
    return outs


def test_device_challenger(libs):
    assert libs[0].challenger_state_size() == libs[1].challenger_state_size()
    both(libs, _challenger, 300)


# ---- the opening's kernel sequence on the reference library, against the CPU oracle ----------

def _open_sequence(lib, oracle, nv, lr):
    """open_ext2's device calls in order (goldilocks-cuda-rs/src/basefold.rs:578-863), partial sums added on the
    host, challenges from the CPU transcript; returns eval, oracles, folded roots and the final codeword."""
    from oracle import pyoracle
    n, cw_len = 1 << nv, 1 << (nv + lr)
    evals = field_elems(3, n)
    point = field_elems(4, 2 * nv)
    table = pyoracle.bf_table(nv, lr)

    class T(ctypes.Structure):
        _fields_ = [("sponge", u64 * 8), ("in_buf", u64 * 4), ("out_buf", u64 * 4),
                    ("in_count", ctypes.c_int), ("out_count", ctypes.c_int), ("perms", u64)]
    t = T()
    oracle.gl_transcript_squeeze.restype = u64
    oracle.gl_transcript_absorb.argtypes = [ctypes.c_void_p, u64]
    oracle.gl_transcript_new(ctypes.byref(t), b"bench", 5)
    absorb = lambda v: oracle.gl_transcript_absorb(ctypes.byref(t), int(v))
    squeeze = lambda: oracle.gl_transcript_squeeze(ctypes.byref(t))

    # commit: interpolate, encode, tree (basefold.rs:382-414)
    d_ev = Buf.of(lib, evals)
    d_co, d_bh = Buf(lib, 8 * n), Buf(lib, 8 * n)
    assert lib.basefold_bhc_interpolate_ffi(d_ev.ptr, d_co.ptr, d_bh.ptr, nv) == 0
    d_cw = Buf(lib, 8 * cw_len)
    assert lib.basefold_encode_ffi(d_co.ptr, d_cw.ptr, nv, lr) == 0
    d_tree = Buf(lib, 32 * (cw_len - 1))
    assert lib.poseidon2_merkle_tree_gl_ffi(d_cw.ptr, d_tree.ptr, cw_len // 2) == 0
    root = canon(d_tree.get()[4 * (cw_len - 2):4 * (cw_len - 1)], P)

    for v in root:
        absorb(v)
    for v in point:
        absorb(v)
    d_point = Buf.of(lib, point)
    d_eq_a, d_eq_b = Buf(lib, 16 * n), Buf(lib, 16 * n)
    res = ctypes.c_void_p()
    assert lib.ext2_eq_dp_all_ffi(d_point.ptr, d_eq_a.ptr, d_eq_b.ptr, nv, ctypes.byref(res)) == 0
    if res.value != d_eq_a.ptr:
        d_eq_a, d_eq_b = d_eq_b, d_eq_a
    assert lib.basefold_bit_reverse_gl_ffi(d_bh.ptr, nv) == 0
    blocks = 4
    d_dp = Buf(lib, 16 * blocks)
    assert lib.basefold_dot_product_mixed_ffi(d_bh.ptr, d_eq_a.ptr, d_dp.ptr, n, blocks) == 0
    out = [int(x) for x in sum_rows(d_dp.get(), blocks, 2, P)]
    pc = [Buf(lib, 16 * 256) for _ in range(3)]

    def reduce3(nb):
        vals = []
        for p in pc:
            vals += [int(x) for x in sum_rows(p.get(), nb, 2, P)]
        return vals

    pair = n // 2
    assert lib.basefold_sumcheck_interp_gl_ffi(d_bh.ptr, pair) == 0
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_eq_a.ptr, pair) == 0
    assert lib.basefold_sumcheck_product_mixed_ffi(d_eq_a.ptr, d_bh.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pair, blocks) == 0
    oracles = [reduce3(blocks)]
    for v in oracles[-1]:
        absorb(v)
    c0, c1 = squeeze(), squeeze()
    d_bh_a, d_bh_b = Buf(lib, 16 * n), Buf(lib, 16 * n)
    assert lib.basefold_sumcheck_eval_mixed_ffi(d_bh.ptr, c0, c1, d_bh_a.ptr, pair) == 0
    assert lib.basefold_sumcheck_eval_ext2_ffi(d_eq_a.ptr, c0, c1, d_eq_b.ptr, pair) == 0
    pair //= 2
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_eq_b.ptr, pair) == 0
    assert lib.basefold_sumcheck_interp_ext2_ffi(d_bh_a.ptr, pair) == 0
    assert lib.basefold_sumcheck_product_ext2_ffi(d_eq_b.ptr, d_bh_a.ptr, pc[0].ptr, pc[1].ptr, pc[2].ptr, pair, blocks) == 0
    oracles.append(reduce3(blocks))
    for v in oracles[-1]:
        absorb(v)
    d_table = Buf.of(lib, table)
    cw_pairs = cw_len // 2
    level_off = 0
    folds = [Buf(lib, 16 * cw_pairs)]
    assert lib.basefold_fold_mixed_ffi(d_cw.ptr, d_table.ptr, c0, c1, folds[0].ptr, cw_pairs) == 0
    roots = []

    def tree_root(buf, pairs):
        d_t = Buf(lib, 32 * (pairs - 1))
        assert lib.poseidon2_merkle_tree_ext2_ffi(buf.ptr, d_t.ptr, pairs // 2) == 0
        return canon(d_t.get()[4 * (pairs - 2):4 * (pairs - 1)], P)
    roots.append(tree_root(folds[0], cw_pairs))
    for v in roots[-1]:
        absorb(v)
    level_off += 2 * cw_pairs
    cw_pairs //= 2
    eq_cur, eq_oth, bh_cur, bh_oth = d_eq_b, d_eq_a, d_bh_a, d_bh_b
    for rnd in range(1, nv - 1):
        c0, c1 = squeeze(), squeeze()
        q = pair // 2
        nb = min(blocks, q)
        assert lib.fused_sumcheck_round_ext2_ffi(eq_cur.ptr, bh_cur.ptr, c0, c1, eq_oth.ptr, bh_oth.ptr, pc[0].ptr,
                                                 pc[1].ptr, pc[2].ptr, q, nb) == 0
        oracles.append(reduce3(nb))
        eq_cur, eq_oth, bh_cur, bh_oth = eq_oth, eq_cur, bh_oth, bh_cur
        pair //= 2
        for v in oracles[-1]:
            absorb(v)
        folds.append(Buf(lib, 16 * cw_pairs))
        assert lib.basefold_fold_ext2_ffi(folds[-2].ptr, d_table.ptr + 8 * level_off, c0, c1, folds[-1].ptr, cw_pairs) == 0
        roots.append(tree_root(folds[-1], cw_pairs))
        for v in roots[-1]:
            absorb(v)
        level_off += 2 * cw_pairs
        cw_pairs //= 2
    c0, c1 = squeeze(), squeeze()
    d_fin = Buf(lib, 16 * cw_pairs)
    assert lib.basefold_fold_ext2_ffi(folds[-1].ptr, d_table.ptr + 8 * level_off, c0, c1, d_fin.ptr, cw_pairs) == 0
    fin = canon(d_fin.get(count=2 * cw_pairs), P)
    words = out + [x for o in oracles for x in o] + [int(x) for r in roots for x in r] + [int(x) for x in fin]
    return root, np.array(words, dtype=np.uint64)


@pytest.mark.parametrize("nv,lr", [(4, 1), (9, 1), (12, 2), (14, 1)])
def test_opening_sequence_on_the_reference_library_matches_the_cpu_oracle(libs, oracle, nv, lr):
    from oracle import pyoracle
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    exp, _ = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, 0)
    for lib in libs:
        root, got = _open_sequence(lib, oracle, nv, lr)
        assert np.array_equal(root, tree[-4:]), "commitment root"
        assert np.array_equal(got, exp[:len(got)]), "eval, oracles, folded roots, final codeword"
