"""This library against the reference's own almost-Goldilocks CUDA wrapper, entry point by entry point.

almost-goldilocks-cuda-rs/cuda/wrapper.cu is compiled unchanged for sm_100a
(oracle/Makefile, target refcuda). Every scenario is one Python function of
`lib`, run once per library on the same seeded inputs; the outputs must be
equal word for word once the reference's words are brought into [0, q). Covered:
linear sumcheck, eq tables, partial evaluation, the batched same-point family,
the K8 product sumcheck and its table helpers, the packed link sumcheck, the
sparse boolean check, the module commitment and the dense Ajtai commit.

Every argument is one the reference accepts: its entry points check nothing, so
scratch buffers are always passed at the size its kernels write, no pointer is
null unless its kernel tests for that, and no size is zero.
"""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import load_agl
from matrix_b200.inputs import field_elems, splitmix64
from .bool_cases import make_terms
from .link_cases import ext, random_bits, sparse_ext, support_lists
from .refcuda import AGL_Q, Buf, canon, ref_agl, sum_rows

pytestmark = pytest.mark.gpu
Q = AGL_Q


@pytest.fixture(scope="module")
def libs():
    ours = load_agl()
    assert ours.almost_goldilocks_cuda_init() == 0
    return ours, ref_agl()


def both(libs, scenario, *args, raw=()):
    """Runs `scenario(lib, *args)` on both libraries and compares. Outputs whose position is in `raw` are not
    field words (flags, indices, offsets) and are compared as they are."""
    out = []
    for lib in libs:
        res = scenario(lib, *args)
        assert lib.cuda_device_synchronize() == 0
        out.append([np.asarray(r) if k in raw else canon(r, Q) for k, r in enumerate(res)])
    ours, ref = out
    assert len(ours) == len(ref)
    for k, (a, b) in enumerate(zip(ours, ref)):
        assert a.shape == b.shape, "output %d" % k
        bad = np.nonzero(a != b)[0]
        assert len(bad) == 0, "output %d differs from the reference at word %d of %d" % (k, bad[0], len(a))
    return ours


def _ptrs(bufs):
    return (ctypes.c_void_p * len(bufs))(*[b.ptr for b in bufs])


# ---- linear sumcheck, eq tables, partial evaluation -----------------------------------------

def _sumcheck_rounds(lib, nv, d, ext2):
    w = 2 if ext2 else 1
    n = 1 << nv
    d_a = Buf.of(lib, field_elems(2100 + nv * 10 + d, n * d * w, Q))
    d_b = Buf(lib, 8 * n * d * w)
    outs = []
    size = n
    for rnd in range(nv):
        half = size // 2
        nb = min((half + 255) // 256, 256)
        d_part = Buf(lib, nb * (d + 1) * 8 * w)
        r = field_elems(3100 + rnd, 2, Q)
        if ext2:
            assert lib.aext2_sumcheck_round_message_ffi(d_a.ptr, d_part.ptr, d, n, half, nb) == 0
            outs.append(sum_rows(d_part.get(), nb, 2 * (d + 1), Q))
            assert lib.aext2_sumcheck_fold_ffi(d_a.ptr, d_b.ptr, int(r[0]), int(r[1]), d, n, half) == 0
        else:
            assert lib.agl_sumcheck_round_message_ffi(d_a.ptr, d_part.ptr, d, n, half, nb) == 0
            outs.append(sum_rows(d_part.get(), nb, d + 1, Q))
            assert lib.agl_sumcheck_fold_ffi(d_a.ptr, d_b.ptr, int(r[0]), d, n, half) == 0
        full = d_b.get(count=n * d * w).reshape(d, n * w)
        outs.append(np.ascontiguousarray(full[:, :half * w]).reshape(-1))
        d_a, d_b = d_b, d_a
        size = half
    return outs


@pytest.mark.parametrize("nv,d,ext2", [(1, 1, False), (6, 2, False), (12, 4, False), (15, 3, False),
                                       (1, 2, True), (7, 3, True), (13, 6, True), (15, 2, True)])
def test_sumcheck_round_and_fold(libs, nv, d, ext2):
    both(libs, _sumcheck_rounds, nv, d, ext2)


def _eq_and_peval(lib, log_n, m):
    n = 1 << log_n
    outs = []
    for w, fn in ((1, lib.agl_eq_dp_all_ffi), (2, lib.aext2_eq_dp_all_ffi)):
        d_r = Buf.of(lib, field_elems(1100 + log_n, log_n * w, Q))
        d_a, d_b = Buf(lib, 8 * n * w), Buf(lib, 8 * n * w)
        res = ctypes.c_void_p()
        assert fn(d_r.ptr, d_a.ptr, d_b.ptr, log_n, ctypes.byref(res)) == 0
        assert res.value in (d_a.ptr, d_b.ptr)
        outs.append((d_a if res.value == d_a.ptr else d_b).get(count=n * w))
    data = field_elems(610 + log_n, n, Q)
    d_r = Buf.of(lib, field_elems(611 + m, 2 * m, Q))
    d_data = Buf.of(lib, data)
    assert lib.agl_partial_eval_ffi(d_data.ptr, d_r.ptr, log_n, m) == 0
    outs.append(d_data.get(count=n >> m))
    d_in, d_out = Buf.of(lib, data), Buf(lib, 16 * max(n // 2, 1))
    assert lib.agl_partial_eval_ext2_from_base_ffi(d_in.ptr, d_out.ptr, d_r.ptr, log_n, m) == 0
    outs.append(d_out.get(count=2 * (n >> m)))
    return outs


@pytest.mark.parametrize("log_n,m", [(1, 1), (6, 3), (12, 5), (16, 9)])
def test_eq_tables_and_partial_eval(libs, log_n, m):
    both(libs, _eq_and_peval, log_n, m)


# ---- batched same-point family -----------------------------------------------------------------

def _packed(seed, leaves, n):
    words = (n + 63) // 64
    return np.ascontiguousarray(splitmix64(seed, leaves * words)), words


def _batched_interleaved(lib, log_n, leaves, blocks):
    n, half = 1 << log_n, 1 << (log_n - 1)
    polys = field_elems(10 + log_n, leaves * 4 * n, Q)
    d_polys = Buf.of(lib, polys)
    d_part = Buf(lib, 8 * blocks * leaves * 6)
    outs = []

    def msg():
        p = d_part.get(count=blocks * leaves * 6).reshape(blocks, leaves * 6)
        return np.array([sum(int(x) for x in p[:, k]) % Q for k in range(leaves * 6)], dtype=np.uint64)

    def live(buf):
        full = buf.get(count=leaves * 4 * n).reshape(leaves * 2, 2 * n)
        return np.ascontiguousarray(full[:, :2 * half]).reshape(-1)

    assert lib.aext2_sumcheck_batched_round_message_ffi(d_polys.ptr, d_part.ptr, n, half, leaves, blocks) == 0
    outs.append(msg())
    r = field_elems(77, 2, Q)
    d_out = Buf(lib, polys.nbytes)
    assert lib.aext2_sumcheck_batched_fold_ffi(d_polys.ptr, d_out.ptr, int(r[0]), int(r[1]), n, half, leaves) == 0
    outs.append(live(d_out))
    packed, words = _packed(20 + log_n, leaves, n)
    d_packed = Buf.of(lib, packed)
    d_polys0 = Buf.of(lib, polys)
    assert lib.aext2_sumcheck_batched_round0_binary_msg_ffi(d_polys0.ptr, d_packed.ptr, d_part.ptr, n, half, leaves, blocks, words) == 0
    outs.append(msg())
    d_out2 = Buf(lib, polys.nbytes)
    assert lib.aext2_sumcheck_batched_round0_binary_fold_ffi(d_polys0.ptr, d_packed.ptr, d_out2.ptr, int(r[0]), int(r[1]), n, half,
                                                             leaves, words) == 0
    outs.append(live(d_out2))
    assert lib.aext2_batched_lift_binary_ffi(d_packed.ptr, d_polys.ptr, n, leaves, words) == 0
    outs.append(d_polys.get(count=leaves * 4 * n))
    return outs


@pytest.mark.parametrize("log_n,leaves,blocks", [(1, 1, 1), (4, 3, 2), (9, 5, 7), (13, 4, 16)])
def test_batched_interleaved(libs, log_n, leaves, blocks):
    both(libs, _batched_interleaved, log_n, leaves, blocks)


def _lifts_and_fu(lib):
    n, leaves = 300, 6
    packed, words = _packed(5, leaves, n)
    neg, _ = _packed(6, leaves, n)
    neg &= ~packed
    d_p, d_n = Buf.of(lib, packed), Buf.of(lib, neg)
    outs = []
    d_f = Buf(lib, 16 * n * leaves)
    assert lib.aext2_lift_binary_contig_ffi(d_p.ptr, d_f.ptr, n, leaves, words) == 0
    outs.append(d_f.get(count=2 * n * leaves))
    d_polys = Buf(lib, 32 * n * leaves)
    assert lib.aext2_batched_lift_ternary_single_ffi(d_p.ptr, d_n.ptr, d_polys.ptr, n, leaves, words) == 0
    full = d_polys.get(count=4 * n * leaves).reshape(leaves, 2, 2 * n)
    outs.append(np.ascontiguousarray(full[:, 1]).reshape(-1))       # the f slots; the eq slots are not written
    d_eq = Buf.of(lib, field_elems(9, 2 * n, Q))
    blocks = 3
    d_part = Buf(lib, 8 * blocks * leaves * 2)
    assert lib.aext2_selective_add_batched_planes_ffi(d_eq.ptr, d_p.ptr, d_part.ptr, n, leaves, words, blocks) == 0
    outs.append(sum_rows(d_part.get(), blocks, leaves * 2, Q))
    alphas = field_elems(12, 2 * leaves, Q)
    order = np.array([4, 0, 2, 5, 1, 3], dtype=np.int32)
    offsets = np.array([0, 2, 2, 6], dtype=np.int32)
    d_a, d_o, d_off = Buf.of(lib, alphas), Buf.of(lib, order), Buf.of(lib, offsets)
    d_fu = Buf(lib, 16 * n * 3)
    assert lib.aext2_build_fu_ffi(d_p.ptr, d_a.ptr, d_o.ptr, d_off.ptr, d_fu.ptr, n, 3, words) == 0
    outs.append(d_fu.get(count=2 * n * 3))
    assert lib.aext2_build_fu_ternary_ffi(d_p.ptr, d_n.ptr, d_a.ptr, d_o.ptr, d_off.ptr, d_fu.ptr, n, 3, words) == 0
    outs.append(d_fu.get(count=2 * n * 3))
    return outs


def test_lifts_selective_add_and_fu(libs):
    both(libs, _lifts_and_fu)


def _shared_and_factored(lib, log_n, uniq):
    n = 1 << log_n
    points = field_elems(31, 2 * log_n * uniq, Q)
    fu = field_elems(32, 2 * n * uniq, Q)
    d_r = Buf.of(lib, points)
    d_a, d_b = Buf(lib, 16 * n * uniq), Buf(lib, 16 * n * uniq)
    res = ctypes.c_void_p()
    assert lib.aext2_eq_dp_all_batched_ffi(d_r.ptr, d_a.ptr, d_b.ptr, log_n, uniq, n, ctypes.byref(res), None) == 0
    eq_dev = (d_a if res.value == d_a.ptr else d_b).get(count=2 * n * uniq)
    outs = [eq_dev]
    stride = 2 * n
    d_suf = Buf(lib, 8 * stride * uniq)
    assert lib.aext2_eq_suffix_dp_ffi(d_r.ptr, d_suf.ptr, log_n, uniq, stride) == 0
    suf = d_suf.get(count=stride * uniq).reshape(uniq, stride)
    outs.append(np.ascontiguousarray(suf[:, :2 * (n - 1)]).reshape(-1))   # stages t = 1..log_n fill n - 1 elements
    d_map = Buf.of(lib, np.arange(uniq, dtype=np.int32))
    d_eq, d_eq2 = Buf.of(lib, canon(eq_dev, Q)), Buf(lib, eq_dev.nbytes)
    d_f, d_f2 = Buf.of(lib, fu), Buf(lib, fu.nbytes)
    blocks = 4
    d_part = Buf(lib, 8 * blocks * uniq * 6)
    half = n // 2
    for t in range(log_n):
        assert lib.aext2_sharedeq_msg_ffi(d_eq.ptr, d_f.ptr, d_map.ptr, d_part.ptr, n, half, uniq, blocks) == 0
        outs.append(sum_rows(d_part.get(), blocks, uniq * 6, Q))
        off = (1 << (log_n - t - 1)) - 1
        assert lib.aext2_sharedeq_factored_msg_ffi(d_suf.ptr, d_f.ptr, d_part.ptr, off, stride, 2 * n, half, uniq, blocks) == 0
        outs.append(sum_rows(d_part.get(), blocks, uniq * 4, Q))
        r = field_elems(90 + t, 2, Q)
        assert lib.aext2_fold_single_ffi(d_eq.ptr, d_eq2.ptr, int(r[0]), int(r[1]), n, half, uniq) == 0
        assert lib.aext2_fold_single_ffi(d_f.ptr, d_f2.ptr, int(r[0]), int(r[1]), n, half, uniq) == 0
        d_eq, d_eq2, d_f, d_f2 = d_eq2, d_eq, d_f2, d_f
        full = d_f.get(count=2 * n * uniq).reshape(uniq, 2 * n)
        outs.append(np.ascontiguousarray(full[:, :2 * half]).reshape(-1))
        half //= 2
        if half == 0:
            break
    return outs


@pytest.mark.parametrize("log_n,uniq", [(3, 1), (7, 2), (11, 3)])
def test_shared_eq_and_factored_eq(libs, log_n, uniq):
    both(libs, _shared_and_factored, log_n, uniq)


# ---- K8 product sumcheck and table helpers -------------------------------------------------------

def _k8_sumcheck(lib, ntab, n):
    tabs = [np.ascontiguousarray(field_elems(400 + j, 8 << n, Q)) for j in range(ntab)]
    cur = [Buf.of(lib, t) for t in tabs]
    outs = []
    sums = np.zeros((ntab + 1) * 8, dtype=np.uint64)
    assert lib.agl_mpiop_sc_round(_ptrs(cur), ntab, 1 << n, ntab, sums.ctypes.data) == 0
    outs.append(sums.copy())
    r = field_elems(9, 8, Q)
    d_one = Buf(lib, 64 << (n - 1))
    assert lib.agl_mpiop_sc_fold(cur[0].ptr, d_one.ptr, 1 << n, r.ctypes.data) == 0
    outs.append(d_one.get(count=8 << (n - 1)))
    length = 1 << n
    while length >= 4:
        r = field_elems(500 + length, 8, Q)
        nxt = [Buf(lib, 64 * (length // 2)) for _ in range(ntab)]
        assert lib.agl_mpiop_sc_fold_round(_ptrs(cur), _ptrs(nxt), ntab, length, r.ctypes.data, ntab, sums.ctypes.data) == 0
        outs.append(sums.copy())
        outs.append(nxt[-1].get(count=8 * (length // 2)))
        cur, length = nxt, length // 2
    return outs


@pytest.mark.parametrize("ntab,n", [(2, 2), (3, 9), (6, 7), (2, 13)])
def test_k8_sumcheck(libs, ntab, n):
    both(libs, _k8_sumcheck, ntab, n)


def _k8_tables(lib):
    outs = []
    for n in (1, 2, 7, 12):
        point = field_elems(600 + n, 8 * n, Q)
        d_out = Buf(lib, 64 << n)
        assert lib.agl_mpiop_eq(point.ctypes.data, n, d_out.ptr) == 0
        outs.append(d_out.get(count=8 << n))
    nlo, nhi = 5, 4
    plo, phi = field_elems(21, 8 * nlo, Q), field_elems(22, 8 * nhi, Q)
    d_lo, d_hi, d_o = Buf(lib, 64 << nlo), Buf(lib, 64 << nhi), Buf(lib, 64 << (nlo + nhi))
    assert lib.agl_mpiop_eq(plo.ctypes.data, nlo, d_lo.ptr) == 0
    assert lib.agl_mpiop_eq(phi.ctypes.data, nhi, d_hi.ptr) == 0
    assert lib.agl_mpiop_eq_outer(d_lo.ptr, nlo, d_hi.ptr, nhi, d_o.ptr) == 0
    outs.append(d_o.get(count=8 << (nlo + nhi)))
    n = 777
    d_a, d_b = Buf.of(lib, field_elems(31, 8 * n, Q)), Buf.of(lib, field_elems(32, 8 * n, Q))
    c = field_elems(33, 8, Q)
    assert lib.agl_mpiop_axpy(d_a.ptr, d_b.ptr, n, c.ctypes.data) == 0
    outs.append(d_a.get(count=8 * n))
    d_base, d_k = Buf.of(lib, field_elems(34, n, Q)), Buf(lib, 64 * n)
    assert lib.agl_mpiop_lift(d_base.ptr, n, d_k.ptr) == 0
    outs.append(d_k.get(count=8 * n))
    # partial evaluation over a permuted split of 9 variables (4 stay, 5 bound), and of 14 (1 stays: wide form)
    for nv, keep, seed in ((9, 4, 3), (14, 1, 4)):
        perm = np.random.default_rng(seed).permutation(nv)
        rest_pos, fix_pos = np.array(perm[:keep], dtype=np.int32), np.array(perm[keep:], dtype=np.int32)
        vals = field_elems(50 + nv, 1 << nv, Q)
        point = field_elems(51, 8 * (nv - keep), Q)
        d_e = Buf(lib, 64 << (nv - keep))
        assert lib.agl_mpiop_eq(point.ctypes.data, nv - keep, d_e.ptr) == 0
        d_v, d_po = Buf.of(lib, vals), Buf(lib, 64 << keep)
        assert lib.agl_mpiop_pe(d_v.ptr, rest_pos.ctypes.data, keep, fix_pos.ctypes.data, nv - keep, d_e.ptr, d_po.ptr) == 0
        outs.append(d_po.get(count=8 << keep))
    for nn in (1, 7, 12, 17):
        d_vv = Buf.of(lib, field_elems(60 + nn, 1 << nn, Q))
        pt = field_elems(70 + nn, 8 * nn, Q)
        out = np.zeros(8, dtype=np.uint64)
        assert lib.agl_mpiop_mle(d_vv.ptr, pt.ctypes.data, nn, out.ctypes.data) == 0
        outs.append(out)
    src = field_elems(80, 8 << 6, Q)
    pos = np.array([5, 0, 9, 3, 7, 2], dtype=np.int32)
    nout = 1 << 10
    d_s, d_g = Buf.of(lib, src), Buf(lib, 64 * nout)
    assert lib.agl_mpiop_gather(d_s.ptr, pos.ctypes.data, 6, nout, d_g.ptr) == 0
    outs.append(d_g.get(count=8 * nout))
    sel = np.random.default_rng(3).integers(0, 2**63, size=500, dtype=np.uint64)
    d_sel, d_l = Buf.of(lib, sel), Buf(lib, 64 * 500)
    assert lib.agl_mpiop_sel_lookup(d_sel.ptr, 500, 7, 63, d_s.ptr, d_l.ptr) == 0
    outs.append(d_l.get(count=8 * 500))
    return outs


def test_k8_table_helpers(libs):
    both(libs, _k8_tables)


# ---- packed link sumcheck ----------------------------------------------------------------------

def _link_round(lib, fn, chunks, nc, *args, tail=()):
    partial = Buf(lib, nc * chunks * 7 * 16)
    out = Buf(lib, 7 * 16)
    assert fn(*args, partial.ptr, chunks, out.ptr, *tail) == 0
    return out.get(count=14)


def _link_dense_and_listed(lib, log_half, nc, density, first, chunks):
    half = 1 << log_half
    stride, ostride = 2 * half + 64, 2 * half
    w = sparse_ext(40 + log_half, nc * stride, density, ternary=bool(first))
    om, eq, tags = ext(41, nc * ostride), ext(42, half), ext(43, nc)
    d_w, d_om, d_eq, d_tags = Buf.of(lib, w), Buf.of(lib, om), Buf.of(lib, eq), Buf.of(lib, tags)
    outs = [_link_round(lib, lib.link_round_message_ffi, chunks, nc, d_w.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, stride, ostride, half,
                        nc, first)]
    wz = np.stack([(w[2 * e * stride:2 * (e * stride + 2 * half)].reshape(2, half, 2) != 0).any(axis=(0, 2)) for e in range(nc)])
    lists = support_lists(wz, extra_seed=2)
    d_eq_g = Buf.of(lib, ext(53, max(int(lists[2].sum()), 1)))     # named: a buffer lives as long as its Python object
    d_l = [Buf.of(lib, a) for a in lists]
    outs.append(_link_round(lib, lib.link_round_message_sparse_ffi, chunks, nc, d_w.ptr, d_om.ptr, d_eq_g.ptr, d_tags.ptr,
                            d_l[0].ptr, d_l[1].ptr, d_l[2].ptr, stride, ostride, half, nc, first))
    r = ext(82, 1)
    assert lib.link_fold_ffi(d_w.ptr, d_om.ptr, stride, ostride, half, nc, int(r[0]), int(r[1])) == 0
    live_w = d_w.get(count=2 * nc * stride).reshape(nc, 2 * stride)[:, :2 * half]
    live_o = d_om.get(count=2 * nc * ostride).reshape(nc, 2 * ostride)[:, :2 * half]
    outs += [np.ascontiguousarray(live_w).reshape(-1), np.ascontiguousarray(live_o).reshape(-1)]
    return outs


@pytest.mark.parametrize("log_half,nc,density,first,chunks", [(2, 1, 1.0, 0, 1), (9, 3, 0.3, 0, 4), (9, 3, 0.05, 1, 7), (13, 2, 1.0, 0, 16)])
def test_link_table_rounds_and_folds(libs, log_half, nc, density, first, chunks):
    both(libs, _link_dense_and_listed, log_half, nc, density, first, chunks)


def _link_bits(lib, log_half, nc, density):
    half = 1 << log_half
    stride = 2 * half
    words, b = random_bits(60 + log_half, nc * stride, density)
    om, eq, tags = ext(61, nc * stride), ext(62, half), ext(63, nc)
    d_bits, d_om, d_eq, d_tags = Buf.of(lib, words), Buf.of(lib, om), Buf.of(lib, eq), Buf.of(lib, tags)
    outs = [_link_round(lib, lib.link_round0_bits_ffi, 6, nc, d_bits.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, stride, half, nc)]
    table = Buf(lib, nc * stride * 16)
    assert lib.link_expand_bits_ffi(d_bits.ptr, table.ptr, len(words)) == 0
    outs.append(table.get(count=2 * nc * stride))
    pair = b.reshape(nc, 2, half).any(axis=1)
    lists = support_lists(pair, extra_seed=4)
    eq_g = np.concatenate([eq.reshape(half, 2)[lists[0][int(o):int(o) + int(n)]] for o, n in zip(lists[1], lists[2])]
                          + [np.zeros((1, 2), dtype=np.uint64)]).reshape(-1)
    d_l = [Buf.of(lib, a) for a in lists]
    d_eq_g = Buf.of(lib, eq_g)
    outs.append(_link_round(lib, lib.link_round0_bits_sparse_ffi, 4, nc, d_bits.ptr, d_om.ptr, d_eq_g.ptr, d_tags.ptr,
                            d_l[0].ptr, d_l[1].ptr, d_l[2].ptr, stride, half, nc))
    r = ext(82, 1)
    d_out = Buf(lib, nc * half * 16)
    assert lib.link_fold0_bits_ffi(d_bits.ptr, d_out.ptr, d_om.ptr, stride, half, nc, int(r[0]), int(r[1])) == 0
    outs.append(d_out.get(count=2 * nc * half))
    outs.append(np.ascontiguousarray(d_om.get(count=2 * nc * stride).reshape(nc, 2 * stride)[:, :2 * half]).reshape(-1))
    d_out2 = Buf(lib, nc * half * 16)
    assert lib.link_fold_w_ffi(d_bits.ptr, table.ptr, d_out2.ptr, stride, stride // 64, half, half, nc, 1, int(r[0]), int(r[1])) == 0
    outs.append(d_out2.get(count=2 * nc * half))
    assert lib.link_fold_w_ffi(d_bits.ptr, table.ptr, d_out2.ptr, stride, stride // 64, half, half, nc, 0, int(r[0]), int(r[1])) == 0
    outs.append(d_out2.get(count=2 * nc * half))
    return outs


def _link_listed_fold(lib, half, nc):
    stride = 2 * half
    w2, om2, r = sparse_ext(83, nc * stride, 0.05), ext(84, nc * stride), ext(82, 1)
    pair = (w2.reshape(nc, 2, half, 2) != 0).any(axis=(1, 3))
    d_l = [Buf.of(lib, a) for a in support_lists(pair, extra_seed=6)]
    d_w, d_om = Buf.of(lib, w2), Buf.of(lib, om2)
    assert lib.link_fold_sparse_ffi(d_w.ptr, d_om.ptr, d_l[0].ptr, d_l[1].ptr, d_l[2].ptr, stride, half, nc, int(r[0]), int(r[1])) == 0
    # only the low halves of the listed pairs are written; compare those rows' low halves
    return [np.ascontiguousarray(d.get(count=2 * nc * stride).reshape(nc, 2 * stride)[:, :2 * half]).reshape(-1) for d in (d_w, d_om)]


def test_link_listed_fold(libs):
    both(libs, _link_listed_fold, 512, 3)


@pytest.mark.parametrize("log_half,nc,density", [(5, 2, 0.5), (10, 3, 0.1), (14, 2, 0.003)])
def test_link_bit_rounds_and_folds(libs, log_half, nc, density):
    both(libs, _link_bits, log_half, nc, density)


def _link_interleaved(lib, first, rnd):
    block_bits, leaf_arity, nc = 3, 7, 2
    blocks = 1 << block_bits
    size = (1 << (leaf_arity - rnd)) * blocks
    half = size // 2
    w_stride = size + 32
    words, _ = random_bits(70 + rnd, nc * size if size >= 64 else 64 * nc, 0.2)
    bits_stride_words = max(size // 64, 1)
    w = sparse_ext(71 + rnd, nc * w_stride, 0.3)
    pts, scale, tags = ext(72, nc * blocks * leaf_arity), ext(73, nc * blocks), ext(74, nc)
    if first:
        bb = np.zeros((nc, size), dtype=bool)
        for e in range(nc):
            row = words[e * bits_stride_words:(e + 1) * bits_stride_words]
            bb[e] = [(int(row[i >> 6]) >> (i & 63)) & 1 for i in range(size)]
        pair = bb.reshape(nc, 2, half).any(axis=1)
    else:
        ws = np.stack([w[2 * e * w_stride:2 * (e * w_stride + size)].reshape(2, half, 2) for e in range(nc)])
        pair = (ws != 0).any(axis=(1, 3))
    lists = support_lists(pair, extra_seed=5)
    eq_g = ext(75, max(int(lists[2].sum()), 1))
    d_l = [Buf.of(lib, a) for a in lists]
    d_bits, d_w = Buf.of(lib, words), Buf.of(lib, w)
    d_pts, d_scale, d_eq_g, d_tags = Buf.of(lib, pts), Buf.of(lib, scale), Buf.of(lib, eq_g), Buf.of(lib, tags)
    return [_link_round(lib, lib.link_round_interleaved_ffi, 3, nc, d_bits.ptr, d_w.ptr, d_pts.ptr, d_scale.ptr,
                        d_eq_g.ptr, d_tags.ptr, d_l[0].ptr, d_l[1].ptr, d_l[2].ptr, w_stride, bits_stride_words,
                        half, nc, blocks - 1, block_bits, leaf_arity, rnd, first)]


@pytest.mark.parametrize("first,rnd", [(1, 0), (0, 2), (0, 5)])
def test_link_interleaved_round(libs, first, rnd):
    both(libs, _link_interleaved, first, rnd)


def _link_expansions(lib):
    nv = 11
    pt = ext(90, nv)
    table = np.zeros(2 << nv, dtype=np.uint64)
    table[0] = 1
    d_t = Buf.of(lib, table)
    span = 1
    for k in reversed(range(nv)):
        assert lib.link_eq_expand_ffi(d_t.ptr, span, int(pt[2 * k]), int(pt[2 * k + 1])) == 0
        span *= 2
    outs = [d_t.get(count=2 << nv)]
    lst = np.random.default_rng(1).integers(0, 1 << nv, size=777, dtype=np.uint32)
    d_o, d_pt, d_lst = Buf(lib, len(lst) * 16), Buf.of(lib, pt), Buf.of(lib, lst)
    assert lib.link_eq_gather_ffi(d_pt.ptr, nv, d_lst.ptr, d_o.ptr, len(lst)) == 0
    outs.append(d_o.get(count=2 * len(lst)))
    span, bases = 300, np.array([0, 1000, 5000], dtype=np.uint64)
    d_om, d_bases, d_rs = Buf.of(lib, ext(91, 6000)), Buf.of(lib, bases), Buf.of(lib, ext(92, 3))
    assert lib.link_omega_expand_ffi(d_om.ptr, d_bases.ptr, d_rs.ptr, span, 3) == 0
    outs.append(d_om.get(count=12000))
    return outs


def test_link_expansions_and_gather(libs):
    both(libs, _link_expansions)


# ---- sparse boolean check ----------------------------------------------------------------------

def _bool_rounds(lib, arity, n_terms, density, rounds):
    idx, off = make_terms(arity, arity, n_terms, density)
    n = len(idx)
    d_idx, d_off = Buf.of(lib, idx), Buf.of(lib, off)
    d_w, d_eq = Buf.of(lib, ext(20, n_terms)), Buf.of(lib, ext(21, 1 << arity))
    d_val = Buf(lib, n * 16)
    assert lib.agl_bool_init_val_ffi(d_val.ptr, n) == 0
    outs, raw = [d_val.get(count=2 * n)], set()
    grid_x = 2
    for rnd in range(rounds):
        d_flags, d_gid = Buf(lib, n * 4), Buf(lib, n * 4)
        d_partial = Buf(lib, grid_x * n_terms * 64)
        nb = (n + 255) // 256
        scratch_len = 8 * nb + 1024
        d_scratch = Buf(lib, 4 * scratch_len)
        msg = np.zeros(8, dtype=np.uint64)
        total = ctypes.c_uint32(0)
        assert lib.agl_bool_round_msg_ffi(d_idx.ptr, d_val.ptr, d_off.ptr, d_w.ptr, d_eq.ptr, n_terms, n, d_flags.ptr, d_gid.ptr,
                                          d_partial.ptr, grid_x, d_scratch.ptr, scratch_len, msg.ctypes.data,
                                          ctypes.byref(total)) == 0
        tot = int(total.value)
        assert 0 < tot <= n
        outs.append(msg.copy())
        raw.add(len(outs)); outs.append(np.array([tot], dtype=np.uint64))
        raw.add(len(outs)); outs.append(d_flags.get(np.uint32, count=n))
        flags = outs[-1].astype(bool)
        raw.add(len(outs)); outs.append(d_gid.get(np.uint32, count=n)[flags])   # ids of group leaders; the rest are not read
        r = ext(30 + rnd, 1)
        d_oidx, d_oval, d_ooff = Buf(lib, tot * 4), Buf(lib, tot * 16), Buf(lib, (n_terms + 1) * 4)
        assert lib.agl_bool_fold_ffi(d_idx.ptr, d_val.ptr, d_flags.ptr, d_gid.ptr, d_off.ptr, n_terms, n, int(r[0]), int(r[1]), tot,
                                     grid_x, d_oidx.ptr, d_oval.ptr, d_ooff.ptr) == 0
        raw.add(len(outs)); outs.append(d_oidx.get(np.uint32, count=tot))
        outs.append(d_oval.get(count=2 * tot))
        raw.add(len(outs)); outs.append(d_ooff.get(np.uint32, count=n_terms + 1))
        half = (1 << (arity - rnd)) // 2
        d_eq2 = Buf(lib, half * 16)
        assert lib.aext2_fold_single_ffi(d_eq.ptr, d_eq2.ptr, int(r[0]), int(r[1]), 2 * half, half, 1) == 0
        d_idx, d_val, d_off, d_eq, n = d_oidx, d_oval, d_ooff, d_eq2, tot
    out = Buf(lib, n_terms * 16)
    assert lib.agl_bool_finish_ffi(d_idx.ptr, d_val.ptr, d_off.ptr, n_terms, n, out.ptr) == 0
    outs.append(out.get(count=2 * n_terms))
    return outs, raw


@pytest.mark.parametrize("arity,n_terms,density", [(5, 3, 0.3), (10, 11, 0.05), (13, 40, 0.02)])
def test_boolean_check_rounds(libs, arity, n_terms, density):
    results = []
    for lib in libs:
        outs, raw = _bool_rounds(lib, arity, n_terms, density, arity)
        assert lib.cuda_device_synchronize() == 0
        results.append([np.asarray(o) if k in raw else canon(o, Q) for k, o in enumerate(outs)])
    ours, ref = results
    assert len(ours) == len(ref)
    for k, (a, b) in enumerate(zip(ours, ref)):
        assert a.shape == b.shape and np.array_equal(a, b), "output %d differs from the reference" % k


# ---- module commitment -------------------------------------------------------------------------

N = 4096


def _mcommit(lib, rows, k, V, C, wide, shards):
    seed = np.asarray([4, 4, 2, 2, 1, 1, 0, 9], dtype=np.uint32)
    rng = np.random.default_rng(8 + rows + C)
    key = Buf(lib, k * C * rows * N * 4)
    assert lib.agl_mcommit_keygen(seed.ctypes.data, 1, rows, 3, C, k, key.ptr) == 0
    if wide:
        x = rng.integers(-(1 << 36), 1 << 36, size=(V, C, N), dtype=np.int64)
    else:
        x = rng.integers(-128, 128, size=(V, C, N), dtype=np.int8)
    accs = []
    bounds = np.linspace(0, C, shards + 1).astype(int)
    for s in range(shards):
        lo, hi = int(bounds[s]), int(bounds[s + 1])
        dx = Buf.of(lib, np.ascontiguousarray(x[:, lo:hi]))
        di = Buf.of(lib, np.arange(lo, hi, dtype=np.uint32))
        acc = Buf(lib, V * k * rows * N * 4)
        assert lib.agl_mcommit_partial(key.ptr, C, rows, k, dx.ptr, x.dtype.itemsize, V, hi - lo, 0, di.ptr, acc.ptr) == 0
        accs.append(acc)
    for a in accs[1:]:
        assert lib.agl_mcommit_add(accs[0].ptr, a.ptr, V, k, rows) == 0
    err = Buf.of(lib, rng.integers(-1, 2, size=(V, rows, N)).astype(np.int64))
    out = Buf(lib, V * rows * N * 8)
    assert lib.agl_mcommit_finish(accs[0].ptr, V, k, rows, err.ptr, out.ptr) == 0
    return [out.get(count=V * rows * N)]


@pytest.mark.parametrize("rows,k,V,C,wide,shards", [(2, 3, 1, 4, False, 1), (16, 5, 2, 5, True, 2), (5, 3, 1, 20, False, 1)])
def test_module_commitment(libs, rows, k, V, C, wide, shards):
    both(libs, _mcommit, rows, k, V, C, wide, shards)


# ---- dense Ajtai commit ------------------------------------------------------------------------

def _ajtai_dense(lib, n_ring, B, chunk, col_offset):
    key = np.arange(1, 9, dtype=np.uint32)
    z = splitmix64(77 + n_ring, B * n_ring)
    d_key, d_z = Buf.of(lib, key), Buf.of(lib, z)
    d_out = Buf(lib, B * 42 * 64 * 8)
    assert lib.ajtai_commit_dense_batched_at_ffi(d_key.ptr, d_z.ptr, n_ring, B, chunk, col_offset, d_out.ptr) == 0
    return [d_out.get(count=B * 42 * 64)]


@pytest.mark.parametrize("n_ring,B,chunk,col_offset", [(64, 1, 64, 0), (256, 4, 128, 1000), (1024, 16, 256, 2**33 + 5)])
def test_ajtai_dense_commit(libs, n_ring, B, chunk, col_offset):
    both(libs, _ajtai_dense, n_ring, B, chunk, col_offset)
