"""GPU parity of the packed link sumcheck (all thirteen entry points) against the CPU oracle, through the C-ABI.
Bit-exact; the different device forms are also checked against one another."""
import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from oracle import pyoracle as po
from .link_cases import Q, e2_add, ext, lagrange_at, random_bits, sparse_ext, support_lists

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


_keep = []


@pytest.fixture(autouse=True)
def _release_buffers():
    yield
    _keep.clear()


def dev(lib, a):
    """Uploads and keeps the buffer alive until the end of the test (calls take raw pointers)."""
    b = DeviceBuffer.from_numpy(lib, a)
    _keep.append(b)
    return b


def _round(lib, fn, chunks, n_commit, *args_before, tail=()):
    partial = DeviceBuffer(lib, n_commit * chunks * 7 * 16)
    out = DeviceBuffer(lib, 7 * 16)
    rc = fn(*args_before, partial.ptr, chunks, out.ptr, *tail)
    assert rc == 0
    return out.to_numpy()


@pytest.mark.parametrize("log_half,nc,density,first,chunks", [(2, 1, 1.0, 0, 1), (9, 3, 0.3, 0, 4), (9, 3, 0.05, 1, 7), (13, 2, 1.0, 0, 16),
                                                              (12, 5, 0.01, 0, 3)])
def test_dense_round_message(lib, log_half, nc, density, first, chunks):
    half = 1 << log_half
    stride, ostride = 2 * half + 64, 2 * half
    w = sparse_ext(40 + log_half, nc * stride, density, ternary=bool(first))
    om, eq, tags = ext(41, nc * ostride), ext(42, half), ext(43, nc)
    got = _round(lib, lib.link_round_message_ffi, chunks, nc, dev(lib, w).ptr, dev(lib, om).ptr, dev(lib, eq).ptr, dev(lib, tags).ptr, stride,
                 ostride, half, nc, first)
    want = po.link_round(eq, tags, half, nc, first, w=w, omega=om, w_stride=stride, omega_stride=ostride)
    assert np.array_equal(got, want)


def test_raw_words_are_reduced(lib):
    """Inputs as any 64-bit representatives."""
    half, nc = 256, 2
    rng = np.random.default_rng(3)
    raw = lambda n: rng.integers(0, 2**64, size=2 * n, dtype=np.uint64)
    w, om, eq, tags = raw(nc * 2 * half), raw(nc * 2 * half), raw(half), raw(nc)
    got = _round(lib, lib.link_round_message_ffi, 3, nc, dev(lib, w).ptr, dev(lib, om).ptr, dev(lib, eq).ptr, dev(lib, tags).ptr, 2 * half,
                 2 * half, half, nc, 0)
    assert np.array_equal(got, po.link_round(eq, tags, half, nc, 0, w=w, omega=om, w_stride=2 * half, omega_stride=2 * half))


@pytest.mark.parametrize("log_half,nc,density,first", [(8, 3, 0.1, 0), (11, 2, 0.02, 1), (6, 4, 0.0, 0)])
def test_listed_round_message(lib, log_half, nc, density, first):
    half = 1 << log_half
    stride = 2 * half
    w = sparse_ext(50 + log_half, nc * stride, density, ternary=bool(first))
    om, tags = ext(51, nc * stride), ext(52, nc)
    wz = (w.reshape(nc, 2, half, 2) != 0).any(axis=(1, 3))
    lists = support_lists(wz, extra_seed=2)
    total = int(lists[2].sum())
    eq_g = ext(53, max(total, 1))
    chunks = 5
    got = _round(lib, lib.link_round_message_sparse_ffi, chunks, nc, dev(lib, w).ptr, dev(lib, om).ptr, dev(lib, eq_g).ptr, dev(lib, tags).ptr,
                 dev(lib, lists[0]).ptr, dev(lib, lists[1]).ptr, dev(lib, lists[2]).ptr, stride, stride, half, nc, first)
    want = po.link_round(eq_g, tags, half, nc, first, w=w, omega=om, lists=lists, w_stride=stride, omega_stride=stride)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("log_half,nc,density", [(5, 2, 0.5), (6, 1, 0.5), (10, 3, 0.1), (14, 2, 0.003), (12, 2, 1.0)])
def test_bit_packed_round_zero(lib, log_half, nc, density):
    half = 1 << log_half
    stride = 2 * half
    words, b = random_bits(60 + log_half, nc * stride, density)
    om, eq, tags = ext(61, nc * stride), ext(62, half), ext(63, nc)
    d_bits, d_om, d_eq, d_tags = dev(lib, words), dev(lib, om), dev(lib, eq), dev(lib, tags)
    got = _round(lib, lib.link_round0_bits_ffi, 6, nc, d_bits.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, stride, half, nc)
    want = po.link_round(eq, tags, half, nc, 1, bits=words, omega=om, bits_stride_words=stride // 64, omega_stride=stride)
    assert np.array_equal(got, want)
    # the expanded table through the general kernel gives the same message
    table = DeviceBuffer(lib, nc * stride * 16)
    assert lib.link_expand_bits_ffi(d_bits.ptr, table.ptr, len(words)) == 0
    assert np.array_equal(table.to_numpy(), po.link_expand_bits(words))
    again = _round(lib, lib.link_round_message_ffi, 6, nc, table.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, stride, stride, half, nc, 1)
    assert np.array_equal(again, want)
    # support lists
    pair = b.reshape(nc, 2, half).any(axis=1)
    lists = support_lists(pair, extra_seed=4)
    eq_g = np.concatenate([eq.reshape(half, 2)[lists[0][int(o):int(o) + int(n)]] for o, n in zip(lists[1], lists[2])]
                          + [np.zeros((1, 2), dtype=np.uint64)]).reshape(-1)
    listed = _round(lib, lib.link_round0_bits_sparse_ffi, 4, nc, d_bits.ptr, d_om.ptr, dev(lib, eq_g).ptr, d_tags.ptr, dev(lib, lists[0]).ptr,
                    dev(lib, lists[1]).ptr, dev(lib, lists[2]).ptr, stride, half, nc)
    assert np.array_equal(listed, want)


@pytest.mark.parametrize("first,rnd", [(1, 0), (0, 2), (0, 5)])
def test_interleaved_round_message(lib, first, rnd):
    """Block index in the low bits (8 blocks), weights evaluated from the leaf points."""
    block_bits, leaf_arity, nc = 3, 7, 2
    blocks = 1 << block_bits
    m = leaf_arity - rnd
    size = (1 << m) * blocks
    half = size // 2
    w_stride = size + 32
    words, b = random_bits(70 + rnd, nc * size if size >= 64 else 64 * nc, 0.2)
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
    d_bits, d_w = dev(lib, words), dev(lib, w)
    got = _round(lib, lib.link_round_interleaved_ffi, 3, nc, d_bits.ptr if first else None, None if first else d_w.ptr, dev(lib, pts).ptr,
                 dev(lib, scale).ptr, dev(lib, eq_g).ptr, dev(lib, tags).ptr, dev(lib, lists[0]).ptr, dev(lib, lists[1]).ptr,
                 dev(lib, lists[2]).ptr, w_stride, bits_stride_words, half, nc, blocks - 1, block_bits, leaf_arity, rnd, first)
    want = po.link_round(eq_g, tags, half, nc, first, bits=words if first else None, w=None if first else w, pts=pts, scale=scale,
                         lists=lists, w_stride=w_stride, bits_stride_words=bits_stride_words, block_mask=blocks - 1,
                         block_bits=block_bits, leaf_arity=leaf_arity, rnd=rnd)
    assert np.array_equal(got, want)


def test_folds(lib):
    half, nc = 512, 3
    stride, ostride = 2 * half + 16, 2 * half
    w, om, r = sparse_ext(80, nc * stride, 0.2), ext(81, nc * ostride), ext(82, 1)
    d_w, d_om = dev(lib, w), dev(lib, om)
    assert lib.link_fold_ffi(d_w.ptr, d_om.ptr, stride, ostride, half, nc, int(r[0]), int(r[1])) == 0
    assert np.array_equal(d_w.to_numpy(), po.link_fold_rows(w, stride, half, nc, r))
    assert np.array_equal(d_om.to_numpy(), po.link_fold_rows(om, ostride, half, nc, r))
    # listed fold touches only the listed pairs
    w2, om2 = sparse_ext(83, nc * ostride, 0.05), ext(84, nc * ostride)
    pair = (w2.reshape(nc, 2, half, 2) != 0).any(axis=(1, 3))
    lists = support_lists(pair, extra_seed=6)
    d_w, d_om = dev(lib, w2), dev(lib, om2)
    assert lib.link_fold_sparse_ffi(d_w.ptr, d_om.ptr, dev(lib, lists[0]).ptr, dev(lib, lists[1]).ptr, dev(lib, lists[2]).ptr, ostride, half, nc,
                                    int(r[0]), int(r[1])) == 0
    assert np.array_equal(d_w.to_numpy(), po.link_fold_rows(w2, ostride, half, nc, r, lists))
    assert np.array_equal(d_om.to_numpy(), po.link_fold_rows(om2, ostride, half, nc, r, lists))
    # bits in, half-size table out, omega in place
    words, _ = random_bits(85, nc * ostride, 0.3)
    d_om, d_out = dev(lib, om), DeviceBuffer(lib, nc * half * 16)
    assert lib.link_fold0_bits_ffi(dev(lib, words).ptr, d_out.ptr, d_om.ptr, ostride, half, nc, int(r[0]), int(r[1])) == 0
    assert np.array_equal(d_out.to_numpy(), po.link_fold_w(words, None, 0, ostride // 64, half, half, nc, r))
    assert np.array_equal(d_om.to_numpy(), po.link_fold_rows(om, ostride, half, nc, r))
    # witness-only folds, both sources, output rows wider than half
    out_stride = half + 8
    d_out = DeviceBuffer(lib, nc * out_stride * 16)
    assert lib.cuda_memset(d_out.ptr, 0, nc * out_stride * 16) == 0
    assert lib.link_fold_w_ffi(dev(lib, words).ptr, None, d_out.ptr, 0, ostride // 64, out_stride, half, nc, 1, int(r[0]), int(r[1])) == 0
    assert np.array_equal(d_out.to_numpy(), po.link_fold_w(words, None, 0, ostride // 64, out_stride, half, nc, r))
    assert lib.link_fold_w_ffi(None, dev(lib, w).ptr, d_out.ptr, stride, 0, out_stride, half, nc, 0, int(r[0]), int(r[1])) == 0
    assert np.array_equal(d_out.to_numpy(), po.link_fold_w(None, w, stride, 0, out_stride, half, nc, r))


def test_expansions_and_gather(lib):
    nv = 11
    pt = ext(90, nv)
    table = np.zeros(2 << nv, dtype=np.uint64)
    table[0] = 1
    d_t = dev(lib, table)
    span = 1
    for k in reversed(range(nv)):
        assert lib.link_eq_expand_ffi(d_t.ptr, span, int(pt[2 * k]), int(pt[2 * k + 1])) == 0
        span *= 2
    lst = np.random.default_rng(1).integers(0, 1 << nv, size=777, dtype=np.uint32)
    got = d_t.to_numpy()
    assert np.array_equal(got, po.link_eq_gather(pt, nv, np.arange(1 << nv, dtype=np.uint32)))
    d_o = DeviceBuffer(lib, len(lst) * 16)
    assert lib.link_eq_gather_ffi(dev(lib, pt).ptr, nv, dev(lib, lst).ptr, d_o.ptr, len(lst)) == 0
    assert np.array_equal(d_o.to_numpy(), got.reshape(-1, 2)[lst].reshape(-1))
    # three weight slices expanded in one launch, each with its own challenge
    span, bases = 300, np.array([0, 1000, 5000], dtype=np.uint64)
    om = ext(91, 6000)
    rs = ext(92, 3)
    d_om = dev(lib, om)
    assert lib.link_omega_expand_ffi(d_om.ptr, dev(lib, bases).ptr, dev(lib, rs).ptr, span, 3) == 0
    want = om.copy()
    for q, base in enumerate(bases):
        sl = po.link_eq_expand(om[2 * int(base):2 * (int(base) + 2 * span)], span, rs[2 * q:2 * q + 2])
        want[2 * int(base):2 * (int(base) + 2 * span)] = sl
    assert np.array_equal(d_om.to_numpy(), want)


def test_rounds_chain_at_a_larger_size(lib):
    """2^20 coefficients per commitment from bits: E_{i+1}(0) + E_{i+1}(1) = E_i(r) across the bit round and two
    table rounds, and the bit round equals the dense round on the expanded table."""
    log_n, nc = 20, 2
    n = 1 << log_n
    half = n // 2
    words, _ = random_bits(95, nc * n, 0.02)
    om, tags = ext(96, nc * n), ext(97, nc)
    d_bits, d_om, d_tags = dev(lib, words), dev(lib, om), dev(lib, tags)
    d_eq = dev(lib, ext(98, half))
    chunks = 64
    msg = _round(lib, lib.link_round0_bits_ffi, chunks, nc, d_bits.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, n, half, nc)
    table = DeviceBuffer(lib, nc * n * 16)
    assert lib.link_expand_bits_ffi(d_bits.ptr, table.ptr, len(words)) == 0
    dense = _round(lib, lib.link_round_message_ffi, chunks, nc, table.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, n, n, half, nc, 1)
    assert np.array_equal(msg, dense)
    d_w = DeviceBuffer(lib, nc * half * 16)
    r = ext(99, 1)
    assert lib.link_fold0_bits_ffi(d_bits.ptr, d_w.ptr, d_om.ptr, n, half, nc, int(r[0]), int(r[1])) == 0
    w_stride = half
    for rnd in range(2):
        E = [(int(msg[8 + 2 * k]), int(msg[9 + 2 * k])) for k in range(3)]
        half //= 2
        msg = _round(lib, lib.link_round_message_ffi, chunks, nc, d_w.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, w_stride, n, half, nc, 0)
        s = e2_add((int(msg[8]), int(msg[9])), (int(msg[10]), int(msg[11])))
        assert s == lagrange_at(E, (int(r[0]), int(r[1])))
        r = ext(100 + rnd, 1)
        assert lib.link_fold_ffi(d_w.ptr, d_om.ptr, w_stride, n, half, nc, int(r[0]), int(r[1])) == 0


def test_argument_errors(lib):
    b = DeviceBuffer(lib, 4096)
    assert lib.link_round_message_ffi(None, b.ptr, b.ptr, b.ptr, 8, 8, 4, 1, 0, b.ptr, 1, b.ptr) == -2
    assert lib.link_round_message_ffi(b.ptr, b.ptr, b.ptr, b.ptr, 8, 8, 4, 1, 0, b.ptr, 0, b.ptr) == -2
    assert lib.link_round0_bits_ffi(b.ptr, b.ptr, b.ptr, b.ptr, 100, 50, 1, b.ptr, 1, b.ptr) == -2
    assert lib.link_eq_gather_ffi(b.ptr, 40, b.ptr, b.ptr, 1) == -2
    assert lib.link_fold_ffi(b.ptr, b.ptr, 8, 8, 0, 1, 1, 0) == 0
