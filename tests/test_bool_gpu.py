"""GPU parity of the sparse boolean-check sumcheck against the CPU oracle, through the C-ABI, round by round
(flags, group ids, message, folded lists, offsets, final values). Bit-exact."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from oracle import pyoracle as po
from .bool_cases import ext, fold_eq, make_terms, ones
from .link_cases import Q, e2_add, lagrange_at

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def _gpu_round(lib, d_idx, d_val, d_off, d_w, d_eq, n_terms, n):
    d_flags, d_gid = DeviceBuffer(lib, max(n, 1) * 4), DeviceBuffer(lib, max(n, 1) * 4)
    msg = np.zeros(8, dtype=np.uint64)
    total = ctypes.c_uint32(0)
    rc = lib.agl_bool_round_msg_ffi(d_idx.ptr, d_val.ptr, d_off.ptr, d_w.ptr, d_eq.ptr, n_terms, n, d_flags.ptr, d_gid.ptr, None, 1, None, 0,
                                    msg.ctypes.data, ctypes.byref(total))
    assert rc == 0
    return d_flags, d_gid, msg, int(total.value)


@pytest.mark.parametrize("arity,n_terms,density", [(5, 3, 0.3), (10, 11, 0.05), (13, 40, 0.02), (12, 5000, 0.001)])
def test_every_round_matches_the_oracle(lib, arity, n_terms, density):
    idx, off = make_terms(arity, arity, n_terms, density)
    n = len(idx)
    w, eq = ext(20, n_terms), ext(21, 1 << arity)
    d_idx, d_off, d_w, d_eq = (DeviceBuffer.from_numpy(lib, a) for a in (idx, off, w, eq))
    d_val = DeviceBuffer(lib, max(n, 1) * 16)
    assert lib.agl_bool_init_val_ffi(d_val.ptr, n) == 0
    val = ones(n)
    assert np.array_equal(d_val.to_numpy(count=2 * n), val)
    for rnd in range(arity):
        flags, gid, msg, total = po.bool_round(idx, val, off, w, eq)
        d_flags, d_gid, g_msg, g_total = _gpu_round(lib, d_idx, d_val, d_off, d_w, d_eq, n_terms, n)
        assert g_total == total and np.array_equal(g_msg, msg)
        assert np.array_equal(d_flags.to_numpy("uint32", count=n), flags)
        assert np.array_equal(d_gid.to_numpy("uint32", count=n), gid)
        r = ext(30 + rnd, 1)
        idx2, val2, off2 = po.bool_fold(idx, val, flags, gid, off, r, total)
        d_oidx, d_oval, d_ooff = DeviceBuffer(lib, max(total, 1) * 4), DeviceBuffer(lib, max(total, 1) * 16), DeviceBuffer(lib, (n_terms + 1) * 4)
        assert lib.agl_bool_fold_ffi(d_idx.ptr, d_val.ptr, d_flags.ptr, d_gid.ptr, d_off.ptr, n_terms, n, int(r[0]), int(r[1]), total, 1,
                                     d_oidx.ptr, d_oval.ptr, d_ooff.ptr) == 0
        assert np.array_equal(d_oidx.to_numpy("uint32", count=total), idx2)
        assert np.array_equal(d_oval.to_numpy(count=2 * total), val2)
        assert np.array_equal(d_ooff.to_numpy("uint32"), off2)
        idx, val, off, n = np.ascontiguousarray(idx2), np.ascontiguousarray(val2), off2.copy(), total
        d_idx, d_val, d_off = d_oidx, d_oval, d_ooff
        eq = fold_eq(eq, r, Q) if arity <= 10 else None
        half = (1 << (arity - rnd)) // 2
        d_eq2 = DeviceBuffer(lib, half * 16)
        assert lib.aext2_fold_single_ffi(d_eq.ptr, d_eq2.ptr, int(r[0]), int(r[1]), 2 * half, half, 1) == 0
        if eq is None:
            eq = d_eq2.to_numpy()
        else:
            assert np.array_equal(d_eq2.to_numpy(), eq)
        d_eq = d_eq2
    out = DeviceBuffer(lib, n_terms * 16)
    assert lib.agl_bool_finish_ffi(d_idx.ptr, d_val.ptr, d_off.ptr, n_terms, n, out.ptr) == 0
    want = np.zeros(2 * n_terms, dtype=np.uint64)
    for t in range(n_terms):
        if off[t] < off[t + 1] and idx[off[t]] == 0:
            want[2 * t:2 * t + 2] = val[2 * off[t]:2 * off[t] + 2]
    assert np.array_equal(out.to_numpy(), want)


def test_sumcheck_identities_at_a_larger_size(lib):
    """About 2^21 entries over 64 terms at arity 22: zero claim, then m_{i+1}(0) + m_{i+1}(1) = m_i(r) for six rounds."""
    arity, n_terms = 22, 64
    rng = np.random.default_rng(4)
    segs = [np.unique(rng.integers(0, 1 << arity, size=1 << 15, dtype=np.uint64)).astype(np.uint32) for _ in range(n_terms)]
    off = np.zeros(n_terms + 1, dtype=np.uint32)
    off[1:] = np.cumsum([len(s) for s in segs])
    idx = np.ascontiguousarray(np.concatenate(segs))
    n = len(idx)
    d_idx, d_off = DeviceBuffer.from_numpy(lib, idx), DeviceBuffer.from_numpy(lib, off)
    d_w = DeviceBuffer.from_numpy(lib, ext(40, n_terms))
    d_eq = DeviceBuffer.from_numpy(lib, ext(41, 1 << arity))
    d_val = DeviceBuffer(lib, n * 16)
    assert lib.agl_bool_init_val_ffi(d_val.ptr, n) == 0
    prev = (0, 0)
    for rnd in range(6):
        d_flags, d_gid, msg, total = _gpu_round(lib, d_idx, d_val, d_off, d_w, d_eq, n_terms, n)
        m = [(int(msg[2 * k]), int(msg[2 * k + 1])) for k in range(4)]
        assert e2_add(m[0], m[1]) == prev
        assert 0 < total <= n
        r = ext(50 + rnd, 1)
        prev = lagrange_at(m, (int(r[0]), int(r[1])))
        d_oidx, d_oval, d_ooff = DeviceBuffer(lib, total * 4), DeviceBuffer(lib, total * 16), DeviceBuffer(lib, (n_terms + 1) * 4)
        assert lib.agl_bool_fold_ffi(d_idx.ptr, d_val.ptr, d_flags.ptr, d_gid.ptr, d_off.ptr, n_terms, n, int(r[0]), int(r[1]), total, 1,
                                     d_oidx.ptr, d_oval.ptr, d_ooff.ptr) == 0
        half = (1 << (arity - rnd)) // 2
        d_eq2 = DeviceBuffer(lib, half * 16)
        assert lib.aext2_fold_single_ffi(d_eq.ptr, d_eq2.ptr, int(r[0]), int(r[1]), 2 * half, half, 1) == 0
        d_idx, d_val, d_off, d_eq, n = d_oidx, d_oval, d_ooff, d_eq2, total


def test_empty_and_argument_errors(lib):
    msg = np.ones(8, dtype=np.uint64)
    total = ctypes.c_uint32(7)
    assert lib.agl_bool_round_msg_ffi(None, None, None, None, None, 0, 0, None, None, None, 1, None, 0, msg.ctypes.data, ctypes.byref(total)) == 0
    assert not msg.any() and total.value == 0
    b = DeviceBuffer(lib, 256)
    assert lib.agl_bool_round_msg_ffi(b.ptr, b.ptr, b.ptr, b.ptr, b.ptr, 0, 4, b.ptr, b.ptr, None, 1, None, 0, msg.ctypes.data, ctypes.byref(total)) == -2
    assert lib.agl_bool_init_val_ffi(None, 0) == 0 and lib.agl_bool_finish_ffi(None, None, None, 0, 0, None) == 0
