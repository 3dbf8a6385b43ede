"""Whole linear sumcheck over almost-Goldilocks through the C-ABI (agl_sumcheck_prove_*_ffi,
agl_sumcheck_verify_ffi) against the CPU oracle, bit for bit: the reference's own deterministic
cases (claim 887 among them), random base-field and extension tables with one to five factors,
non-canonical input words, a transcript that continues across two proofs, and prove -> verify at a
size the oracle does not run."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from matrix_b200.inputs import AGL_Q, splitmix64
from oracle import pyoracle

from .agl_sumcheck_cases import CASES, lifted

pytestmark = pytest.mark.gpu
Q = AGL_Q


def _transcript(lib, label):
    h = ctypes.c_void_p()
    assert lib.agl_transcript_create(label, len(label), ctypes.byref(h)) == 0
    return h


def _state(lib, h):
    st = np.zeros(12, dtype=np.uint64)
    assert lib.agl_transcript_state(h, st.ctypes.data) == 0
    return st


def _prove(lib, tables, d, nv, base, h, host=False):
    msgs = np.zeros(max(nv, 1) * (d + 1) * 2, dtype=np.uint64)
    ch = np.zeros(max(nv, 1) * 2, dtype=np.uint64)
    fe = np.zeros(2 * d, dtype=np.uint64)
    fin = np.zeros(2, dtype=np.uint64)
    tables = np.ascontiguousarray(tables, dtype=np.uint64)
    if host:
        rc = lib.agl_sumcheck_prove_host_ffi(tables.ctypes.data, d, nv, int(base), h, msgs.ctypes.data, ch.ctypes.data,
                                             fe.ctypes.data, fin.ctypes.data)
    else:
        dt = DeviceBuffer.from_numpy(lib, tables)
        rc = lib.agl_sumcheck_prove_device_ffi(dt.ptr, d, nv, int(base), h, msgs.ctypes.data, ch.ctypes.data,
                                               fe.ctypes.data, fin.ctypes.data)
    assert rc == 0
    return msgs[:nv * (d + 1) * 2], ch[:2 * nv], fe, fin


def _verify(lib, msgs, fin, claim, d, nv, label):
    h = _transcript(lib, label)
    ok = ctypes.c_int(-1)
    ch = np.zeros(max(nv, 1) * 2, dtype=np.uint64)
    msgs = np.ascontiguousarray(msgs, dtype=np.uint64)
    cl = np.array(claim, dtype=np.uint64)
    assert lib.agl_sumcheck_verify_ffi(msgs.ctypes.data, fin.ctypes.data, cl.ctypes.data, d, nv, h, ch.ctypes.data,
                                       ctypes.byref(ok)) == 0
    st = _state(lib, h)
    lib.agl_transcript_destroy(h)
    return ok.value == 1, ch[:2 * nv], st


def test_reference_cases():
    lib = load_agl()
    for label, nv, tables, claim in CASES:
        d = len(tables)
        want = pyoracle.agl_sumcheck_prove(lifted(tables), d, nv, False, label)
        for base, tabs in ((False, lifted(tables)), (True, np.array(tables, dtype=np.uint64).reshape(-1))):
            for host in (False, True):
                h = _transcript(lib, label)
                msgs, ch, fe, fin = _prove(lib, tabs, d, nv, base, h, host)
                assert list(msgs) == list(want[0]) and list(ch) == list(want[1])
                assert list(fe) == list(want[2]) and list(fin) == list(want[3])
                assert list(_state(lib, h)) == list(want[4])
                lib.agl_transcript_destroy(h)
        assert (int(msgs[0]) + int(msgs[2])) % Q == claim
        ok, vch, _ = _verify(lib, msgs, fin, [claim, 0], d, nv, label)
        assert ok and list(vch) == list(ch)
        assert _verify(lib, msgs, fin, [claim, 0], d, nv, label)[0] == pyoracle.agl_sumcheck_verify(msgs, fin, [claim, 0], d, nv, label)[0]
        bad = msgs.copy()
        bad[0] = (int(bad[0]) + 1) % Q
        assert not _verify(lib, bad, fin, [claim, 0], d, nv, label)[0]
        assert not _verify(lib, msgs, fin, [claim + 1, 0], d, nv, label)[0]


@pytest.mark.parametrize("d,nv,base", [(1, 9, True), (2, 12, True), (3, 11, False), (4, 8, False), (5, 7, True),
                                        (2, 1, False), (3, 0, False), (2, 14, False), (1, 19, True)])
def test_random_tables_match_oracle(d, nv, base):
    lib = load_agl()
    n = 1 << nv
    raw = splitmix64(100 + 10 * d + nv, n * d * (1 if base else 2))  # raw words: some at or above q
    raw[:3] = [Q, 2**64 - 1, Q - 1][:len(raw[:3])]
    label = b"parity"
    want = pyoracle.agl_sumcheck_prove(raw, d, nv, base, label)
    h = _transcript(lib, label)
    msgs, ch, fe, fin = _prove(lib, raw, d, nv, base, h)
    assert list(msgs) == list(want[0]) and list(ch) == list(want[1])
    assert list(fe) == list(want[2]) and list(fin) == list(want[3])
    assert list(_state(lib, h)) == list(want[4])
    lib.agl_transcript_destroy(h)


def test_transcript_continues_and_large_case_verifies():
    lib = load_agl()
    d, nv = 3, 20
    n = 1 << nv
    tabs = splitmix64(7, n * d) % np.uint64(Q)
    # the claim with Python integers
    cols = [[int(x) for x in tabs[i * n:(i + 1) * n]] for i in range(d)]
    claim = sum(a * b * c for a, b, c in zip(*cols)) % Q
    h = _transcript(lib, b"two-proofs")
    m1, c1, _, f1 = _prove(lib, tabs, d, nv, True, h)
    mid = _state(lib, h).copy()
    m2, c2, _, f2 = _prove(lib, tabs, d, nv, True, h)  # same tables, later transcript state: other challenges
    lib.agl_transcript_destroy(h)
    assert list(m1[:8]) == list(m2[:8]) and list(c1) != list(c2)
    ok, vch, st = _verify(lib, m1, f1, [claim, 0], d, nv, b"two-proofs")
    assert ok and list(vch) == list(c1) and list(st) == list(mid)
    assert not _verify(lib, m2, f2, [claim, 0], d, nv, b"two-proofs")[0]  # needs the transcript after proof one
    # argument errors
    out = np.zeros(8, dtype=np.uint64)
    assert lib.agl_sumcheck_prove_device_ffi(None, 2, 2, 1, None, out.ctypes.data, None, None, out.ctypes.data) != 0
