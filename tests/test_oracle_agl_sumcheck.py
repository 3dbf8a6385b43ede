"""The oracle's almost-Goldilocks linear sumcheck prover and verifier on the reference's own test
cases (zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:117-207: prove -> verify, first message sums to
the claim 887, a tampered message is rejected) and against Python integers on random tables."""
import numpy as np

from matrix_b200.inputs import AGL_Q, splitmix64
from oracle import pyoracle

from .agl_sumcheck_cases import CASES, lifted

Q = AGL_Q


def _mul(a, b):
    return ((a[0] * b[0] + 3 * a[1] * b[1]) % Q, (a[0] * b[1] + a[1] * b[0]) % Q)


def test_reference_cases():
    for label, nv, tables, claim in CASES:
        d = len(tables)
        msgs, ch, fe, fin, _ = pyoracle.agl_sumcheck_prove(lifted(tables), d, nv, False, label)
        assert (int(msgs[0]) + int(msgs[2])) % Q == claim and (int(msgs[1]) + int(msgs[3])) % Q == 0
        ok, vch = pyoracle.agl_sumcheck_verify(msgs, fin, [claim, 0], d, nv, label)
        assert ok and list(vch) == list(ch)
        # the same tables given as base-field words
        base = np.array(tables, dtype=np.uint64).reshape(-1)
        msgs_b, ch_b, _, fin_b, _ = pyoracle.agl_sumcheck_prove(base, d, nv, True, label)
        assert list(msgs_b) == list(msgs) and list(fin_b) == list(fin) and list(ch_b) == list(ch)
        # tampering (cpu_ext2_prover.rs:140-157) and a wrong claim are rejected; another label changes the challenges
        bad = msgs.copy()
        bad[0] = (int(bad[0]) + 1) % Q
        assert not pyoracle.agl_sumcheck_verify(bad, fin, [claim, 0], d, nv, label)[0]
        assert not pyoracle.agl_sumcheck_verify(msgs, fin, [claim + 1, 0], d, nv, label)[0]
        assert not pyoracle.agl_sumcheck_verify(msgs, fin, [claim, 0], d, nv, label + b"x")[0]


def test_random_tables_against_python_integers():
    nv, d = 5, 3
    n = 1 << nv
    raw = splitmix64(31, 2 * n * d)
    raw[:4] = [Q, Q - 1, 2**64 - 1, 0]  # non-canonical words are reduced on the way in
    msgs, ch, fe, fin, _ = pyoracle.agl_sumcheck_prove(raw, d, nv, False, b"rand")
    tabs = [[(int(raw[2 * (i * n + j)]) % Q, int(raw[2 * (i * n + j) + 1]) % Q) for j in range(n)] for i in range(d)]
    claim = [0, 0]
    for j in range(n):
        pr = (1, 0)
        for i in range(d):
            pr = _mul(pr, tabs[i][j])
        claim = [(claim[0] + pr[0]) % Q, (claim[1] + pr[1]) % Q]
    ok, _ = pyoracle.agl_sumcheck_verify(msgs, fin, claim, d, nv, b"rand")
    assert ok
    # round by round: message values and folds with Python integers
    for rnd in range(nv):
        half = len(tabs[0]) // 2
        for e in range(d + 1):
            s = [0, 0]
            for j in range(half):
                pr = (1, 0)
                for i in range(d):
                    a, b = tabs[i][2 * j], tabs[i][2 * j + 1]
                    pr = _mul(pr, ((a[0] + e * (b[0] - a[0])) % Q, (a[1] + e * (b[1] - a[1])) % Q))
                s = [(s[0] + pr[0]) % Q, (s[1] + pr[1]) % Q]
            k = (rnd * (d + 1) + e) * 2
            assert [int(msgs[k]), int(msgs[k + 1])] == s
        r = (int(ch[2 * rnd]) % Q, int(ch[2 * rnd + 1]) % Q)
        tabs = [[tuple((a[k] + _mul(r, ((b[0] - a[0]) % Q, (b[1] - a[1]) % Q))[k]) % Q for k in range(2))
                 for a, b in zip(t[0::2], t[1::2])] for t in tabs]
    assert [int(x) for x in fe] == [w for t in tabs for w in t[0]]
    pr = (1, 0)
    for t in tabs:
        pr = _mul(pr, t[0])
    assert [int(fin[0]), int(fin[1])] == list(pr)


def test_library_verifier_agrees_with_oracle_verifier():
    """agl_sumcheck_verify_ffi (SumcheckVerifier::verify, zk-torch-4/src/sumcheck/verifier.rs:14-113; host code of the
    CUDA library, no device call) on proofs written by the oracle prover: accepts them with the same challenges, and
    gives the oracle verifier's verdict on every tampered word, a wrong claim and a wrong label."""
    import ctypes
    from matrix_b200.ffi import load_agl
    lib = load_agl()

    def ours(msgs, fin, claim, d, nv, label):
        msgs, fin = np.ascontiguousarray(msgs, dtype=np.uint64), np.ascontiguousarray(fin, dtype=np.uint64)
        cl, ch = np.array(claim, dtype=np.uint64), np.zeros(max(nv, 1) * 2, dtype=np.uint64)
        h, ok = ctypes.c_void_p(), ctypes.c_int(-1)
        assert lib.agl_transcript_create(label, len(label), ctypes.byref(h)) == 0
        rc = lib.agl_sumcheck_verify_ffi(msgs.ctypes.data, fin.ctypes.data, cl.ctypes.data, d, nv, h, ch.ctypes.data, ctypes.byref(ok))
        lib.agl_transcript_destroy(h)
        assert rc == 0
        return bool(ok.value), ch[:2 * nv]

    cases = [(label, nv, lifted(tables), len(tables), [claim, 0]) for label, nv, tables, claim in CASES]
    for seed, (nv, d) in enumerate([(1, 1), (4, 2), (6, 3), (5, 4), (3, 6)]):
        n = 1 << nv
        raw = splitmix64(200 + seed, 2 * n * d) % np.uint64(Q)
        tabs = [[(int(raw[2 * (i * n + j)]), int(raw[2 * (i * n + j) + 1])) for j in range(n)] for i in range(d)]
        claim = [0, 0]
        for j in range(n):
            pr = (1, 0)
            for i in range(d):
                pr = _mul(pr, tabs[i][j])
            claim = [(claim[0] + pr[0]) % Q, (claim[1] + pr[1]) % Q]
        cases.append((b"lib-%d" % seed, nv, raw, d, claim))
    for label, nv, polys, d, claim in cases:
        msgs, ch, _, fin, _ = pyoracle.agl_sumcheck_prove(polys, d, nv, False, label)
        ok, vch = ours(msgs, fin, claim, d, nv, label)
        assert ok and list(vch) == list(ch)
        for pos in range(len(msgs)):
            bad = msgs.copy()
            bad[pos] ^= np.uint64(1)
            assert ours(bad, fin, claim, d, nv, label)[0] == pyoracle.agl_sumcheck_verify(bad, fin, claim, d, nv, label)[0] is False
        bad_fin = fin.copy()
        bad_fin[1] ^= np.uint64(1)
        assert not ours(msgs, bad_fin, claim, d, nv, label)[0]
        assert not ours(msgs, fin, [(claim[0] + 1) % Q, claim[1]], d, nv, label)[0]
        assert not ours(msgs, fin, claim, d, nv, label + b"x")[0]
