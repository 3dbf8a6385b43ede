"""CPU tests of the Goldilocks oracle: field arithmetic against Python integers,
Poseidon2 against the vector produced by the reference's own code, and the
sumcheck prover against the tiny cases of the reference's tests."""
import ctypes
import json
import os
import random

import numpy as np
import pytest

from .conftest import GL_P, ROOT, field_elems

P = GL_P
GOLDEN = os.path.join(ROOT, "tests", "golden")


def test_field_ops_match_python_ints(oracle):
    rnd = random.Random(1)
    edge = [0, 1, 2, P - 1, P - 2, 2**32, 2**32 - 1, 2**63, P // 2]
    vals = edge + [rnd.randrange(P) for _ in range(2000)]
    for a in vals[:60]:
        assert oracle.gl_inv(a) == (pow(a, P - 2, P))
    for _ in range(3000):
        a, e = rnd.choice(vals), rnd.randrange(1, 50)
        assert oracle.gl_pow(a, e) == pow(a, e, P)


def test_poseidon2_matches_reference_code_vector(oracle):
    # tests/golden/gl_poseidon2.json holds outputs of the reference's own
    # poseidon2_permute_8 (cuda/poseidon2.cuh:322-358) compiled host-side.
    vec = json.load(open(os.path.join(GOLDEN, "gl_poseidon2.json")))
    for case in vec["permute"]:
        s = (ctypes.c_uint64 * 8)(*case["in"])
        oracle.gl_poseidon2_permute(s)
        assert list(s) == case["out"]


def _py_round_message(polys, d, n):
    half = n // 2
    out = []
    for c in range(d + 1):
        acc = 0
        for y in range(half):
            prod = 1
            for i in range(d):
                a, b = int(polys[i * n + 2 * y]), int(polys[i * n + 2 * y + 1])
                prod = prod * ((a + c * (b - a)) % P) % P
            acc = (acc + prod) % P
        out.append(acc)
    return out


def test_base_round_and_fold_match_python(oracle):
    # The deterministic inputs of the reference's test_gpu_sumcheck_vs_cpu_large
    # (goldilocks-cuda-rs/src/sumcheck_prover.rs:527-556), at 6 variables.
    nv, d = 6, 3
    n = 1 << nv
    polys = np.array([(i * m + k) % P for (m, k) in ((37, 1), (53, 7), (71, 13)) for i in range(n)], dtype=np.uint64)
    cur = polys.copy()
    size = n
    for rnd_i in range(nv):
        half = size // 2
        msg = np.zeros(d + 1, dtype=np.uint64)
        oracle.oracle_gl_round_message(cur.ctypes.data, d, n, half, msg.ctypes.data)
        live = np.concatenate([cur[i * n:i * n + size] for i in range(d)])
        assert list(map(int, msg)) == _py_round_message(live, d, size)
        r = rnd_i * 11 + 5
        nxt = np.zeros_like(cur)
        oracle.oracle_gl_fold(cur.ctypes.data, nxt.ctypes.data, r, d, n, half)
        for i in range(d):
            for y in range(half):
                a, b = int(cur[i * n + 2 * y]), int(cur[i * n + 2 * y + 1])
                assert int(nxt[i * n + y]) == (a + r * (b - a)) % P
        cur, size = nxt, half


def test_sumcheck_tiny_claim_and_verifier(oracle):
    # Tables 1..4 and 5..8 (zk-torch-3/src/sumcheck/cpu_ext2_prover.rs:120-140):
    # sum of products = 5 + 12 + 21 + 32 = 70.
    from oracle import pyoracle
    polys = np.array([1, 2, 3, 4, 5, 6, 7, 8], dtype=np.uint64)
    res = pyoracle.sumcheck_prove(polys, 2, 2, True, b"test")
    m0 = res["round_msgs"][0]
    assert (int(m0[0][0]) + int(m0[1][0])) % P == 70 and int(m0[0][1]) == 0 and int(m0[1][1]) == 0
    claim = np.array([70, 0], dtype=np.uint64)
    rc = oracle.oracle_gl_sumcheck_verify(2, 2, b"test", 4, claim.ctypes.data, res["round_msgs"].ctypes.data,
                                          res["final_eval"].ctypes.data)
    assert rc == 0
    bad = res["round_msgs"].copy()
    bad[1, 2, 0] ^= np.uint64(1)
    rc = oracle.oracle_gl_sumcheck_verify(2, 2, b"test", 4, claim.ctypes.data, bad.ctypes.data,
                                          res["final_eval"].ctypes.data)
    assert rc != 0


def test_sumcheck_random_prover_verifier_roundtrip(oracle):
    from oracle import pyoracle
    for nv, d, base in ((1, 1, True), (3, 2, True), (5, 3, False), (7, 2, False), (4, 4, True)):
        n = 1 << nv
        polys = field_elems(100 + nv, n * d * (1 if base else 2))
        res = pyoracle.sumcheck_prove(polys, d, nv, base, b"bench")
        m0 = res["round_msgs"][0]
        claim = np.array([(int(m0[0][0]) + int(m0[1][0])) % P, (int(m0[0][1]) + int(m0[1][1])) % P], dtype=np.uint64)
        rc = oracle.oracle_gl_sumcheck_verify(d, nv, b"bench", 5, claim.ctypes.data, res["round_msgs"].ctypes.data,
                                              res["final_eval"].ctypes.data)
        assert rc == 0


def test_library_sumcheck_verifier_agrees_with_oracle_verifier(oracle):
    """gl_sumcheck_verify_ffi (host code of the CUDA library, no device call; zk-torch-3/src/sumcheck/verifier.rs) on
    proofs written by the oracle prover: accepts them with the prover's challenges, and gives the oracle verifier's
    verdict on every flipped word of the messages, a wrong final value, a wrong claim and a wrong label."""
    import ctypes
    from matrix_b200.ffi import load_gl
    from oracle import pyoracle
    lib = load_gl()

    def ours(msgs, fin, claim, d, nv, label):
        msgs = np.ascontiguousarray(msgs, dtype=np.uint64)
        ch, ok = np.zeros((max(nv, 1), 2), dtype=np.uint64), ctypes.c_int(-1)
        assert lib.gl_sumcheck_verify_ffi(msgs.ctypes.data, fin.ctypes.data, claim.ctypes.data, d, nv, label, len(label),
                                          ch.ctypes.data, ctypes.byref(ok)) == 0
        return bool(ok.value), ch[:nv]

    def theirs(msgs, fin, claim, d, nv, label):
        msgs = np.ascontiguousarray(msgs, dtype=np.uint64)
        return oracle.oracle_gl_sumcheck_verify(d, nv, label, len(label), claim.ctypes.data, msgs.ctypes.data, fin.ctypes.data) == 0

    cases = [(2, 2, True, np.array([1, 2, 3, 4, 5, 6, 7, 8], dtype=np.uint64), b"test")]
    for nv, d, base in ((1, 1, True), (3, 2, True), (5, 3, False), (6, 2, False), (4, 4, True), (3, 6, False)):
        cases.append((nv, d, base, field_elems(300 + nv, (1 << nv) * d * (1 if base else 2)), b"bench"))
    for nv, d, base, polys, label in cases:
        res = pyoracle.sumcheck_prove(polys, d, nv, base, label)
        msgs, fin = res["round_msgs"], res["final_eval"]
        m0 = msgs[0]
        claim = np.array([(int(m0[0][0]) + int(m0[1][0])) % P, (int(m0[0][1]) + int(m0[1][1])) % P], dtype=np.uint64)
        ok, ch = ours(msgs, fin, claim, d, nv, label)
        assert ok and theirs(msgs, fin, claim, d, nv, label) and np.array_equal(ch, res["challenges"])
        flat_len = msgs.size
        for pos in range(flat_len):
            bad = msgs.copy()
            bad.reshape(-1)[pos] ^= np.uint64(1)
            assert ours(bad, fin, claim, d, nv, label)[0] == theirs(bad, fin, claim, d, nv, label) is False, "word %d" % pos
        bad_fin = fin.copy()
        bad_fin[0] ^= np.uint64(1)
        assert not ours(msgs, bad_fin, claim, d, nv, label)[0] and not theirs(msgs, bad_fin, claim, d, nv, label)
        bad_claim = claim.copy()
        bad_claim[1] ^= np.uint64(1)
        assert not ours(msgs, fin, bad_claim, d, nv, label)[0]
        assert not ours(msgs, fin, claim, d, nv, label + b"x")[0]


@pytest.mark.parametrize("K,nv", [(1, 1), (1, 4), (3, 5), (16, 6), (5, 9)])
def test_library_batched_verifier_accepts_oracle_proofs_and_rejects_tampering(K, nv):
    """gl_batched_verify_host (host code of the CUDA library, no device call) on the batched eq * a * b proofs the
    oracle prover writes: the round sums chain from sum_k alpha^k y_k down to eq(R) sum_k alpha^k a_k(R) b_k(R), the
    revealed eq(R) is the eq polynomial of the point at the challenges, the challenges are the prover's, and the
    claims are the sums over the cube computed with Python integers. Every flipped word of the claims, the messages
    and the reveals, a wrong point and a wrong label are rejected."""
    import ctypes
    from matrix_b200.ffi import load_gl
    from oracle import pyoracle
    lib = load_gl()
    n = 1 << nv
    a, b = field_elems(400 + K, K * n), field_elems(500 + nv, K * n)
    point = field_elems(600 + K + nv, 2 * nv)
    res = pyoracle.batched_prove(a, b, point, K, nv, b"cfg4")

    def verify(claims, msgs, finals, pt=point, label=b"cfg4"):
        claims, msgs, finals = (np.ascontiguousarray(x, dtype=np.uint64) for x in (claims, msgs, finals))
        ch, ok = np.zeros((nv, 2), dtype=np.uint64), ctypes.c_int(-1)
        assert lib.gl_batched_verify_host(K, nv, pt.ctypes.data, label, len(label), claims.ctypes.data, msgs.ctypes.data,
                                          finals.ctypes.data, ch.ctypes.data, ctypes.byref(ok)) == 0
        return bool(ok.value), ch

    ok, ch = verify(res["claims"], res["round_msgs"], res["finals"])
    assert ok and np.array_equal(ch, res["challenges"])
    # the claims are what they say: y_k = sum_x eq(point, x) a_k(x) b_k(x), here for a small case with Python integers
    if nv <= 5:
        def mul(x, y):
            return ((x[0] * y[0] + 7 * x[1] * y[1]) % P, (x[0] * y[1] + x[1] * y[0]) % P)
        pt = [(int(point[2 * i]), int(point[2 * i + 1])) for i in range(nv)]
        for k in range(K):
            y = (0, 0)
            for x in range(n):
                e = (1, 0)
                for i in range(nv):
                    e = mul(e, pt[i] if (x >> i) & 1 else ((1 - pt[i][0]) % P, (-pt[i][1]) % P))
                t = mul(e, (int(a[k * n + x]) * int(b[k * n + x]) % P, 0))
                y = ((y[0] + t[0]) % P, (y[1] + t[1]) % P)
            assert (int(res["claims"][k][0]), int(res["claims"][k][1])) == y
    rng = np.random.default_rng(K * 100 + nv)
    for key in ("claims", "round_msgs", "finals"):
        size = res[key].size
        positions = range(size) if size <= 64 else sorted(set(int(x) for x in rng.integers(0, size, 48)) | {0, size - 1})
        for pos in positions:
            parts = {k: res[k].copy() for k in ("claims", "round_msgs", "finals")}
            parts[key].reshape(-1)[pos] ^= np.uint64(1)
            assert not verify(parts["claims"], parts["round_msgs"], parts["finals"])[0], "%s word %d accepted" % (key, pos)
    bad_point = point.copy()
    bad_point[2 * (nv - 1)] ^= np.uint64(1)
    assert not verify(res["claims"], res["round_msgs"], res["finals"], pt=bad_point)[0]
    assert not verify(res["claims"], res["round_msgs"], res["finals"], label=b"cfg5")[0]
