"""The oracle's same-point sumcheck (zk-torch-4/src/fold/same_point_sumcheck.rs) on the reference's own test
cases: the three deterministic instances of its unit tests (single instance with arity = N, :1709-1730; two
instances of different arity, :1732-1759; three instances that exercise the constant mode, :1761-1795) must prove,
verify to the same challenges, reveal the witness' multilinear extension at R[..arity], and a tampered reveal
must be rejected (:1879-1899). Random instances of every witness kind follow."""
import numpy as np
import pytest

from matrix_b200.inputs import AGL_Q, splitmix64
from oracle import pyoracle


def lift(v):
    return [v % AGL_Q, 0]


def binary_instance(words, arity, point):
    w = np.array(words, dtype=np.uint64)
    pt = np.array(point, dtype=np.uint64)
    return dict(arity=arity, kind=0, witness=w, point=pt, value=pyoracle.agl_witness_eval(0, w, arity, pt))


def check(instances, n, label):
    proof = pyoracle.agl_same_point_prove(instances, n, label)
    ok, ch = pyoracle.agl_same_point_verify(instances, n, proof, label)
    assert ok
    assert np.array_equal(ch, proof["challenges"])
    for i, inst in enumerate(instances):
        want = pyoracle.agl_witness_eval(inst["kind"], inst["witness"], inst["arity"], proof["challenges"][:inst["arity"]])
        assert np.array_equal(proof["f_evals"][i], want), "f_eval of instance %d" % i
    bad = {k: v.copy() for k, v in proof.items()}
    bad["f_evals"][0, 0] = (int(bad["f_evals"][0, 0]) + 1) % AGL_Q
    assert not pyoracle.agl_same_point_verify(instances, n, bad, label)[0]
    bad = {k: v.copy() for k, v in proof.items()}
    bad["round_msgs"][n - 1, 2, 1] ^= np.uint64(1)
    assert not pyoracle.agl_same_point_verify(instances, n, bad, label)[0]
    return proof


def test_single_instance_arity_equals_max():
    n = 4
    inst = binary_instance([0b10101100 ^ (0b11110000 << 8)], n, [lift(i * 7 + 3) for i in range(n)])
    check([inst], n, b"sp-single")


def test_two_instances_of_different_arity():
    inst0 = binary_instance([0b1011], 2, [lift(i * 5 + 1) for i in range(2)])
    inst1 = binary_instance([0b0101001111001010], 4, [lift(i * 11 + 2) for i in range(4)])
    check([inst0, inst1], 4, b"sp-two")


def test_three_instances_constant_mode_after_arity():
    inst0 = binary_instance([0b1010], 2, [lift(i + 1) for i in range(2)])
    inst1 = binary_instance([0b11110011], 3, [lift(i * 2 + 5) for i in range(3)])
    inst2 = binary_instance([0b01010101 | (0b1010 << 16)], 5, [lift(i * 3 + 9) for i in range(5)])
    check([inst0, inst1, inst2], 5, b"sp-three")


def random_instance(seed, kind, arity):
    n = 1 << arity
    words = max(1, n >> 6)
    pt = (splitmix64(seed, 2 * arity) % np.uint64(AGL_Q)).reshape(arity, 2)
    if kind == 0:
        w = splitmix64(seed + 1, words)
        if n < 64:
            w[0] &= np.uint64((1 << n) - 1)
    elif kind == 1:
        a, b = splitmix64(seed + 1, words), splitmix64(seed + 2, words)
        if n < 64:
            a[0] &= np.uint64((1 << n) - 1)
            b[0] &= np.uint64((1 << n) - 1)
        w = np.concatenate([a & ~b, b & ~a])     # disjoint masks
    else:
        w = splitmix64(seed + 1, n) % np.uint64(AGL_Q)
    return dict(arity=arity, kind=kind, witness=w, point=pt, value=pyoracle.agl_witness_eval(kind, w, arity, pt))


@pytest.mark.parametrize("kinds,arities,n", [((0, 0, 0), (7, 7, 7), 7), ((1, 1), (8, 8), 8), ((2, 2, 2, 2), (6, 6, 6, 6), 6),
                                               ((0, 1, 2), (3, 9, 6), 9), ((2,), (1,), 3), ((0, 2), (10, 10), 12)])
def test_random_instances_of_every_kind(kinds, arities, n):
    insts = [random_instance(40 + 10 * i, k, a) for i, (k, a) in enumerate(zip(kinds, arities))]
    check(insts, n, b"sp-random")


def test_claim_sum_identity():
    """The first message sums to sum_i alpha^i y_i 2^(N - k_i): checked through the verifier's first round, and
    the evaluation helper agrees with a direct multilinear evaluation on Python integers."""
    inst = random_instance(7, 2, 5)
    pt = [(int(a), int(b)) for a, b in inst["point"]]
    q, w = AGL_Q, 3

    def mul(x, y):
        return ((x[0] * y[0] + w * x[1] * y[1]) % q, (x[0] * y[1] + x[1] * y[0]) % q)

    acc = (0, 0)
    for j in range(32):
        e = (1, 0)
        for k in range(5):
            t = pt[k] if (j >> k) & 1 else ((1 - pt[k][0]) % q, (-pt[k][1]) % q)
            e = mul(e, t)
        f = int(inst["witness"][j])
        acc = ((acc[0] + e[0] * f) % q, (acc[1] + e[1] * f) % q)
    assert [int(x) for x in inst["value"]] == list(acc)


def _library_verify(lib, instances, n, proof, label):
    """agl_same_point_verify_ffi (host code of the CUDA library; no device call) on a proof in the oracle's layout."""
    import ctypes
    arity = np.array([i["arity"] for i in instances], dtype=np.int32)
    pts = np.concatenate([np.ascontiguousarray(i["point"], dtype=np.uint64).reshape(-1) for i in instances])
    vals = np.ascontiguousarray([i["value"] for i in instances], dtype=np.uint64).reshape(-1)
    msgs = np.ascontiguousarray(proof["round_msgs"], dtype=np.uint64)
    fe = np.ascontiguousarray(proof["f_evals"], dtype=np.uint64)
    fin = np.ascontiguousarray(proof["final_eval"], dtype=np.uint64)
    ch = np.zeros((n, 2), dtype=np.uint64)
    h, ok = ctypes.c_void_p(), ctypes.c_int(-1)
    assert lib.agl_transcript_create(label, len(label), ctypes.byref(h)) == 0
    rc = lib.agl_same_point_verify_ffi(len(instances), n, arity.ctypes.data, pts.ctypes.data, vals.ctypes.data, msgs.ctypes.data,
                                       fe.ctypes.data, fin.ctypes.data, h, ch.ctypes.data, ctypes.byref(ok))
    lib.agl_transcript_destroy(h)
    assert rc == 0
    return bool(ok.value), ch


@pytest.mark.parametrize("kinds,arities,n", [((0,), (4,), 4), ((0, 0), (2, 4), 4), ((0, 1, 2), (3, 9, 6), 9), ((2, 2), (5, 5), 7),
                                               ((1, 0, 2, 0), (6, 1, 6, 3), 6)])
def test_library_verifier_agrees_with_oracle_verifier(kinds, arities, n):
    """The library's host verifier (same_point_sumcheck.rs:161-219) against the oracle's on proofs written by the
    oracle prover, instances of different arities included (the case only the verifier has to handle): both accept,
    return the same challenges, and reject the same tampered proofs."""
    from matrix_b200.ffi import load_agl
    lib = load_agl()
    instances = [random_instance(900 + 10 * k, kind, a) for k, (kind, a) in enumerate(zip(kinds, arities))]
    label = b"sp-lib"
    proof = pyoracle.agl_same_point_prove(instances, n, label)
    ok, ch = _library_verify(lib, instances, n, proof, label)
    ok_o, ch_o = pyoracle.agl_same_point_verify(instances, n, proof, label)
    assert ok and ok_o and np.array_equal(ch, ch_o) and np.array_equal(ch, proof["challenges"])
    rng = np.random.default_rng(n)
    for key in ("round_msgs", "f_evals", "final_eval"):
        flat = proof[key].reshape(-1)
        for pos in sorted(set(int(x) for x in rng.integers(0, len(flat), 12))):
            bad = {k: v.copy() for k, v in proof.items()}
            bad[key].reshape(-1)[pos] ^= np.uint64(1)
            got = _library_verify(lib, instances, n, bad, label)[0]
            assert got == pyoracle.agl_same_point_verify(instances, n, bad, label)[0], "%s word %d" % (key, pos)
            assert not got
    # a wrong claim and a wrong label
    wrong = [dict(i) for i in instances]
    wrong[0]["value"] = np.array([(int(wrong[0]["value"][0]) + 1) % AGL_Q, int(wrong[0]["value"][1])], dtype=np.uint64)
    assert not _library_verify(lib, wrong, n, proof, label)[0]
    assert not _library_verify(lib, instances, n, proof, b"other")[0]
