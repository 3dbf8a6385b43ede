"""The library's own Basefold verifier (basefold_verify_host; the reference's BasefoldProver::verify_ext2,
goldilocks-cuda-rs/src/basefold.rs:1759-1925 with the query checks of :2222-2402) against the CPU oracle's
restatement of the same verifier: both must accept the proofs the GPU prover writes, and on tampered proofs both
must stop at the same check (the same negative code)."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import load_gl
from .conftest import field_elems

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    return lib


def _prove(lib, nv, lr, nq, hash_id=0, label=b"bench"):
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    h = ctypes.c_void_p()
    assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
    proof = np.zeros(lib.basefold_proof_words(nv, lr, nq), dtype=np.uint64)
    root = np.zeros(4, dtype=np.uint64)
    assert lib.basefold_set_merkle_hash(hash_id) == 0
    try:
        assert lib.basefold_prove_host(evals.ctypes.data, nv, lr, point.ctypes.data, h, label, len(label), nq,
                                       root.ctypes.data, proof.ctypes.data) == 0
    finally:
        assert lib.basefold_set_merkle_hash(0) == 0
    return h, point, root, proof


def _verify(lib, h, nv, lr, nq, point, root, proof, hash_id=0, label=b"bench"):
    res = ctypes.c_int(12345)
    rc = lib.basefold_verify_host(root.ctypes.data, nv, lr, point.ctypes.data, h, label, len(label), nq, hash_id,
                                  proof.ctypes.data, ctypes.byref(res))
    assert rc == 0, "basefold_verify_host: %d" % rc
    return res.value


@pytest.mark.parametrize("nv,lr,nq", [(2, 1, 2), (2, 0, 1), (3, 1, 4), (4, 3, 5), (7, 1, 9), (10, 2, 16),
                                      (13, 1, 34), (16, 1, 100)])
def test_accepts_gpu_proofs_and_agrees_with_oracle_on_tampering(lib, nv, lr, nq):
    from oracle import pyoracle
    h, point, root, proof = _prove(lib, nv, lr, nq)
    table = pyoracle.bf_table(nv, lr)
    assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) == 0
    assert _verify(lib, h, nv, lr, nq, point, root, proof) == 0
    # every word for the small proofs, a seeded sample of 200 otherwise (first, last and the section borders always)
    words = len(proof)
    if words <= 400:
        positions = list(range(words))
    else:
        rng = np.random.default_rng(nv * 100 + lr)
        borders = [0, 1, 2, 2 + 6 * nv - 1, 2 + 6 * nv, 2 + 6 * nv + 4 * (nv - 1) - 1, 2 + 6 * nv + 4 * (nv - 1),
                   words - 1]
        positions = sorted(set(borders) | set(int(x) for x in rng.integers(0, words, 200)))
    for pos in positions:
        bad = proof.copy()
        bad[pos] ^= np.uint64(1)
        want = pyoracle.bf_verify(root, nv, lr, point, table, nq, bad)
        got = _verify(lib, h, nv, lr, nq, point, root, bad)
        assert got == want, "word %d flipped: library %d, oracle %d" % (pos, got, want)
        # a final-codeword element is only looked at by the queries that fold onto it
        in_final = 2 + 6 * nv + 4 * (nv - 1) <= pos < 2 + 6 * nv + 4 * (nv - 1) + (2 << lr)
        assert got != 0 or in_final, "tampered word %d accepted" % pos
    # wrong root, wrong point, wrong label
    bad_root = root.copy()
    bad_root[3] ^= np.uint64(1)
    assert _verify(lib, h, nv, lr, nq, point, bad_root, proof) == pyoracle.bf_verify(bad_root, nv, lr, point, table, nq, proof) != 0
    bad_point = point.copy()
    bad_point[0] ^= np.uint64(1)
    # the point enters through the transcript only: the oracle chain breaks at the first challenge
    assert _verify(lib, h, nv, lr, nq, bad_point, root, proof) == pyoracle.bf_verify(root, nv, lr, bad_point, table, nq, proof) != 0
    assert _verify(lib, h, nv, lr, nq, point, root, proof, label=b"other") == \
        pyoracle.bf_verify(root, nv, lr, point, table, nq, proof, label=b"other") != 0
    lib.basefold_table_destroy(h)


@pytest.mark.parametrize("nv,lr,nq", [(3, 0, 3), (10, 3, 34), (14, 1, 100)])
def test_monolith_proofs(lib, nv, lr, nq):
    from oracle import pyoracle
    h, point, root, proof = _prove(lib, nv, lr, nq, hash_id=1)
    assert _verify(lib, h, nv, lr, nq, point, root, proof, hash_id=1) == 0
    assert _verify(lib, h, nv, lr, nq, point, root, proof, hash_id=0) == -101    # not a Poseidon2 tree
    # negative = the library's current setting
    assert _verify(lib, h, nv, lr, nq, point, root, proof, hash_id=-1) == -101
    assert lib.basefold_set_merkle_hash(1) == 0
    try:
        assert _verify(lib, h, nv, lr, nq, point, root, proof, hash_id=-1) == 0
    finally:
        assert lib.basefold_set_merkle_hash(0) == 0
    table = pyoracle.bf_table(nv, lr)
    with pyoracle.merkle_hash(1):
        assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) == 0
    lib.basefold_table_destroy(h)


def test_no_queries_and_bad_arguments(lib):
    nv, lr = 6, 1
    h, point, root, proof = _prove(lib, nv, lr, 0)
    assert _verify(lib, h, nv, lr, 0, point, root, proof) == 0
    bad = proof.copy()
    bad[0] ^= np.uint64(1)
    assert _verify(lib, h, nv, lr, 0, point, root, bad) == -1
    res = ctypes.c_int(0)
    # a table of another shape, a null proof
    assert lib.basefold_verify_host(root.ctypes.data, nv + 1, lr, point.ctypes.data, h, b"bench", 5, 0, 0,
                                    proof.ctypes.data, ctypes.byref(res)) != 0
    assert lib.basefold_verify_host(root.ctypes.data, nv, lr, point.ctypes.data, h, b"bench", 5, 0, 0, None,
                                    ctypes.byref(res)) != 0
    lib.basefold_table_destroy(h)


def test_full_size_proof_2_24(lib):
    """The benchmarked configuration (2^24 evaluations, rate 1/2, 100 queries): the proof verifies, and a flipped
    word in each section of it is caught at that section's check."""
    nv, lr, nq = 24, 1, 100
    h, point, root, proof = _prove(lib, nv, lr, nq)
    assert _verify(lib, h, nv, lr, nq, point, root, proof) == 0
    words = len(proof)
    qw = (words - (2 + 6 * nv + 4 * (nv - 1) + (2 << lr))) // nq
    q0 = words - nq * qw
    cases = [(0, -1), (2, -1), (2 + 6 * 3, -12), (2 + 6 * nv, -11), (q0 - 1, -400), (q0, -100), (q0 + 1, -101),
             (q0 + 1 + 4 * nv, -101), (words - 1, -(300 + nv - 2))]
    for pos, code in cases:
        bad = proof.copy()
        bad[pos] ^= np.uint64(1)
        got = _verify(lib, h, nv, lr, nq, point, root, bad)
        assert got != 0, "tampered word %d accepted" % pos
        assert got == code, "word %d: code %d, expected %d" % (pos, got, code)
    lib.basefold_table_destroy(h)
