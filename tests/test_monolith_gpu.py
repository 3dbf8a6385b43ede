"""GPU parity of the Monolith path: the permutation, Monolith Merkle trees and the Basefold
commit + opening with Monolith trees, against the CPU oracle, through the C-ABI. Bit-exact."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from oracle import pyoracle
from .conftest import GL_P, field_elems, splitmix64
from .test_monolith import GL_KAT

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    assert lib.monolith_cuda_init() == 0
    return lib


def test_permute_known_answer_on_device(lib):
    # goldilocks-cuda-rs/src/cpu_monolith.rs:237-254 through the reference's own test entry point
    inp, out = np.arange(12, dtype=np.uint64), np.zeros(12, dtype=np.uint64)
    assert lib.monolith_permute_test_ffi(inp.ctypes.data, out.ctypes.data) == 0
    assert [int(x) for x in out] == GL_KAT
    # the large-value case of cpu_monolith.rs:257-277
    inp = np.array([8, GL_P - 8] + [0] * 10, dtype=np.uint64)
    assert lib.monolith_permute_test_ffi(inp.ctypes.data, out.ctypes.data) == 0
    exp = inp.copy()
    pyoracle.load().oracle_gl_monolith_permute(exp.ctypes.data)
    assert np.array_equal(out, exp)


def test_permute_batch_matches_oracle(lib, oracle):
    n = 3000
    states = splitmix64(31, 12 * n)  # raw 64-bit words: non-canonical inputs included
    states[:12] = 2**64 - 1
    states[12:24] = GL_P - 1
    d_in = DeviceBuffer.from_numpy(lib, states)
    d_out = DeviceBuffer(lib, states.nbytes)
    assert lib.monolith_permute_batch_ffi(d_in.ptr, d_out.ptr, n) == 0
    got = d_out.to_numpy().reshape(n, 12)
    for i in list(range(64)) + list(range(n - 64, n)) + list(range(64, n - 64, 37)):
        s = states[12 * i:12 * i + 12].copy()
        oracle.oracle_gl_monolith_permute(s.ctypes.data)
        assert np.array_equal(got[i], s), i
    assert (got < GL_P).all()
    assert lib.monolith_permute_batch_ffi(d_in.ptr, d_out.ptr, 0) == 0
    assert lib.monolith_permute_batch_ffi(None, d_out.ptr, 4) != 0


@pytest.mark.parametrize("leaves,ext2", [(1, False), (2, True), (8, False), (64, True), (128, False), (2048, False),
                                         (4096, True), (1 << 15, False)])
def test_merkle_tree_matches_oracle(lib, oracle, leaves, ext2):
    words = leaves * (4 if ext2 else 2)
    cw = field_elems(810 + leaves, words)
    d_cw = DeviceBuffer.from_numpy(lib, cw)
    d_t = DeviceBuffer(lib, 32 * (2 * leaves - 1))
    fn = lib.monolith_merkle_tree_ext2_ffi if ext2 else lib.monolith_merkle_tree_gl_ffi
    assert fn(d_cw.ptr, d_t.ptr, leaves) == 0
    exp = np.zeros(4 * (2 * leaves - 1), dtype=np.uint64)
    with pyoracle.merkle_hash(1):
        oracle.oracle_bf_merkle_tree(cw.ctypes.data, leaves, 1 if ext2 else 0, exp.ctypes.data)
    assert np.array_equal(d_t.to_numpy(), exp)
    # and it differs from the Poseidon2 tree over the same codeword
    oracle.oracle_bf_merkle_tree(cw.ctypes.data, leaves, 1 if ext2 else 0, exp.ctypes.data)
    assert not np.array_equal(d_t.to_numpy(), exp)
    assert fn(d_cw.ptr, d_t.ptr, 3) != 0 and fn(d_cw.ptr, d_t.ptr, 0) != 0


def test_merkle_leaves_of_reference_specific_input(lib, oracle):
    """The codeword of test_monolith_gpu_vs_cpu_specific_input (goldilocks-cuda-rs/src/cpu_monolith.rs:364-393):
    words just below the modulus."""
    cw = np.array([1, 2, 8, 18446744069414584313, 12, 18446744069414584317, 7, 8], dtype=np.uint64)
    d_cw = DeviceBuffer.from_numpy(lib, cw)
    d_t = DeviceBuffer(lib, 32 * 7)
    assert lib.monolith_merkle_tree_gl_ffi(d_cw.ptr, d_t.ptr, 4) == 0
    exp = np.zeros(4 * 7, dtype=np.uint64)
    with pyoracle.merkle_hash(1):
        oracle.oracle_bf_merkle_tree(cw.ctypes.data, 4, 0, exp.ctypes.data)
    assert np.array_equal(d_t.to_numpy(), exp)


@pytest.mark.parametrize("nv,lr,nq", [(2, 1, 2), (3, 0, 3), (7, 1, 9), (10, 3, 34), (13, 1, 34), (16, 1, 100)])
def test_commit_open_with_monolith_trees(lib, nv, lr, nq):
    """The reference's default build hashes Merkle trees with Monolith and keeps the Poseidon2
    transcript (zk-torch-3/Cargo.toml:22-23, zk-torch-3/src/commit/cpu_basefold.rs:6-9)."""
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    with pyoracle.merkle_hash(1):
        cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
        exp, exp_state = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)
    h = ctypes.c_void_p()
    assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
    words = lib.basefold_proof_words(nv, lr, nq)
    proof, root, st = np.zeros(words, dtype=np.uint64), np.zeros(4, dtype=np.uint64), np.zeros(8, dtype=np.uint64)
    c = ctypes.c_void_p()
    assert lib.basefold_set_merkle_hash(2) != 0
    assert lib.basefold_set_merkle_hash(1) == 0
    try:
        assert lib.basefold_commit_host(evals.ctypes.data, nv, lr, ctypes.byref(c), root.ctypes.data) == 0
    finally:
        assert lib.basefold_set_merkle_hash(0) == 0
    # the commitment remembers its hash: the opening below runs with the library back on Poseidon2
    assert lib.basefold_open_ext2(c, point.ctypes.data, h, b"bench", 5, nq, proof.ctypes.data, st.ctypes.data) == 0
    assert np.array_equal(root, tree[-4:])
    bad = np.nonzero(proof != exp)[0]
    assert len(bad) == 0, "first differing proof word: %d of %d" % (bad[0], words)
    assert np.array_equal(st, exp_state)
    with pyoracle.merkle_hash(1):
        assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) == 0
    assert pyoracle.bf_verify(root, nv, lr, point, table, nq, proof) != 0  # not a Poseidon2 proof
    lib.basefold_commitment_destroy(c)
    lib.basefold_table_destroy(h)
