"""One Basefold commitment + opening partitioned over several ranks, bit for bit against the single-GPU proof.

The ranks here are host threads of this process on one GPU (the library's "local" exchange: host words under a
barrier, device pieces by device-to-device copies), which runs every line of the sharded host loop and all of
its kernels; tests/test_multigpu.py runs the same entry point with one process per GPU over NCCL.
"""
import ctypes
import threading

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


def _single(lib, evals, point, nv, lr, nq, h):
    words = lib.basefold_proof_words(nv, lr, nq)
    proof, root = np.zeros(words, dtype=np.uint64), np.zeros(4, dtype=np.uint64)
    assert lib.basefold_prove_host(evals.ctypes.data, nv, lr, point.ctypes.data, h, b"bench", 5, nq, root.ctypes.data,
                                   proof.ctypes.data) == 0
    return root, proof


def prove_with_threads(lib, evals, point, nv, lr, nq, h, world):
    """Runs `world` ranks as threads; returns the (root, proof) pair of every rank."""
    words = lib.basefold_proof_words(nv, lr, nq)
    exs = (ctypes.c_void_p * world)()
    assert lib.mb_exchange_local_create(world, exs) == 0
    n_loc = (1 << nv) // world
    shards = [np.ascontiguousarray(evals[r * n_loc:(r + 1) * n_loc]) for r in range(world)]
    roots = [np.zeros(4, dtype=np.uint64) for _ in range(world)]
    proofs = [np.zeros(words, dtype=np.uint64) for _ in range(world)]
    rcs = [None] * world

    def run(r):
        rcs[r] = lib.basefold_prove_sharded_host(shards[r].ctypes.data, nv, lr, point.ctypes.data, h, b"bench", 5, nq, exs[r],
                                                 roots[r].ctypes.data, proofs[r].ctypes.data)

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for r in range(world):
        lib.mb_exchange_destroy(exs[r])
    return rcs, roots, proofs


@pytest.mark.parametrize("nv,lr,nq,world", [(4, 1, 3, 2), (6, 0, 4, 4), (7, 2, 5, 8), (10, 1, 5, 2), (12, 1, 9, 2), (12, 1, 9, 4), (13, 2, 16, 4), (14, 1, 34, 8),
                                            (13, 0, 7, 2), (14, 0, 7, 4), (16, 3, 20, 8), (18, 1, 100, 8), (20, 1, 100, 4)])
def test_sharded_proof_equals_single_gpu_proof(lib, nv, lr, nq, world):
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    h = ctypes.c_void_p()
    assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
    root, proof = _single(lib, evals, point, nv, lr, nq, h)
    rcs, roots, proofs = prove_with_threads(lib, evals, point, nv, lr, nq, h, world)
    assert rcs == [0] * world
    for r in range(world):
        assert np.array_equal(roots[r], root), "root on rank %d" % r
        bad = np.nonzero(proofs[r] != proof)[0]
        assert len(bad) == 0, "rank %d: first differing proof word %d of %d" % (r, bad[0], len(proof))
    lib.basefold_table_destroy(h)


def test_sharded_proof_verifies_under_the_oracle(lib):
    from oracle import pyoracle
    nv, lr, nq, world = 15, 1, 40, 4
    evals = field_elems(3, 1 << nv)
    point = field_elems(4, 2 * nv)
    h = ctypes.c_void_p()
    assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
    rcs, roots, proofs = prove_with_threads(lib, evals, point, nv, lr, nq, h, world)
    assert rcs == [0] * world
    table = pyoracle.bf_table(nv, lr)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    exp, _ = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)
    assert np.array_equal(roots[0], tree[-4:]) and np.array_equal(proofs[0], exp)
    assert pyoracle.bf_verify(roots[0], nv, lr, point, table, nq, proofs[0]) == 0
    lib.basefold_table_destroy(h)


def test_unsupported_shapes_are_refused(lib):
    nv, lr = 4, 1
    evals, point = field_elems(3, 1 << nv), field_elems(4, 2 * nv)
    h = ctypes.c_void_p()
    assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
    rcs, _, _ = prove_with_threads(lib, evals, point, nv, lr, 2, h, 4)     # too few variables for four ranks
    assert rcs == [-3] * 4
    lib.basefold_table_destroy(h)
    nv, lr = 12, 2
    evals, point = field_elems(3, 1 << nv), field_elems(4, 2 * nv)
    assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
    rcs, _, _ = prove_with_threads(lib, evals, point, nv, lr, 2, h, 2)     # fewer ranks than codeword blocks
    assert rcs == [-3, -3]
    lib.basefold_table_destroy(h)
