"""GPU parity of the batched eq * a_k * b_k sumcheck: one shard, and several
shards simulated on one GPU, against the unsharded CPU oracle. Bit-exact. Both
drivers are covered: the per-round C-ABI under the Python loop, and the whole
proof inside the library with the ranks as host threads on one GPU."""
import ctypes
import threading

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from matrix_b200.sharded import GpuShard, LibTranscript, SingleComm, prove_batched_native, prove_sharded
from .sharded_helpers import assert_same_proof, inputs, shard_slices

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K,nv,g_bits", [(1, 1, 0), (1, 2, 0), (2, 3, 0), (3, 6, 0), (16, 10, 0), (5, 14, 0),
                                         (2, 5, 1), (3, 9, 2), (16, 12, 3), (4, 4, 3),
                                         (33, 8, 0), (64, 7, 1), (8, 17, 0), (1, 15, 0), (16, 18, 1)])
def test_batched_sumcheck_matches_oracle(K, nv, g_bits):
    from oracle import pyoracle
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    a, b, point = inputs(K, nv)
    keep = []

    def make_shard(g, point_low, scale):
        sa, sb = shard_slices(a, b, K, nv, g_bits, g)
        d_a, d_b = DeviceBuffer.from_numpy(lib, sa), DeviceBuffer.from_numpy(lib, sb)
        keep.extend([d_a, d_b])
        return GpuShard(lib, d_a.ptr, d_b.ptr, point_low, scale, K, nv - g_bits)

    got = prove_sharded(make_shard, LibTranscript(lib, b"bench"), SingleComm(1 << g_bits), point, K, nv, g_bits)
    exp = pyoracle.batched_prove(a, b, np.array([c for t in point for c in t], dtype=np.uint64), K, nv)
    assert_same_proof(got, exp)


@pytest.mark.parametrize("K,nv,g_bits", [(1, 1, 0), (2, 3, 0), (16, 10, 0), (5, 14, 0), (33, 8, 0),
                                         (2, 5, 1), (3, 9, 2), (16, 12, 3), (4, 4, 3), (64, 7, 1), (16, 18, 1), (8, 16, 2)])
def test_whole_proof_inside_the_library(K, nv, g_bits):
    from oracle import pyoracle
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    a, b, point = inputs(K, nv)
    world = 1 << g_bits
    exs = (ctypes.c_void_p * world)()
    assert lib.mb_exchange_local_create(world, exs) == 0
    bufs = []
    for g in range(world):
        sa, sb = shard_slices(a, b, K, nv, g_bits, g)
        bufs.append((DeviceBuffer.from_numpy(lib, sa), DeviceBuffer.from_numpy(lib, sb)))
    got, errs = [None] * world, [None] * world

    def run(g):
        try:
            got[g] = prove_batched_native(lib, exs[g], bufs[g][0].ptr, bufs[g][1].ptr, K, nv, point, b"bench")
        except Exception as exc:
            errs[g] = exc

    threads = [threading.Thread(target=run, args=(g,)) for g in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for g in range(world):
        lib.mb_exchange_destroy(exs[g])
    assert errs == [None] * world
    exp = pyoracle.batched_prove(a, b, np.array([c for t in point for c in t], dtype=np.uint64), K, nv)
    for g in range(world):
        assert_same_proof(got[g], exp)
    # and the library's own verifier of the protocol accepts what the ranks wrote
    pt = np.array([c for t in point for c in t], dtype=np.uint64)
    ch, ok = np.zeros((nv, 2), dtype=np.uint64), ctypes.c_int(-1)
    assert lib.gl_batched_verify_host(K, nv, pt.ctypes.data, b"bench", 5, got[0]["claims"].ctypes.data,
                                      got[0]["round_msgs"].ctypes.data, got[0]["finals"].ctypes.data, ch.ctypes.data,
                                      ctypes.byref(ok)) == 0
    assert ok.value == 1 and np.array_equal(ch, got[0]["challenges"])


def test_whole_proof_refuses_a_world_larger_than_the_hypercube():
    lib = load_gl()
    a, b, point = inputs(1, 2)
    exs = (ctypes.c_void_p * 4)()
    assert lib.mb_exchange_local_create(4, exs) == 0
    d_a, d_b = DeviceBuffer.from_numpy(lib, a), DeviceBuffer.from_numpy(lib, b)
    with pytest.raises(RuntimeError, match="-3"):
        prove_batched_native(lib, exs[0], d_a.ptr, d_b.ptr, 1, 2, point, b"bench")   # n_loc = 0: refused before any exchange
    for g in range(4):
        lib.mb_exchange_destroy(exs[g])
