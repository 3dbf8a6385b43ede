"""GPU parity of the batched eq * a_k * b_k sumcheck: one shard, and several
shards simulated on one GPU, against the unsharded CPU oracle. Bit-exact."""
import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from matrix_b200.sharded import GpuShard, LibTranscript, SingleComm, prove_sharded
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
