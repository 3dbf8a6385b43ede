"""One process of the shared-memory exchange test: the sharded batched sumcheck with oracle shards (CPU only)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from matrix_b200 import load_gl  # noqa: E402
from matrix_b200.sharded import LibTranscript, ShmComm, prove_sharded  # noqa: E402
from oracle import pyoracle  # noqa: E402
from tests.sharded_helpers import OracleShard, assert_same_proof, inputs, shard_slices  # noqa: E402


def main():
    path, rank, world = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    comm = ShmComm(path, rank, world, timeout_s=60.0)
    # many small calls first: ordering and slot reuse
    for i in range(200):
        got = comm.allgather([np.array([rank, i, rank * 1000 + i], dtype=np.uint64)])
        assert [list(map(int, g)) for g in got] == [[g, i, g * 1000 + i] for g in range(world)]
    K, nv, g_bits = 3, 6, world.bit_length() - 1
    a, b, point = inputs(K, nv)
    lib = load_gl()
    oracle = pyoracle.load()

    def make_shard(g, point_low, scale):
        sa, sb = shard_slices(a, b, K, nv, g_bits, g)
        return OracleShard(oracle, sa, sb, point_low, scale, K, nv - g_bits)

    got = prove_sharded(make_shard, LibTranscript(lib, b"bench"), comm, point, K, nv, g_bits)
    exp = pyoracle.batched_prove(a, b, np.array([c for t in point for c in t], dtype=np.uint64), K, nv)
    assert_same_proof(got, exp)
    with open("%s.ok.%d" % (path, rank), "w") as f:
        f.write("ok")


if __name__ == "__main__":
    main()
