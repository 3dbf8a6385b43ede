"""One rank of the world-size-2 CPU test (gloo): the orchestration of
matrix_b200.sharded with oracle-computed shards. Started by test_sharded_cpu.py."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch.distributed as dist  # noqa: E402

from matrix_b200 import load_gl  # noqa: E402
from matrix_b200.sharded import LibTranscript, TorchComm, prove_sharded  # noqa: E402
from oracle import pyoracle  # noqa: E402
from tests.sharded_helpers import OracleShard, assert_same_proof, inputs, shard_slices  # noqa: E402


def main():
    out_path = sys.argv[1]
    dist.init_process_group("gloo")
    comm = TorchComm()
    K, nv, g_bits = 3, 6, 1
    a, b, point = inputs(K, nv)
    lib = load_gl()  # only the host transcript is used here (no GPU needed)
    oracle = pyoracle.load()

    def make_shard(g, point_low, scale):
        sa, sb = shard_slices(a, b, K, nv, g_bits, g)
        return OracleShard(oracle, sa, sb, point_low, scale, K, nv - g_bits)

    got = prove_sharded(make_shard, LibTranscript(lib, b"bench"), comm, point, K, nv, g_bits)
    exp = pyoracle.batched_prove(a, b, np.array([c for t in point for c in t], dtype=np.uint64), K, nv)
    assert_same_proof(got, exp)
    with open("%s.%d" % (out_path, comm.rank), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
