"""Host logic of the sharded batched sumcheck on CPU: shards computed by the
oracle, transcript by the library's host code, ranks in one process and as two
gloo processes; every variant must reproduce the unsharded oracle proof."""
import os
import subprocess
import sys

import numpy as np
import pytest

from matrix_b200 import load_gl
from matrix_b200.sharded import LibTranscript, SingleComm, prove_sharded
from .conftest import ROOT
from .sharded_helpers import OracleShard, assert_same_proof, inputs, shard_slices


@pytest.mark.parametrize("K,nv,g_bits", [(1, 3, 0), (2, 5, 1), (3, 6, 2), (2, 4, 3)])
def test_in_process_shards_match_unsharded_oracle(oracle, K, nv, g_bits):
    from oracle import pyoracle
    a, b, point = inputs(K, nv)
    lib = load_gl()

    def make_shard(g, point_low, scale):
        sa, sb = shard_slices(a, b, K, nv, g_bits, g)
        return OracleShard(oracle, sa, sb, point_low, scale, K, nv - g_bits)

    got = prove_sharded(make_shard, LibTranscript(lib, b"bench"), SingleComm(1 << g_bits), point, K, nv, g_bits)
    exp = pyoracle.batched_prove(a, b, np.array([c for t in point for c in t], dtype=np.uint64), K, nv)
    assert_same_proof(got, exp)
    # the claimed sums are what they say: s_k = sum_x eq(x) a_k(x) b_k(x); round 0 sums to the combined claim
    from matrix_b200.sharded import e2_add, e2_mul
    tot, pw = (0, 0), (1, 0)
    alpha = tuple(int(x) for x in got["alpha"])
    for k in range(K):
        tot = e2_add(tot, e2_mul(pw, tuple(int(x) for x in got["claims"][k])))
        pw = e2_mul(pw, alpha)
    m0, m1 = got["round_msgs"][0][0], got["round_msgs"][0][1]
    assert e2_add(tuple(int(x) for x in m0), tuple(int(x) for x in m1)) == tot


def test_two_gloo_ranks(tmp_path):
    out = str(tmp_path / "done")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "sharded_worker.py"), out]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert os.path.exists(out + ".0") and os.path.exists(out + ".1")


@pytest.mark.parametrize("world", [2, 4])
def test_shared_memory_exchange(tmp_path, world):
    """The host mailbox exchange between processes of one node: 200 ordered calls, then a whole sharded proof."""
    path = str(tmp_path / "mailbox")
    env = dict(os.environ, OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "shm_worker.py"), path, str(r), str(world)],
                              cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=280)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\\n".join(o[-1500:] for o in outs)
    assert all(os.path.exists("%s.ok.%d" % (path, r)) for r in range(world))
