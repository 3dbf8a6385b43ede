"""Column-sharded Ajtai commitment, host logic on CPU: partial commitments from the oracle over column windows,
ranks in one process and as two gloo processes; the sum must equal the unsharded commitment."""
import os
import subprocess
import sys

import numpy as np
import pytest

from matrix_b200.sharded import SingleComm, column_range, commit_sharded
from oracle import pyoracle
from .conftest import ROOT

KEY = np.arange(1, 9, dtype=np.uint32)


def digits_for(n_ring, planes, seed=5):
    return np.random.default_rng(seed).integers(-127, 128, size=planes * n_ring * 64, dtype=np.int8)


def oracle_columns(digits, n_ring, planes):
    d = digits.reshape(planes, n_ring, 64)

    def commit(lo, hi):
        if hi == lo:
            return np.zeros(planes * 42 * 64, dtype=np.uint64)
        part = np.ascontiguousarray(d[:, lo:hi, :]).reshape(-1)
        return pyoracle.ajtai_commit(KEY, part, 1, hi - lo, planes, lo)
    return commit


@pytest.mark.parametrize("n_ring,planes,world", [(7, 1, 2), (10, 3, 4), (3, 2, 8)])
def test_in_process_column_shards(n_ring, planes, world):
    digits = digits_for(n_ring, planes)
    whole = pyoracle.ajtai_commit(KEY, digits, 1, n_ring, planes)
    got = commit_sharded(oracle_columns(digits, n_ring, planes), SingleComm(world), n_ring, planes)
    assert np.array_equal(got, whole)
    ranges = [column_range(n_ring, world, g) for g in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n_ring and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))


def test_two_gloo_ranks(tmp_path):
    out = str(tmp_path / "done")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29541", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "sharded_ajtai_worker.py"), out]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert os.path.exists(out + ".0") and os.path.exists(out + ".1")
