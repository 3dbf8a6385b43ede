"""Column-sharded module commitment, host logic on CPU: partial commitments from the oracle over column
ranges, ranks in one process and as two gloo processes; the sum must equal the unsharded commitment."""
import os
import subprocess
import sys

import numpy as np
import pytest

from matrix_b200.sharded import SingleComm, module_commit_sharded
from oracle import pyoracle
from .conftest import ROOT

SEED = [4, 4, 2, 2, 1, 1, 0, 9]
KIND = 1
N = 4096


def columns_for(ncols, seed=5):
    return np.random.default_rng(seed).integers(-1, 2, size=(ncols, N), dtype=np.int8)


def oracle_columns(x, rows):
    def commit(lo, hi):
        if hi == lo:
            return np.zeros(rows * N, dtype=np.uint64)
        return pyoracle.mcommit_commit(SEED, KIND, rows, list(range(lo, hi)), x[lo:hi].astype(np.int64)).reshape(-1)
    return commit


@pytest.mark.parametrize("ncols,rows,world", [(3, 1, 2), (2, 2, 4)])
def test_in_process_column_shards(ncols, rows, world):
    x = columns_for(ncols)
    whole = pyoracle.mcommit_commit(SEED, KIND, rows, list(range(ncols)), x.astype(np.int64))
    got = module_commit_sharded(oracle_columns(x, rows), SingleComm(world), ncols, 1, rows)
    assert np.array_equal(got, whole.reshape(-1))


def test_two_gloo_ranks(tmp_path):
    out = str(tmp_path / "done")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29547", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29547", os.path.join(ROOT, "tests", "sharded_mcommit_worker.py"), out]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert os.path.exists(out + ".0") and os.path.exists(out + ".1")
