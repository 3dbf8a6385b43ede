"""The sharded Basefold scheme on CPU with two gloo ranks: partition, exchange and recombination restated in
numpy over the CPU oracle (tests/sharded_basefold_worker.py); every recombined value equals the unsharded one."""
import os
import subprocess
import sys

from .conftest import ROOT


def test_two_gloo_ranks_recombine_to_the_unsharded_commitment_and_first_oracle(tmp_path):
    out = str(tmp_path / "done")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29537", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29537", os.path.join(ROOT, "tests", "sharded_basefold_worker.py"), out]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert os.path.exists(out + ".0") and os.path.exists(out + ".1")
