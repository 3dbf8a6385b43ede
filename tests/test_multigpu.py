"""The sharded provers on two or more real GPUs, one process per GPU (NCCL): skipped on a box with fewer."""
import os
import subprocess
import sys

import pytest

from .conftest import ROOT

pytestmark = pytest.mark.gpu


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs at least two GPUs")
def test_sharded_sumcheck_over_nccl(tmp_path):
    n = 1
    while n * 2 <= min(_gpu_count(), 8):
        n *= 2
    out = str(tmp_path / "done")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "sharded_worker_gpu.py"), out]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    for g in range(n):
        assert os.path.exists("%s.%d" % (out, g))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs at least two GPUs")
def test_column_sharded_ajtai_over_nccl(tmp_path):
    n = min(_gpu_count(), 8)
    out = str(tmp_path / "done")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", "29543", os.path.join(ROOT, "tests", "sharded_ajtai_worker.py"), out, "gpu"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    for g in range(n):
        assert os.path.exists("%s.%d" % (out, g))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs at least two GPUs")
def test_column_sharded_module_commit_over_nccl(tmp_path):
    n = min(_gpu_count(), 8)
    out = str(tmp_path / "done")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", "29549", os.path.join(ROOT, "tests", "sharded_mcommit_worker.py"), out, "gpu"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    for g in range(n):
        assert os.path.exists("%s.%d" % (out, g))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs at least two GPUs")
def test_one_basefold_proof_over_several_gpus(tmp_path):
    """One commitment + opening partitioned over the GPUs: every rank's proof equals the CPU oracle's."""
    n = 1
    while n * 2 <= min(_gpu_count(), 8):
        n *= 2
    out = str(tmp_path / "done")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", "29551", os.path.join(ROOT, "tests", "sharded_basefold_worker_gpu.py"), out]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    for g in range(n):
        assert os.path.exists("%s.%d" % (out, g))
