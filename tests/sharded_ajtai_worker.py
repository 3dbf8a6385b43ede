"""One rank of the column-sharded Ajtai commitment. With `gpu` as the second argument the rank commits its
columns on its own GPU through the C-ABI (NCCL); otherwise the oracle computes them (gloo, CPU only)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch.distributed as dist  # noqa: E402

from matrix_b200.sharded import TorchComm, commit_sharded  # noqa: E402
from oracle import pyoracle  # noqa: E402
from tests.test_sharded_ajtai_cpu import KEY, digits_for, oracle_columns  # noqa: E402


def main():
    out_path = sys.argv[1]
    on_gpu = len(sys.argv) > 2 and sys.argv[2] == "gpu"
    n_ring, planes = (301, 3) if on_gpu else (9, 2)
    digits = digits_for(n_ring, planes)
    if on_gpu:
        import torch
        from matrix_b200.ffi import DeviceBuffer, load_agl
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        comm = TorchComm(device=torch.device("cuda", local))
        lib = load_agl()
        assert lib.cuda_set_device(local) == 0
        d_k = DeviceBuffer.from_numpy(lib, KEY)
        d3 = digits.reshape(planes, n_ring, 64)

        def commit(lo, hi):
            out = DeviceBuffer(lib, planes * 42 * 64 * 8)
            part = np.ascontiguousarray(d3[:, lo:hi, :]).reshape(-1)
            d_z = DeviceBuffer.from_numpy(lib, part if part.size else np.zeros(64, dtype=np.int8))
            assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, hi - lo, planes, lo, out.ptr) == 0
            return out.to_numpy()
    else:
        dist.init_process_group("gloo")
        comm = TorchComm()
        commit = oracle_columns(digits, n_ring, planes)
    got = commit_sharded(commit, comm, n_ring, planes)
    assert np.array_equal(got, pyoracle.ajtai_commit(KEY, digits, 1, n_ring, planes))
    with open("%s.%d" % (out_path, comm.rank), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
