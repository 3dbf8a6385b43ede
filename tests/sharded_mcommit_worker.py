"""One rank of the column-sharded module commitment. With `gpu` as the second argument the rank builds the
key cache of its column range and commits on its own GPU through the C-ABI (NCCL); otherwise the oracle
computes its columns (gloo, CPU only)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch.distributed as dist  # noqa: E402

from matrix_b200.sharded import TorchComm, module_commit_sharded  # noqa: E402
from oracle import pyoracle  # noqa: E402
from tests.test_sharded_mcommit_cpu import KIND, SEED, columns_for, oracle_columns  # noqa: E402

N = 4096


def main():
    out_path = sys.argv[1]
    on_gpu = len(sys.argv) > 2 and sys.argv[2] == "gpu"
    rows, ncols = (4, 11) if on_gpu else (1, 3)
    x = columns_for(ncols)
    if on_gpu:
        import torch
        from matrix_b200.ffi import DeviceBuffer, load_agl
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        comm = TorchComm(device=torch.device("cuda", local))
        lib = load_agl()
        assert lib.cuda_set_device(local) == 0
        seed = np.asarray(SEED, dtype=np.uint32)

        def commit(lo, hi):
            if hi == lo:
                return np.zeros(rows * N, dtype=np.uint64)
            key = DeviceBuffer(lib, 3 * (hi - lo) * rows * N * 4)
            assert lib.agl_mcommit_keygen(seed.ctypes.data, KIND, rows, lo, hi - lo, 3, key.ptr) == 0
            d_x = DeviceBuffer.from_numpy(lib, np.ascontiguousarray(x[lo:hi]))
            acc = DeviceBuffer(lib, 3 * rows * N * 4)
            assert lib.agl_mcommit_partial(key.ptr, hi - lo, rows, 3, d_x.ptr, 1, 1, hi - lo, 0, None, acc.ptr) == 0
            out = DeviceBuffer(lib, rows * N * 8)
            assert lib.agl_mcommit_finish(acc.ptr, 1, 3, rows, None, out.ptr) == 0
            return out.to_numpy()
    else:
        dist.init_process_group("gloo")
        comm = TorchComm()
        commit = oracle_columns(x, rows)
    got = module_commit_sharded(commit, comm, ncols, 1, rows)
    want = pyoracle.mcommit_commit(SEED, KIND, rows, list(range(ncols)), x.astype(np.int64))
    assert np.array_equal(got, want.reshape(-1))
    with open("%s.%d" % (out_path, comm.rank), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
