"""One rank of the multi-GPU test: the sharded batched sumcheck with a GPU shard
per rank, first under the Python round loop with NCCL for the per-round exchange,
then with the whole loop inside the library over its shared-memory mailbox.
Started by test_multigpu.py."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from matrix_b200 import load_gl  # noqa: E402
from matrix_b200.ffi import DeviceBuffer  # noqa: E402
from matrix_b200.sharded import (GpuShard, LibTranscript, MailboxExchange, TorchComm, prove_batched_native,  # noqa: E402
                                 prove_sharded)
from oracle import pyoracle  # noqa: E402
from tests.sharded_helpers import assert_same_proof, inputs, shard_slices  # noqa: E402


def main():
    out_path = sys.argv[1]
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = load_gl()
    assert lib.cuda_set_device(local) == 0
    comm = TorchComm(device=torch.device("cuda", local))
    g_bits = comm.world.bit_length() - 1
    K, nv = 4, 14
    a, b, point = inputs(K, nv)
    keep = []

    def make_shard(g, point_low, scale):
        sa, sb = shard_slices(a, b, K, nv, g_bits, g)
        d_a, d_b = DeviceBuffer.from_numpy(lib, sa), DeviceBuffer.from_numpy(lib, sb)
        keep.extend([d_a, d_b])
        return GpuShard(lib, d_a.ptr, d_b.ptr, point_low, scale, K, nv - g_bits)

    got = prove_sharded(make_shard, LibTranscript(lib, b"bench"), comm, point, K, nv, g_bits)
    exp = pyoracle.batched_prove(a, b, np.array([c for t in point for c in t], dtype=np.uint64), K, nv)
    assert_same_proof(got, exp)
    # the same proof with the round loop in the library
    token = [os.urandom(6).hex() if comm.rank == 0 else None]
    dist.broadcast_object_list(token, src=0)
    ex = MailboxExchange(lib, "/mb_test_batched_%s" % token[0], comm.rank, comm.world)
    dist.barrier()
    sa, sb = shard_slices(a, b, K, nv, g_bits, comm.rank)
    d_a, d_b = DeviceBuffer.from_numpy(lib, sa), DeviceBuffer.from_numpy(lib, sb)
    native = prove_batched_native(lib, ex.handle, d_a.ptr, d_b.ptr, K, nv, point, b"bench")
    assert_same_proof(native, exp)
    dist.barrier()
    ex.close()
    with open("%s.%d" % (out_path, comm.rank), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
