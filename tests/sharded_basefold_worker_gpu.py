"""One rank of the multi-GPU test of the sharded Basefold prover: one process per GPU, host words through the
shared-memory mailbox, the device all-to-all through NCCL. Every rank's proof must equal the CPU oracle's proof of
the whole polynomial (and so the single-GPU proof). Started by test_multigpu.py."""
import ctypes
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from matrix_b200 import load_gl  # noqa: E402
from matrix_b200.inputs import field_elems  # noqa: E402
from matrix_b200.sharded import ProcessExchange  # noqa: E402
from oracle import pyoracle  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = load_gl()
    assert lib.cuda_set_device(local) == 0
    token = [os.urandom(6).hex() if rank == 0 else None]
    dist.broadcast_object_list(token, src=0)
    ex = ProcessExchange(lib, "/mb_test_basefold_%s" % token[0], rank, world, torch.device("cuda", local))
    for nv, lr, nq in ((16, 1, 30), (18, 1, 100)):
        n = 1 << nv
        evals, point = field_elems(3, n), field_elems(4, 2 * nv)
        table = pyoracle.bf_table(nv, lr)
        cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
        exp, _ = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, nq)
        h = ctypes.c_void_p()
        assert lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(h)) == 0
        n_loc = n // world
        shard = np.ascontiguousarray(evals[rank * n_loc:(rank + 1) * n_loc])
        proof = np.zeros(lib.basefold_proof_words(nv, lr, nq), dtype=np.uint64)
        root = np.zeros(4, dtype=np.uint64)
        for _ in range(2):   # twice: the mailbox generations and the pooled buffers carry over
            rc = lib.basefold_prove_sharded_host(shard.ctypes.data, nv, lr, point.ctypes.data, h, b"bench", 5, nq, ex.handle,
                                                 root.ctypes.data, proof.ctypes.data)
            assert rc == 0, "basefold_prove_sharded_host: %d" % rc
            assert np.array_equal(root, tree[-4:]), "root"
            bad = np.nonzero(proof != exp)[0]
            assert len(bad) == 0, "rank %d: first differing proof word %d of %d" % (rank, bad[0], len(exp))
        lib.basefold_table_destroy(h)
    assert ex.calls == 4
    dist.barrier()
    ex.close()
    with open("%s.%d" % (out_path, rank), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
