"""One rank of the world-size-2 CPU test (gloo) of the sharded Basefold scheme: the partition, the exchange
pattern and the recombination rules of matrix_b200/csrc/host/gl_basefold_sharded.cu restated in numpy, with
the CPU oracle doing the per-rank work. Every recombined value must equal the unsharded oracle's.
Started by test_sharded_basefold_cpu.py."""
import ctypes
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from matrix_b200.inputs import field_elems  # noqa: E402
from oracle import pyoracle  # noqa: E402

P = 0xFFFFFFFF00000001


def all_gather_words(arr):
    """Rank-major concatenation of every rank's uint64 array (same length on all ranks)."""
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int64).copy())
    outs = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(outs, t)
    return [o.numpy().view(np.uint64).copy() for o in outs]


def e2_mul(a, b):
    return ((a[0] * b[0] + 7 * a[1] * b[1]) % P, (a[0] * b[1] + a[1] * b[0]) % P)


def check(nv, lr, oracle):
    G, g = dist.get_world_size(), dist.get_rank()
    gamma = G.bit_length() - 1
    m = gamma - lr
    assert m >= 0
    n = 1 << nv
    evals = field_elems(3, n)
    point = field_elems(4, 2 * nv)
    table = pyoracle.bf_table(nv, lr)
    cw, bh, tree = pyoracle.bf_commit(evals, nv, lr)
    n_loc, C = n // G, (n << lr) // G
    mine = [int(x) for x in evals[g * n_loc:(g + 1) * n_loc]]

    # low m bits of the commitment transform, then the pieces: slot r holds the entries whose low bits are tau_r
    for bit in range(m):
        for x in range(n_loc):
            if not (x >> bit) & 1:
                e0, e1 = mine[x], mine[x | 1 << bit]
                mine[x], mine[x | 1 << bit] = e1, (2 * e0 - e1) % P
    width, pieces = 1 << m, n_loc >> m
    send = np.zeros(G * pieces, dtype=np.uint64)
    for r in range(G):
        s = r & (width - 1)
        tau = int(bin(s)[2:].zfill(m)[::-1], 2) if m else 0
        send[r * pieces:(r + 1) * pieces] = [mine[xh * width + tau] for xh in range(pieces)]
    gathered = all_gather_words(send)                       # all-to-all as a gather + selection
    recv = np.concatenate([gathered[src][g * pieces:(g + 1) * pieces] for src in range(G)])
    assert len(recv) == C
    # the remaining nv - m bits: the ordinary interpolate + encode on the slice
    coeffs, scratch = np.zeros(C, dtype=np.uint64), np.zeros(C, dtype=np.uint64)
    oracle.oracle_bf_bhc_interpolate(recv.ctypes.data, coeffs.ctypes.data, scratch.ctypes.data, nv - m)
    slice_cw = np.zeros(C, dtype=np.uint64)
    oracle.oracle_bf_encode(coeffs.ctypes.data, slice_cw.ctypes.data, nv - m, 0)
    assert np.array_equal(slice_cw, cw[g * C:(g + 1) * C]), "codeword range of rank %d" % g

    # commitment tree: one part per rank, parts in block order, lr levels of equal children on top
    b_idx, s_idx = g >> m, g & (width - 1)
    part_leaves = (n // 2) // G
    part_cw = np.ascontiguousarray(slice_cw[2 * b_idx * part_leaves:2 * (b_idx + 1) * part_leaves])
    ptree = np.zeros(4 * (2 * part_leaves - 1), dtype=np.uint64)
    oracle.oracle_bf_merkle_tree(part_cw.ctypes.data, part_leaves, 0, ptree.ctypes.data)
    roots = all_gather_words(ptree[-4:])
    parts = [None] * G
    for r in range(G):
        parts[(r & (width - 1)) * (1 << lr) + (r >> m)] = roots[r]
    oracle.gl_compress.argtypes = [ctypes.c_void_p] * 3

    def compress(a, b):
        o = np.zeros(4, dtype=np.uint64)
        a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
        oracle.gl_compress(a.ctypes.data, b.ctypes.data, o.ctypes.data)
        return o

    level = parts
    while len(level) > 1:
        level = [compress(level[2 * j], level[2 * j + 1]) for j in range(len(level) // 2)]
    top = level[0]
    for _ in range(lr):
        top = compress(top, top)
    assert np.array_equal(top, tree[-4:]), "commitment root"

    # eq over the low coordinates scaled by the eq value of the rank's high bits = the rank's range of the table
    nv_loc = nv - gamma
    eq_full = np.zeros(2 * n, dtype=np.uint64)
    oracle.oracle_gl_eq_ext2(point.ctypes.data, nv, eq_full.ctypes.data)
    eq_low = np.zeros(2 * n_loc, dtype=np.uint64)
    oracle.oracle_gl_eq_ext2(point.ctypes.data, nv_loc, eq_low.ctypes.data)
    scale = (1, 0)
    for k in range(gamma):
        r = (int(point[2 * (nv_loc + k)]), int(point[2 * (nv_loc + k) + 1]))
        scale = e2_mul(scale, r if (g >> k) & 1 else ((1 - r[0]) % P, (-r[1]) % P))
    for x in range(n_loc):
        v = e2_mul((int(eq_low[2 * x]), int(eq_low[2 * x + 1])), scale)
        assert v == (int(eq_full[2 * (g * n_loc + x)]), int(eq_full[2 * (g * n_loc + x) + 1]))

    # first oracle: partial coefficient sums per rank add up to the proof's
    exp, _ = pyoracle.bf_open(cw, bh, tree, nv, lr, point, table, 3)
    part = [0] * 6
    for j in range(n_loc // 2):
        x = g * n_loc + 2 * j
        q0 = (int(eq_full[2 * x]), int(eq_full[2 * x + 1]))
        q1 = (int(eq_full[2 * x + 2]), int(eq_full[2 * x + 3]))
        b0, b1 = int(evals[x]), int(evals[x + 1])
        qd, bd = ((q1[0] - q0[0]) % P, (q1[1] - q0[1]) % P), (b1 - b0) % P
        terms = [(q0[0] * b0, q0[1] * b0), (q0[0] * bd + qd[0] * b0, q0[1] * bd + qd[1] * b0), (qd[0] * bd, qd[1] * bd)]
        for k, tm in enumerate(terms):
            part[2 * k] = (part[2 * k] + tm[0]) % P
            part[2 * k + 1] = (part[2 * k + 1] + tm[1]) % P
    allp = all_gather_words(np.array(part, dtype=np.uint64))
    tot = [sum(int(a[k]) for a in allp) % P for k in range(6)]
    assert tot == [int(x) for x in exp[2:8]], "first oracle"
    assert [(2 * tot[0] + tot[2] + tot[4]) % P, (2 * tot[1] + tot[3] + tot[5]) % P] == [int(exp[0]), int(exp[1])], "claimed value"
    return True


def main():
    out_path = sys.argv[1]
    dist.init_process_group("gloo")
    oracle = pyoracle.load()
    for nv, lr in ((6, 1), (7, 0), (5, 1)):
        assert check(nv, lr, oracle)
    with open("%s.%d" % (out_path, dist.get_rank()), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
