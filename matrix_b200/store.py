"""On-disk store of Ajtai edge commitments, byte-compatible with the reference's `GpuAjtaiStore::save` / `load`
(zk-torch-4/src/commit/mod.rs:199-310): the data format on the output side of the ring commit.

    magic "ZKAJTAI1" | max_num_vars u32 | b u32 | seed 8 x u32 | num_edges u32
    per edge: has_commitment u8; when 1: is_sparse u8 | arity u32 | num_planes u32 |
              planes: num_planes x 42 x 64 u64 (row-major)
All integers little-endian. (The reference's format comment omits `arity`; its writer and reader both have it.)
"""
import struct

import numpy as np

MAGIC = b"ZKAJTAI1"
KAPPA, RING_DIM = 42, 64


class EdgeCommitment:
    """planes: uint64 [num_planes][42][64], canonical coefficients as the commit entry points return them."""

    def __init__(self, planes, is_sparse, arity):
        self.planes = np.ascontiguousarray(planes, dtype=np.uint64).reshape(-1, KAPPA, RING_DIM)
        self.is_sparse = bool(is_sparse)
        self.arity = int(arity)
        # the loader's rule: sparse commitments are unary, dense ones binary-decomposed (commit/mod.rs:296-300)
        self.base = 1 if self.is_sparse else 2

    def __eq__(self, other):
        return (isinstance(other, EdgeCommitment) and self.is_sparse == other.is_sparse and self.arity == other.arity
                and np.array_equal(self.planes, other.planes))


class AjtaiStore:
    def __init__(self, max_num_vars, b, seed, commitments):
        self.max_num_vars, self.b = int(max_num_vars), int(b)
        self.seed = [int(w) for w in seed]
        if len(self.seed) != 8:
            raise ValueError("seed is 8 words")
        self.commitments = list(commitments)   # EdgeCommitment or None per edge

    def save(self, path):
        with open(path, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<II8II", self.max_num_vars, self.b, *self.seed, len(self.commitments)))
            for ec in self.commitments:
                if ec is None:
                    f.write(b"\x00")
                    continue
                f.write(struct.pack("<BBII", 1, int(ec.is_sparse), ec.arity, ec.planes.shape[0]))
                f.write(ec.planes.astype("<u8").tobytes())

    @classmethod
    def load(cls, path):
        with open(path, "rb") as f:
            data = f.read()
        if data[:8] != MAGIC:
            raise ValueError("bad magic")
        head = struct.unpack_from("<II8II", data, 8)
        max_num_vars, b, seed, num_edges = head[0], head[1], head[2:10], head[10]
        pos = 8 + 44
        commitments = []
        for edge in range(num_edges):
            if pos >= len(data):
                raise ValueError("edge %d: truncated" % edge)
            tag = data[pos]
            pos += 1
            if tag == 0:
                commitments.append(None)
                continue
            if tag != 1:
                raise ValueError("edge %d: invalid commit tag %d" % (edge, tag))
            sparse, arity, n_planes = struct.unpack_from("<BII", data, pos)
            pos += 9
            if sparse > 1:
                raise ValueError("edge %d: invalid is_sparse %d" % (edge, sparse))
            nbytes = n_planes * KAPPA * RING_DIM * 8
            if pos + nbytes > len(data):
                raise ValueError("edge %d: truncated planes" % edge)
            planes = np.frombuffer(data, dtype="<u8", count=n_planes * KAPPA * RING_DIM, offset=pos).astype(np.uint64)
            pos += nbytes
            commitments.append(EdgeCommitment(planes, sparse == 1, arity))
        return cls(max_num_vars, b, seed, commitments)
