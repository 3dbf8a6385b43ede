"""Link sumcheck round sharded over commitments, host logic on CPU (messages from the oracle)."""
import numpy as np
import pytest

from matrix_b200.sharded import SingleComm, link_round_sharded
from oracle import pyoracle as po
from .link_cases import ext, sparse_ext


@pytest.mark.parametrize("nc,world", [(5, 2), (3, 4), (8, 8)])
def test_commitment_shards_add_up(nc, world):
    half = 64
    stride = 2 * half
    w, om, eq, tags = sparse_ext(1, nc * stride, 0.4), ext(2, nc * stride), ext(3, half), ext(4, nc)

    def part(lo, hi):
        if hi == lo:
            return np.zeros(14, dtype=np.uint64)
        return po.link_round(eq, np.ascontiguousarray(tags[2 * lo:2 * hi]), half, hi - lo, 0, w=np.ascontiguousarray(w[2 * lo * stride:2 * hi * stride]),
                             omega=np.ascontiguousarray(om[2 * lo * stride:2 * hi * stride]), w_stride=stride, omega_stride=stride)
    whole = po.link_round(eq, tags, half, nc, 0, w=w, omega=om, w_stride=stride, omega_stride=stride)
    assert np.array_equal(link_round_sharded(part, SingleComm(world), nc), whole)
