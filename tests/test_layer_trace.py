"""Host logic of the decoder-layer trace (no GPU): variable classes of the layer's equations and the
index tables of the fused permutation kernel against a direct bit permutation."""
import numpy as np

from matrix_b200.layer_trace import EinsumPlan, llama_layer_ops, split_luts


def test_layer_plans():
    ops = llama_layer_ops()
    assert len(ops) == 7 + 16 * 5
    shapes = {name: EinsumPlan(eq, dims) for name, eq, dims in ops}
    q = shapes["attn_q"]            # [128 x 4096] . [4096 x 4096]: 12 summation rounds, no shared variable
    assert (q.rounds, len(q.shared), [len(f) for f in q.fixed]) == (12, 0, [7, 12])
    assert q.operand_order(1)[0] == list(range(24))            # the weight's fixed variables are its low bits
    assert q.operand_order(0)[0] == list(range(12, 19)) + list(range(12))
    sc = shapes["attn_scores"]      # heads are shared (eq table), head_dim is summed
    assert (sc.rounds, len(sc.shared), len(sc.summed)) == (12, 5, 7)
    assert shapes["attn_scale"].rounds == 0 and len(shapes["attn_scale"].fixed[0]) == 19
    ew = shapes["ffn3_mul"]         # element-wise product: every variable shared
    assert (ew.rounds, len(ew.shared), ew.fixed) == (17, 17, [[], []])
    assert shapes["ffn0_down"].rounds == 10 and [len(f) for f in shapes["ffn0_down"].fixed] == [7, 12]


def test_split_luts_compose_to_the_permutation():
    rng = np.random.default_rng(5)
    for n, half in ((6, 3), (11, 5), (13, 6)):
        order = [int(x) for x in rng.permutation(n)]
        lo, hi = split_luts(n, order, half)
        for x in [0, 1, (1 << n) - 1] + [int(v) for v in rng.integers(0, 1 << n, 50)]:
            want = sum(1 << order[b] for b in range(n) if x >> b & 1)
            assert int(lo[x & ((1 << half) - 1)]) | int(hi[x >> half]) == want
