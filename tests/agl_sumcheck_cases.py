"""The deterministic cases of the reference's own tests for the almost-Goldilocks linear sumcheck
(zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:117-207), shared by the oracle and the GPU tests:
(label, num_var, tables as lists of base-field values, claimed sum)."""
CASES = [
    (b"cpu-ext2-roundtrip", 2, [[1, 2, 3, 4], [5, 6, 7, 8]], 1 * 5 + 2 * 6 + 3 * 7 + 4 * 8),
    (b"tamper", 2, [[1, 2, 3, 4], [5, 6, 7, 8]], 70),
    (b"three-poly", 2, [[1, 2, 3, 4], [2, 3, 5, 7], [11, 13, 17, 19]], 887),
    (b"larger", 4, [[i * 3 + 1 for i in range(16)], [i * 5 + 7 for i in range(16)]],
     sum((i * 3 + 1) * (i * 5 + 7) for i in range(16))),
]


def lifted(tables):
    """Tables of base-field values as poly-major (c0, c1) words."""
    import numpy as np
    out = np.zeros((len(tables), len(tables[0]), 2), dtype=np.uint64)
    for i, t in enumerate(tables):
        out[i, :, 0] = t
    return out.reshape(-1)
