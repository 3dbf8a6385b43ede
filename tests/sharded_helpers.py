"""Test doubles for the sharded batched sumcheck: a shard computed by the CPU
oracle (same methods as matrix_b200.sharded.GpuShard) and seeded inputs."""
import numpy as np

from matrix_b200.inputs import field_elems
from matrix_b200.sharded import GL_P, e2_mul


def inputs(K, nv, seed=100):
    n = 1 << nv
    a = np.concatenate([field_elems(seed + k, n) for k in range(K)])
    b = np.concatenate([field_elems(seed + 100 + k, n) for k in range(K)])
    pt = field_elems(6, 2 * nv)
    point = [(int(pt[2 * i]), int(pt[2 * i + 1])) for i in range(nv)]
    return a, b, point


def shard_slices(a, b, K, nv, g_bits, g):
    """Rows [K][2^n_loc] of rank g: the entries whose top g_bits index bits equal g."""
    n, n_loc = 1 << nv, nv - g_bits
    m = 1 << n_loc
    sa = np.concatenate([a[k * n + g * m:k * n + (g + 1) * m] for k in range(K)])
    sb = np.concatenate([b[k * n + g * m:k * n + (g + 1) * m] for k in range(K)])
    return sa, sb


class OracleShard:
    """A shard evaluated by the CPU oracle's batched message / fold / claims functions."""

    def __init__(self, oracle, sa, sb, point_low, scale, K, n_loc):
        self.o, self.K, self.n = oracle, K, 1 << n_loc
        n = self.n
        pl = np.array([c for t in point_low for c in t], dtype=np.uint64)
        eq = np.zeros(2 * n, dtype=np.uint64)
        oracle.oracle_gl_eq_ext2(pl.ctypes.data, n_loc, eq.ctypes.data)
        self.eq = np.array([c for i in range(n) for c in e2_mul((int(eq[2 * i]), int(eq[2 * i + 1])), scale)], dtype=np.uint64)
        self.ab = np.zeros(2 * K * n * 2, dtype=np.uint64)
        for k in range(K):
            self.ab[(2 * k) * n * 2:(2 * k + 1) * n * 2:2] = sa[k * n:(k + 1) * n]
            self.ab[(2 * k + 1) * n * 2:(2 * k + 2) * n * 2:2] = sb[k * n:(k + 1) * n]
        self.size = n
        self.alpha_pows = None

    def claims(self):
        out = np.zeros(2 * self.K, dtype=np.uint64)
        self.o.oracle_gl_batched_claims(self.eq.ctypes.data, self.ab.ctypes.data, self.K, self.n, self.size, out.ctypes.data)
        return out

    def set_alpha(self, alpha):
        pw, p = [], (1, 0)
        for _ in range(self.K):
            pw += [p[0], p[1]]
            p = e2_mul(p, alpha)
        self.alpha_pows = np.array(pw, dtype=np.uint64)
        self.alpha = alpha

    def round_message(self):
        out = np.zeros(8, dtype=np.uint64)
        self.o.oracle_gl_batched_message(self.eq.ctypes.data, self.ab.ctypes.data, self.alpha_pows.ctypes.data, self.K,
                                         self.n, self.size // 2, out.ctypes.data)
        return out

    def fold(self, r):
        self.o.oracle_gl_batched_fold(self.eq.ctypes.data, self.ab.ctypes.data, r[0], r[1], self.K, self.n, self.size // 2)
        self.size //= 2

    def finals(self):
        # eq, alpha^k a_k, b_k (the GPU shard carries the alpha^k factor in a_k)
        out = [int(self.eq[0]), int(self.eq[1])]
        n = self.n
        for k in range(self.K):
            a = (int(self.ab[(2 * k) * n * 2]), int(self.ab[(2 * k) * n * 2 + 1]))
            w = (int(self.alpha_pows[2 * k]), int(self.alpha_pows[2 * k + 1]))
            out += list(e2_mul(w, a))
        for k in range(self.K):
            out += [int(self.ab[(2 * k + 1) * n * 2]), int(self.ab[(2 * k + 1) * n * 2 + 1])]
        return np.array(out, dtype=np.uint64)


def assert_same_proof(got, exp):
    for key in ("claims", "alpha", "round_msgs", "challenges", "finals", "final_eval", "state"):
        assert np.array_equal(np.asarray(got[key]).reshape(-1), np.asarray(exp[key]).reshape(-1)), key
