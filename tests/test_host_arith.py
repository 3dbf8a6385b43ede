"""The library's own field / Poseidon2 / transcript code, compiled for the host,
against the oracle and Python integers (no GPU needed)."""
import ctypes
import random

import numpy as np

from .conftest import GL_P

P = GL_P
u64 = ctypes.c_uint64


def _setup(hc):
    for name in ("hc_gl_add", "hc_gl_sub", "hc_gl_mul", "hc_gl_inv"):
        getattr(hc, name).restype = u64
        getattr(hc, name).argtypes = [u64, u64] if name != "hc_gl_inv" else [u64]
    hc.hc_gl_mul_small.restype = u64
    hc.hc_gl_mul_small.argtypes = [u64, ctypes.c_uint32]


def test_loose_arithmetic_is_correct_mod_p(hostcheck):
    _setup(hostcheck)
    rnd = random.Random(7)
    edge = [0, 1, P - 1, P, P + 1, 2**64 - 1, 2**64 - 2, 2**32 - 1, 2**32, 2**63, 0xFFFFFFFF00000000]
    vals = edge + [rnd.randrange(2**64) for _ in range(300)]
    for a in vals:
        for b in edge + [rnd.randrange(2**64) for _ in range(20)]:
            assert hostcheck.hc_gl_add(a, b) % P == (a + b) % P
            assert hostcheck.hc_gl_sub(a, b) % P == (a - b) % P
            assert hostcheck.hc_gl_mul(a, b) % P == (a * b) % P
        assert hostcheck.hc_gl_mul_small(a, 7) % P == (a * 7) % P
        assert hostcheck.hc_gl_mul_small(a, 2**32 - 1) % P == (a * (2**32 - 1)) % P
    for a in vals[:40]:
        inv = hostcheck.hc_gl_inv(a) % P
        assert (inv * a) % P == (1 if a % P else 0)


def test_limb_reductions(hostcheck):
    _setup(hostcheck)
    hostcheck.hc_gl_mul_add.restype = u64
    hostcheck.hc_gl_mul_add.argtypes = [u64, u64, u64]
    hostcheck.hc_gl_reduce_limb_sums.restype = u64
    hostcheck.hc_gl_reduce_limb_sums.argtypes = [u64, u64]
    hostcheck.hc_gl_reduce_limbs.restype = u64
    hostcheck.hc_gl_reduce_limbs.argtypes = [ctypes.c_uint32] * 4
    rnd = random.Random(11)
    edge32 = [0, 1, 2, 0xFFFFFFFF, 0xFFFFFFFE, 0x80000000, 0x7FFFFFFF]
    for z0 in edge32:
        for z1 in edge32:
            for z2 in edge32:
                for z3 in edge32:
                    v = z0 + (z1 << 32) + (z2 << 64) + (z3 << 96)
                    assert hostcheck.hc_gl_reduce_limbs(z0, z1, z2, z3) % P == v % P
    for _ in range(3000):
        z = [rnd.randrange(2**32) for _ in range(4)]
        v = z[0] + (z[1] << 32) + (z[2] << 64) + (z[3] << 96)
        assert hostcheck.hc_gl_reduce_limbs(*z) % P == v % P
    edge64 = [0, 1, P - 1, P, 2**64 - 1, 2**64 - 2**32, 2**32 - 1, 2**32]
    for a in edge64 + [rnd.randrange(2**64) for _ in range(40)]:
        for b in edge64 + [rnd.randrange(2**64) for _ in range(10)]:
            for c in edge64 + [rnd.randrange(2**64) for _ in range(4)]:
                assert hostcheck.hc_gl_mul_add(a, b, c) % P == (a * b + c) % P
    edge40 = [0, 1, 2**32 - 1, 2**32, 2**40 - 1, 2**37, 21 * (2**32 - 1)]
    for L in edge40 + [rnd.randrange(2**40) for _ in range(60)]:
        for H in edge40 + [rnd.randrange(2**40) for _ in range(60)]:
            assert hostcheck.hc_gl_reduce_limb_sums(L, H) % P == (L + (H << 32)) % P


def test_ext2_mul_inv(hostcheck):
    rnd = random.Random(8)
    for _ in range(500):
        a = [rnd.randrange(2**64), rnd.randrange(2**64)]
        b = [rnd.randrange(2**64), rnd.randrange(2**64)]
        A, B, O = (u64 * 2)(*a), (u64 * 2)(*b), (u64 * 2)()
        hostcheck.hc_e2_mul(A, B, O)
        assert O[0] % P == (a[0] * b[0] + 7 * a[1] * b[1]) % P
        assert O[1] % P == (a[0] * b[1] + a[1] * b[0]) % P
    for _ in range(20):
        a = [rnd.randrange(P), rnd.randrange(P)]
        A, I, O = (u64 * 2)(*a), (u64 * 2)(), (u64 * 2)()
        hostcheck.hc_e2_inv(A, I)
        hostcheck.hc_e2_mul(A, I, O)
        assert (O[0] % P, O[1] % P) == (1, 0)


def test_poseidon2_matches_oracle(hostcheck, oracle):
    rnd = random.Random(9)
    for k in range(50):
        inp = list(range(8)) if k == 0 else [rnd.randrange(P) for _ in range(8)]
        a, b = (u64 * 8)(*inp), (u64 * 8)(*inp)
        hostcheck.hc_poseidon2(a)
        oracle.gl_poseidon2_permute(b)
        assert [x % P for x in a] == list(b)


def test_host_form_of_poseidon2_and_its_reductions(hostcheck, oracle):
    """Transcripts and tree tops run a permutation written for a host core (128-bit products); it must be the
    same function as the device form and the oracle on canonical, loose and extreme words."""
    AGL_P = 2**64 - 2**32 - 31
    rnd = random.Random(19)
    edge = [0, 1, P - 1, P, P + 1, 2**64 - 1, 2**64 - 2**32, 2**32 - 1, 2**32, 2**63]
    cases = [[e] * 8 for e in edge] + [[rnd.choice(edge) for _ in range(8)] for _ in range(40)]
    cases += [[rnd.randrange(2**64) for _ in range(8)] for _ in range(200)]
    for inp in cases:
        a, b, c = (u64 * 8)(*inp), (u64 * 8)(*inp), (u64 * 8)(*[x % P for x in inp])
        hostcheck.hc_poseidon2_host(a)
        hostcheck.hc_poseidon2(b)
        oracle.gl_poseidon2_permute(c)
        assert list(a) == [x % P for x in b] == list(c)
    for f in (hostcheck.hc_p2host_red, hostcheck.hc_aglm_reduce_wide, hostcheck.hc_aglm_reduce_small):
        f.restype, f.argtypes = u64, [u64, u64]
    words = edge + [AGL_P - 1, AGL_P, AGL_P + 1, 2**64 - 32, 2**64 - 31]
    pairs = [(lo, hi) for lo in words for hi in words] + [(rnd.randrange(2**64), rnd.randrange(2**64)) for _ in range(2000)]
    for lo, hi in pairs:
        x = lo + (hi << 64)
        assert hostcheck.hc_p2host_red(lo, hi) % P == x % P
        assert hostcheck.hc_aglm_reduce_wide(lo, hi) % AGL_P == x % AGL_P
    # sums of up to 161 words (one row of the MDS layer plus a constant): high word below 2^31
    for lo in words:
        for hi in (0, 1, 160, 161, 2**20, 2**31 - 1):
            assert hostcheck.hc_aglm_reduce_small(lo, hi) % AGL_P == (lo + (hi << 64)) % AGL_P


def test_host_form_extension_arithmetic(hostcheck):
    """The host rounds of a sumcheck multiply in F[X]/(X^2 - 7) over Goldilocks and F[X]/(X^2 - 3) over
    almost-Goldilocks through 128-bit products; canonical words in, canonical words out."""
    rnd = random.Random(23)
    for agl_field, q, w in ((0, P, 7), (1, 2**64 - 2**32 - 31, 3)):
        edge = [0, 1, 2, q - 1, q - 2, 2**32 - 1, 2**32, 2**63, q // 2]
        cases = [(x, y, z, t) for x in edge for y in edge[:5] for z in edge[:5] for t in edge[:4]]
        cases += [tuple(rnd.randrange(q) for _ in range(4)) for _ in range(3000)]
        for a0, a1, b0, b1 in cases:
            o = (u64 * 6)()
            hostcheck.hc_hf_e2(agl_field, (u64 * 2)(a0, a1), (u64 * 2)(b0, b1), o)
            assert o[0] == (a0 * b0 + w * a1 * b1) % q and o[1] == (a0 * b1 + a1 * b0) % q
            assert (o[2], o[3]) == ((a0 + b0) % q, (a1 + b1) % q)
            assert (o[4], o[5]) == ((a0 - b0) % q, (a1 - b1) % q)


def test_transcript_matches_oracle(hostcheck, oracle):
    # Random scripts of absorbs and squeezes against the oracle's transcript.
    class T(ctypes.Structure):
        _fields_ = [("sponge", u64 * 8), ("in_buf", u64 * 4), ("out_buf", u64 * 4),
                    ("in_count", ctypes.c_int), ("out_count", ctypes.c_int), ("perms", u64)]
    oracle.gl_transcript_squeeze.restype = u64
    oracle.gl_transcript_absorb.argtypes = [ctypes.c_void_p, u64]
    rnd = random.Random(10)
    for trial in range(20):
        nops = rnd.randrange(1, 60)
        ops = [rnd.choice([0, 0, 1]) for _ in range(nops)]
        vals = [rnd.randrange(P) for _ in range(nops)]
        label = bytes(rnd.randrange(256) for _ in range(rnd.randrange(0, 9)))
        out = (u64 * nops)()
        k = hostcheck.hc_transcript_script(label, len(label), (ctypes.c_int * nops)(*ops), (u64 * nops)(*vals), nops, out)
        t = T()
        oracle.gl_transcript_new(ctypes.byref(t), label, len(label))
        exp = []
        for o, v in zip(ops, vals):
            if o == 0:
                oracle.gl_transcript_absorb(ctypes.byref(t), v)
            else:
                exp.append(oracle.gl_transcript_squeeze(ctypes.byref(t)))
        assert list(out[:k]) == exp


def test_almost_goldilocks_loose_arithmetic(hostcheck):
    Q = 0xFFFFFFFEFFFFFFE1
    for name in ("hc_agl_add", "hc_agl_sub", "hc_agl_mul"):
        getattr(hostcheck, name).restype = u64
        getattr(hostcheck, name).argtypes = [u64, u64]
    hostcheck.hc_agl_inv.restype = u64
    hostcheck.hc_agl_inv.argtypes = [u64]
    rnd = random.Random(12)
    edge = [0, 1, Q - 1, Q, Q + 1, 2**64 - 1, 2**64 - 2, 2**32 + 31, 2**32 + 30, 2**32, 2**63, 0xFFFFFFFF00000000]
    vals = edge + [rnd.randrange(2**64) for _ in range(300)]
    for a in vals:
        for b in edge + [rnd.randrange(2**64) for _ in range(20)]:
            assert hostcheck.hc_agl_add(a, b) % Q == (a + b) % Q
            assert hostcheck.hc_agl_sub(a, b) % Q == (a - b) % Q
            assert hostcheck.hc_agl_mul(a, b) % Q == (a * b) % Q
    for a in vals[:30]:
        assert (hostcheck.hc_agl_inv(a) * a) % Q == (1 if a % Q else 0)
    # (1 + 2X)(3 + 4X) = 27 + 10X with X^2 = 3 (almost-goldilocks-cuda-rs/tests/integration.rs:141-146)
    A, B, O = (u64 * 2)(1, 2), (u64 * 2)(3, 4), (u64 * 2)()
    hostcheck.hc_aext2_mul(A, B, O)
    assert (O[0] % Q, O[1] % Q) == (27, 10)


def test_lazy_accumulators(hostcheck):
    """Sums of products kept exact in 160 bits and reduced once: base dot products of up to
    128 terms of all-ones words, the precomputed-factor multiply-add, extension dot products."""
    hc = hostcheck
    hc.hc_gl_dot.restype = u64
    hc.hc_gl_dot.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, u64]
    hc.hc_gl_sub_canon.restype = u64
    hc.hc_gl_sub_canon.argtypes = [u64, u64]
    rnd = random.Random(21)
    for n in (0, 1, 2, 3, 16, 64, 128):
        for mode in ("max", "rand", "mixed"):
            if mode == "max":
                x, y = [2**64 - 1] * n, [2**64 - 1] * n
            elif mode == "rand":
                x, y = [rnd.randrange(2**64) for _ in range(n)], [rnd.randrange(2**64) for _ in range(n)]
            else:
                x = [rnd.choice([0, 1, P - 1, P, 2**64 - 1, 2**32, 2**32 - 1]) for _ in range(n)]
                y = [rnd.choice([0, 1, P - 1, P, 2**64 - 1, 2**32, 2**32 - 1]) for _ in range(n)]
            c = rnd.choice([0, 2**64 - 1, rnd.randrange(2**64)])
            X, Y = np.array(x, dtype=np.uint64), np.array(y, dtype=np.uint64)
            got = hc.hc_gl_dot(X.ctypes.data, Y.ctypes.data, n, c)
            assert got == (sum(a * b for a, b in zip(x, y)) + c) % P
    edge = [0, 1, 2, P - 1, P - 2, 2**32, 2**32 - 1, 2**63]
    for a in edge + [rnd.randrange(P) for _ in range(100)]:
        for b in edge + [rnd.randrange(P) for _ in range(10)]:
            assert hc.hc_gl_sub_canon(a, b) == (a - b) % P
    for _ in range(400):
        r, d, a = ([rnd.choice([rnd.randrange(2**64), 2**64 - 1, P - 1, 0]) for _ in range(2)] for _ in range(3))
        R, D, A, O = (u64 * 2)(*r), (u64 * 2)(*d), (u64 * 2)(*a), (u64 * 2)()
        hc.hc_e2_fma_pre(R, D, A, O)
        assert O[0] == (a[0] + r[0] * d[0] + 7 * r[1] * d[1]) % P
        assert O[1] == (a[1] + r[0] * d[1] + r[1] * d[0]) % P
    for n in (1, 5, 16, 64):
        for mode in ("max", "rand"):
            v = [2**64 - 1] * (4 * n) if mode == "max" else [rnd.randrange(2**64) for _ in range(4 * n)]
            a, b = np.array(v[:2 * n], dtype=np.uint64), np.array(v[2 * n:], dtype=np.uint64)
            O = (u64 * 2)()
            hc.hc_e2_dot(a.ctypes.data, b.ctypes.data, n, O)
            c0 = sum(int(a[2 * i]) * int(b[2 * i]) + 7 * int(a[2 * i + 1]) * int(b[2 * i + 1]) for i in range(n)) % P
            c1 = sum(int(a[2 * i]) * int(b[2 * i + 1]) + int(a[2 * i + 1]) * int(b[2 * i]) for i in range(n)) % P
            assert (O[0], O[1]) == (c0, c1)


def test_almost_goldilocks_extension_lazy_forms(hostcheck):
    """Products of F_q[X]/(X^2 - 3) through exact sums reduced once, loose inputs."""
    hc = hostcheck
    Q = 2**64 - 2**32 - 31
    hc.hc_aext2_fma_pre_base.argtypes = [ctypes.c_void_p, u64, u64, ctypes.c_void_p]
    rnd = random.Random(33)
    pick = lambda: rnd.choice([rnd.randrange(2**64), 2**64 - 1, Q - 1, Q, Q + 1, 0, 1])
    for _ in range(600):
        r, d, a = ([pick() for _ in range(2)] for _ in range(3))
        R, D, A, O = (u64 * 2)(*r), (u64 * 2)(*d), (u64 * 2)(*a), (u64 * 2)()
        hc.hc_aext2_mul_lazy(R, D, O)
        assert (O[0], O[1]) == ((r[0] * d[0] + 3 * r[1] * d[1]) % Q, (r[0] * d[1] + r[1] * d[0]) % Q)
        hc.hc_aext2_fma_pre(R, D, A, O)
        assert (O[0], O[1]) == ((a[0] + r[0] * d[0] + 3 * r[1] * d[1]) % Q, (a[1] + r[0] * d[1] + r[1] * d[0]) % Q)
        hc.hc_aext2_fma_pre_base(R, d[0], a[0], O)
        assert (O[0], O[1]) == ((a[0] + r[0] * d[0]) % Q, (r[1] * d[0]) % Q)


def _e5_mul_int(a, b):
    """Schoolbook product in F_p[X]/(X^5 - 3) with Python integers."""
    t = [0] * 9
    for i in range(5):
        for j in range(5):
            t[i + j] += a[i] * b[j]
    return [(t[k] + (3 * t[k + 5] if k < 4 else 0)) % P for k in range(5)]


def _e5_pow_int(a, e):
    r, b = [1, 0, 0, 0, 0], [x % P for x in a]
    while e:
        if e & 1:
            r = _e5_mul_int(r, b)
        b = _e5_mul_int(b, b)
        e >>= 1
    return r


def test_ext5_oracle_and_host_forms(hostcheck, oracle):
    """Degree-5 extension: the oracle against Python integers (the Frobenius map is x -> x^p, the
    inverse multiplies back to one), and the library's lazy-sum forms against the oracle."""
    from oracle import pyoracle
    rnd = random.Random(21)
    edge = [0, 1, P - 1, P, 2**64 - 1]
    u5 = u64 * 5
    elems = [[rnd.choice(edge) for _ in range(5)] for _ in range(20)] + [[rnd.randrange(2**64) for _ in range(5)] for _ in range(200)]
    for k, a in enumerate(elems):
        b = elems[(k * 7 + 3) % len(elems)]
        want = _e5_mul_int(a, b)
        assert pyoracle.e5_op("mul", a, b) == want
        O = u5()
        hostcheck.hc_e5_mul(u5(*a), u5(*b), O)
        assert list(O) == want
        hostcheck.hc_e5_frobenius(u5(*a), O)
        assert list(O) == pyoracle.e5_op("frobenius", a)
    for a in elems[:4] + elems[20:26]:
        assert pyoracle.e5_op("frobenius", a) == _e5_pow_int(a, P)
    for a in elems[:30] + [[0] * 5, [P] * 5, [5, 0, 0, 0, 0]]:
        inv = pyoracle.e5_op("inv", a)
        O = u5()
        hostcheck.hc_e5_inv(u5(*a), O)
        assert list(O) == inv
        assert _e5_mul_int(a, inv) == ([1, 0, 0, 0, 0] if any(x % P for x in a) else [0] * 5)
        for e in (0, 1, 2, 5, 2**40 + 3, 2**64 - 1):
            want = _e5_pow_int(a, e)
            assert pyoracle.e5_op("pow", a, e=e) == want
            hostcheck.hc_e5_pow(u5(*a), u64(e), O)
            assert list(O) == want
