"""Monolith (width 12) over both fields and the almost-Goldilocks transcript: the CPU oracle
and the library's host code against the reference's known-answer tests, and against each other
on seeded inputs. No GPU needed."""
import ctypes

import numpy as np
import pytest

from matrix_b200.inputs import AGL_Q, GL_P, field_elems, splitmix64
from oracle import pyoracle

# goldilocks-cuda-rs/src/cpu_monolith.rs:237-254: permutation of [0..11]
GL_KAT = [5867581605548782913, 588867029099903233, 6043817495575026667, 805786589926590032,
          9919982299747097782, 6718641691835914685, 7951881005429661950, 15453177927755089358,
          974633365445157727, 9654662171963364206, 6281307445101925412, 13745376999934453119]
# zk-torch-4/src/crypto/monolith.rs:379-392: the same for almost-Goldilocks
AGL_KAT = [0xed82a66d4453e6b3, 0x752b191c23268621, 0x590fab26245cc4e9, 0xa63b2125e2a94a88,
           0x6ab5bea637404df2, 0x6dbeafbbb35f0b77, 0xfc9cdfae47529f13, 0xe57947afed67d70f,
           0x59da37a113e7987e, 0x95662ed82cec7bb2, 0x7429836455d95e39, 0x91861bd52d8c67f2]
# zk-torch-4/src/crypto/monolith.rs:403-408: round constants [1][0..3]
AGL_RC1 = [0xdc5869754490c2c9, 0x8df3ae2a26b03334, 0x6531a374c7fc9b9b, 0x0758fb4f5d864daf]
# zk-torch-4/src/transcript.rs:358-371
TRANSCRIPT_GOLDEN = 0x5df33cda688d0bce
GOLDEN_SCRIPT = [(pyoracle.APPEND, b"a", 1), (pyoracle.APPEND, b"b", 2), (pyoracle.APPEND, b"c", 0xDEADBEEF),
                 (pyoracle.CHALLENGE, b"out", 0)]


def _perm(fn, state):
    s = np.array(state, dtype=np.uint64)
    fn(s.ctypes.data_as(ctypes.c_void_p))
    return [int(x) for x in s]


def test_oracle_gl_monolith_kat(oracle):
    assert _perm(oracle.oracle_gl_monolith_permute, range(12)) == GL_KAT


def test_oracle_agl_monolith_kat(oracle):
    assert _perm(oracle.oracle_agl_monolith_permute, range(12)) == AGL_KAT
    rc = np.zeros(84, dtype=np.uint64)
    oracle.oracle_agl_monolith_rc(rc.ctypes.data_as(ctypes.c_void_p))
    assert [int(x) for x in rc[12:16]] == AGL_RC1
    assert not rc[:12].any() and not rc[72:].any()
    assert all(int(x) < AGL_Q for x in rc) and len(set(int(x) for x in rc[12:72])) == 60


def test_oracle_agl_transcript_golden(oracle):
    out, _ = pyoracle.agl_transcript_run(b"zk-torch-4-test", GOLDEN_SCRIPT)
    assert int(out[0]) == TRANSCRIPT_GOLDEN


def test_host_monolith_kats(hostcheck):
    assert _perm(hostcheck.hc_gl_monolith, range(12)) == GL_KAT
    assert _perm(hostcheck.hc_gl_monolith_host, range(12)) == GL_KAT
    assert _perm(hostcheck.hc_agl_monolith, range(12)) == AGL_KAT


def test_host_monolith_matches_oracle(oracle, hostcheck):
    """Seeded states, including non-canonical words and the large-value case of
    goldilocks-cuda-rs/src/cpu_monolith.rs:257-277 (state[0] = 8, state[1] = p - 8)."""
    cases = [[8, GL_P - 8] + [0] * 10, [GL_P - 1] * 12, [2**64 - 1] * 12, [0] * 12]
    raw = splitmix64(77, 12 * 200).reshape(200, 12)
    cases += [list(map(int, r)) for r in raw]
    for c in cases:
        assert _perm(hostcheck.hc_gl_monolith, c) == _perm(oracle.oracle_gl_monolith_permute, c)
        assert _perm(hostcheck.hc_gl_monolith_host, c) == _perm(oracle.oracle_gl_monolith_permute, c)   # tree tops
        assert _perm(hostcheck.hc_agl_monolith, c) == _perm(oracle.oracle_agl_monolith_permute, c)


def test_host_mds_layer_as_split_convolution(hostcheck):
    """The host form of the MDS layer computes the circulant (first row 7 23 8 26 13 10 9 7 6 22 21 8,
    zk-torch-4/src/crypto/monolith.rs) on 32-bit halves through a split cyclic convolution; it must equal the
    direct sum as integers, extreme halves included."""
    import random
    row = [7, 23, 8, 26, 13, 10, 9, 7, 6, 22, 21, 8]
    rnd = random.Random(31)
    top = 2**32 - 1
    cases = [[0] * 12, [top] * 12, [top if j % 2 else 0 for j in range(12)], [top if j < 6 else 0 for j in range(12)],
             [0 if j < 6 else top for j in range(12)]]
    cases += [[rnd.choice([0, 1, top, top - 1, rnd.randrange(2**32)]) for _ in range(12)] for _ in range(2000)]
    i64 = ctypes.c_int64 * 12
    for x in cases:
        out = i64()
        hostcheck.hc_aglm_circulant12(i64(*x), out)
        assert list(out) == [sum(row[(j - i) % 12] * x[j] for j in range(12)) for i in range(12)]


def test_agl_reduce_limb_sums(hostcheck):
    hostcheck.hc_agl_reduce_limb_sums.restype = ctypes.c_uint64
    hostcheck.hc_agl_reduce_limb_sums.argtypes = [ctypes.c_uint64, ctypes.c_uint64]
    rng = np.random.default_rng(5)
    vals = [(0, 0), (2**40 - 1, 2**40 - 1), (161 * (2**32 - 1), 161 * (2**32 - 1))]
    vals += [(int(a), int(b)) for a, b in rng.integers(0, 2**40, size=(2000, 2), dtype=np.uint64)]
    for L, H in vals:
        assert hostcheck.hc_agl_reduce_limb_sums(L, H) % AGL_Q == (L + (H << 32)) % AGL_Q


def _lib_transcript(lib, init, script):
    h = ctypes.c_void_p()
    assert lib.agl_transcript_create(init, len(init), ctypes.byref(h)) == 0
    outs = []
    for kind, label, v in script:
        if kind == pyoracle.APPEND:
            assert lib.agl_transcript_append_u64(h, label, len(label), v) == 0
        elif kind == pyoracle.CHALLENGE:
            o = ctypes.c_uint64()
            assert lib.agl_transcript_challenge_scalar(h, label, len(label), ctypes.byref(o)) == 0
            outs.append(o.value)
        else:
            f = ctypes.c_void_p()
            assert lib.agl_transcript_fork(h, label, len(label), v, ctypes.byref(f)) == 0
            lib.agl_transcript_destroy(h)
            h = f
    st = np.zeros(12, dtype=np.uint64)
    assert lib.agl_transcript_state(h, st.ctypes.data) == 0
    lib.agl_transcript_destroy(h)
    return outs, st


@pytest.fixture(scope="module")
def agl_lib():
    from matrix_b200.ffi import load_agl
    return load_agl()


def test_library_transcript_golden(agl_lib):
    """The C-ABI transcript (host code, no device work) reproduces the reference's golden squeeze."""
    outs, _ = _lib_transcript(agl_lib, b"zk-torch-4-test", GOLDEN_SCRIPT)
    assert outs == [TRANSCRIPT_GOLDEN]
    s = np.arange(12, dtype=np.uint64)
    assert agl_lib.agl_monolith_permute_host(s.ctypes.data) == 0
    assert [int(x) for x in s] == AGL_KAT
    rc = np.zeros(84, dtype=np.uint64)
    assert agl_lib.agl_monolith_round_constants(rc.ctypes.data) == 0
    assert [int(x) for x in rc[12:16]] == AGL_RC1


def test_library_transcript_matches_oracle(agl_lib):
    """Long scripted runs: labels of several lengths (empty too), non-canonical values, forks,
    challenges across duplexing boundaries."""
    rng = np.random.default_rng(11)
    labels = [b"", b"x", b"round_message", b"challenge", b"ft_bucket0", b"a-much-longer-label-than-the-rate"]
    for trial in range(8):
        script = []
        for _ in range(120):
            kind = int(rng.choice([pyoracle.APPEND, pyoracle.APPEND, pyoracle.CHALLENGE, pyoracle.FORK], p=[.4, .2, .3, .1]))
            v = int(rng.integers(0, 2**64, dtype=np.uint64)) if kind == pyoracle.APPEND else int(rng.integers(0, 1000))
            script.append((kind, labels[int(rng.integers(0, len(labels)))], v))
        want, want_state = pyoracle.agl_transcript_run(b"trial%d" % trial, script)
        got, got_state = _lib_transcript(agl_lib, b"trial%d" % trial, script)
        assert got == [int(x) for x in want]
        assert np.array_equal(got_state, want_state)


def test_transcript_properties(agl_lib):
    """The behavioural tests of zk-torch-4/src/transcript.rs:252-345 on the library transcript."""
    A, C, F = pyoracle.APPEND, pyoracle.CHALLENGE, pyoracle.FORK
    run = lambda init, sc: _lib_transcript(agl_lib, init, sc)[0]
    assert run(b"test", [(A, b"val", 42), (C, b"c", 0)]) == run(b"test", [(A, b"val", 42), (C, b"c", 0)])
    assert run(b"test", [(A, b"val", 42), (C, b"c", 0)]) != run(b"test", [(A, b"val", 43), (C, b"c", 0)])
    assert run(b"a", [(C, b"c", 0)]) != run(b"b", [(C, b"c", 0)])
    assert (run(b"x", [(A, b"ab", 0), (A, b"c", 0), (C, b"", 0)]) != run(b"x", [(A, b"a", 0), (A, b"bc", 0), (C, b"", 0)]))
    two = run(b"test", [(C, b"x", 0), (C, b"x", 0)])
    assert two[0] != two[1]
    many = run(b"test", [(C, b"x", 0)] + [(C, b"", 0)] * 23)
    assert len(set(many)) == 24
    after = run(b"test", [(C, b"a", 0), (A, b"b", 7), (C, b"c", 0)])[-1]
    assert after != run(b"test", [(C, b"a", 0), (C, b"c", 0)])[-1]
    assert run(b"root", [(F, b"fam", 0), (C, b"c", 0)]) != run(b"root", [(F, b"fam", 1), (C, b"c", 0)])
    assert run(b"root", [(F, b"dag_partition", 3), (C, b"c", 0)]) != run(b"root", [(F, b"open_reducer", 3), (C, b"c", 0)])
    assert run(b"root", [(F, b"ft_bucket", 0), (C, b"c", 0)]) != run(b"root", [(F, b"ft_bucket0", 0), (C, b"c", 0)])
    # values are reduced mod q before absorption
    assert run(b"t", [(A, b"v", AGL_Q + 5), (C, b"c", 0)]) == run(b"t", [(A, b"v", 5), (C, b"c", 0)])
