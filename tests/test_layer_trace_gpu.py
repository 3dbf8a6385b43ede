"""Einsum proofs of the decoder-layer trace on the GPU at small sizes: for each kind of equation of
the layer the proof must pass the sumcheck verifier against the claim computed directly (the output
tensor with Python integers, its multilinear extension evaluated at the output point), and the final
evaluation must equal eq(shared point, challenges) times the operands' final evaluations."""
import ctypes
import itertools

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from matrix_b200.inputs import AGL_Q, field_elems
from matrix_b200.layer_trace import EinsumPlan, LayerProver, _bits, synthetic_operand

pytestmark = pytest.mark.gpu
Q = AGL_Q


def _mul(a, b):
    return ((a[0] * b[0] + 3 * a[1] * b[1]) % Q, (a[0] * b[1] + a[1] * b[0]) % Q)


def _mle(values, point):
    """Multilinear extension of base-field values at extension challenges, low variable first."""
    t = [(v % Q, 0) for v in values]
    for r in point:
        t = [tuple((a[k] + _mul(r, ((b[0] - a[0]) % Q, (b[1] - a[1]) % Q))[k]) % Q for k in range(2))
             for a, b in zip(t[0::2], t[1::2])]
    return t[0]


def _einsum_int(equation, dims, operands):
    lhs, out = equation.split("->")
    ins = lhs.split(",")
    letters = sorted(set("".join(ins)))
    size = {c: 1 << dims[c] for c in letters}

    def flat(term, idx):
        f = 0
        for c in term:
            f = f * size[c] + idx[c]
        return f
    res = [0] * (1 << sum(dims[c] for c in out))
    for combo in itertools.product(*[range(size[c]) for c in letters]):
        idx = dict(zip(letters, combo))
        p = 1
        for term, op in zip(ins, operands):
            p = p * int(op[flat(term, idx)]) % Q
        o = flat(out, idx)
        res[o] = (res[o] + p) % Q
    return res


CASES = [("si,ij->sj", dict(s=2, i=3, j=2)), ("hsd,htd->hst", dict(h=1, s=2, t=2, d=2)),
         ("hst,htd->hsd", dict(h=2, s=1, t=2, d=2)), ("si,si->si", dict(s=2, i=3)), ("hst,z->hst", dict(h=1, s=2, t=2, z=0)),
         ("si,ij->sj", dict(s=3, i=4, j=5))]


@pytest.mark.parametrize("equation,dims", CASES, ids=[c[0] + str(i) for i, c in enumerate(CASES)])
def test_einsum_proof_verifies_against_direct_claim(equation, dims):
    lib = load_agl()
    prover = LayerProver(lib)
    pl = EinsumPlan(equation, dims)
    ops = [synthetic_operand(40 + k, sum(dims[c] for c in t)) for k, t in enumerate(pl.inputs)]
    bufs = [DeviceBuffer.from_numpy(lib, o) for o in ops]
    n_out = sum(dims[c] for c in pl.out)
    point = field_elems(77, 2 * max(n_out, 1), Q)[:2 * n_out].reshape(n_out, 2)
    h = ctypes.c_void_p()
    assert lib.agl_transcript_create(b"layer", 5, ctypes.byref(h)) == 0
    msgs, ch, fe, fin = prover.prove_einsum(equation, dims, [b.ptr for b in bufs], point, h)
    lib.agl_transcript_destroy(h)
    pt = [(int(a), int(b)) for a, b in point]
    claim = _mle(_einsum_int(equation, dims, ops), pt)
    d, rounds = len(pl.inputs) + 1, pl.rounds
    v = ctypes.c_void_p()
    assert lib.agl_transcript_create(b"layer", 5, ctypes.byref(v)) == 0
    ok = ctypes.c_int(0)
    cl = np.array(claim, dtype=np.uint64)
    assert lib.agl_sumcheck_verify_ffi(msgs.ctypes.data if rounds else None, fin.ctypes.data, cl.ctypes.data, d, rounds, v, None,
                                       ctypes.byref(ok)) == 0
    lib.agl_transcript_destroy(v)
    assert ok.value == 1
    # the last table is eq(shared point, first challenges): its final evaluation by the closed form
    out_bits = _bits(pl.out, dims)
    eq = (1, 0)
    for k, var in enumerate(pl.shared):
        r, x = pt[out_bits.index(var)], (int(ch[2 * k]), int(ch[2 * k + 1]))
        one_r, one_x = ((1 - r[0]) % Q, (-r[1]) % Q), ((1 - x[0]) % Q, (-x[1]) % Q)
        t1, t2 = _mul(r, x), _mul(one_r, one_x)
        eq = _mul(eq, ((t1[0] + t2[0]) % Q, (t1[1] + t2[1]) % Q))
    assert (int(fe[2 * (d - 1)]), int(fe[2 * (d - 1) + 1])) == eq
    prod = (1, 0)
    for i in range(d):
        prod = _mul(prod, (int(fe[2 * i]), int(fe[2 * i + 1])))
    assert (int(fin[0]), int(fin[1])) == prod


NATIVE_CASES = CASES + [("si,ij->sj", dict(s=4, i=7, j=6)), ("hsd,htd->hst", dict(h=2, s=3, t=3, d=4)),
                        ("hst,htd->hsd", dict(h=2, s=3, t=4, d=3)), ("si,si->si", dict(s=5, i=8))]


@pytest.mark.parametrize("equation,dims", NATIVE_CASES, ids=[c[0] + str(i) for i, c in enumerate(NATIVE_CASES)])
def test_one_call_per_einsum_equals_the_step_by_step_sequence(equation, dims):
    """agl_einsum_prove_device_ffi (the whole device sequence inside the library) against the same sequence issued
    call by call from Python, bit for bit, on two einsums sharing one transcript."""
    from matrix_b200.layer_trace import prove_einsum_native
    lib = load_agl()
    prover = LayerProver(lib)
    pl = EinsumPlan(equation, dims)
    ops = [synthetic_operand(140 + k, sum(dims[c] for c in t)) for k, t in enumerate(pl.inputs)]
    bufs = [DeviceBuffer.from_numpy(lib, o) for o in ops]
    n_out = sum(dims[c] for c in pl.out)
    results = []
    for fn in (lambda *a: prover.prove_einsum(*a), lambda *a: prove_einsum_native(prover, *a)):
        h = ctypes.c_void_p()
        assert lib.agl_transcript_create(b"layer", 5, ctypes.byref(h)) == 0
        outs = []
        for seed in (77, 78):
            point = field_elems(seed, 2 * max(n_out, 1), Q)[:2 * n_out].reshape(n_out, 2)
            outs.append(fn(equation, dims, [b.ptr for b in bufs], point, h))
        st = np.zeros(12, dtype=np.uint64)
        assert lib.agl_transcript_state(h, st.ctypes.data) == 0
        lib.agl_transcript_destroy(h)
        results.append((outs, st))
    (a_outs, a_st), (b_outs, b_st) = results
    assert np.array_equal(a_st, b_st)
    for x, y in zip(a_outs, b_outs):
        for u, v in zip(x, y):
            assert np.array_equal(u, v)
