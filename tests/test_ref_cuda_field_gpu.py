"""Element-wise field operations of both libraries against the reference's own CUDA wrappers.

Base field, quadratic extension (both fields) and the degree-5 extension of
Goldilocks (goldilocks-cuda-rs/src/ffi.rs:230-281): every batch entry point the
reference exports runs on the same seeded device inputs in the reference's
library (compiled unchanged, oracle/Makefile target refcuda) and in ours; the
outputs must be equal after bringing the reference's words into [0, p).
Inputs are canonical and non-zero: the reference's kernels define nothing for
other representatives or for the inverse of zero (those cases are pinned
against Python integers in test_batch_ops_gpu.py).
"""
import numpy as np
import pytest

from matrix_b200.ffi import load_agl, load_gl
from matrix_b200.inputs import splitmix64
from .refcuda import AGL_Q, GL_P, Buf, canon, ref_agl, ref_gl

pytestmark = pytest.mark.gpu
N = 1537   # not a multiple of any block size


def _elems(seed, words, p):
    v = splitmix64(seed, words) % np.uint64(p)
    v[v == 0] = 1
    return v


def _run(lib, name, width_in, width_out, p, arity, scalar=None, exponent=None):
    """One call of `name` on N elements of `width_in` words; returns the output words, or None when the
    library does not export the name."""
    fn = getattr(lib, name, None)
    if fn is None:
        return None
    a = Buf.of(lib, _elems(11, width_in * N, p))
    b = Buf.of(lib, _elems(12, width_in * N, p))
    r = Buf(lib, 8 * width_out * N)
    if scalar is not None:
        rc = fn(scalar, a.ptr, r.ptr, N)
    elif exponent is not None:
        rc = fn(a.ptr, exponent, r.ptr, N)
    elif arity == 2:
        rc = fn(a.ptr, b.ptr, r.ptr, N)
    else:
        rc = fn(a.ptr, r.ptr, N)
    assert rc == 0, name
    return canon(r.get(count=width_out * N), p)


def _compare(ours, ref, name, *args, **kw):
    want = _run(ref, name, *args, **kw)
    if want is None:
        pytest.skip("%s is not exported by the reference" % name)
    got = _run(ours, name, *args, **kw)
    bad = np.nonzero(got != want)[0]
    assert len(bad) == 0, "%s differs from the reference at word %d" % (name, bad[0])


GL_OPS = [
    # name, words per input element, words per output element, operands
    ("gl_batch_add", 1, 1, 2), ("gl_batch_sub", 1, 1, 2), ("gl_batch_mul", 1, 1, 2), ("gl_batch_div", 1, 1, 2),
    ("gl_batch_inverse", 1, 1, 1), ("gl_batch_neg", 1, 1, 1), ("gl_batch_square", 1, 1, 1), ("gl_batch_double", 1, 1, 1),
    ("ext2_batch_add_ffi", 2, 2, 2), ("ext2_batch_sub_ffi", 2, 2, 2), ("ext2_batch_mul_ffi", 2, 2, 2),
    ("ext2_batch_inverse_ffi", 2, 2, 1), ("ext2_batch_neg_ffi", 2, 2, 1), ("ext2_batch_square_ffi", 2, 2, 1),
    ("ext2_batch_frobenius_ffi", 2, 2, 1), ("ext2_batch_conjugate_ffi", 2, 2, 1),
    ("gl_to_ext2_batch_ffi", 1, 2, 1), ("ext2_to_gl_batch_ffi", 2, 1, 1),
    ("ext5_batch_add_ffi", 5, 5, 2), ("ext5_batch_sub_ffi", 5, 5, 2), ("ext5_batch_mul_ffi", 5, 5, 2),
    ("ext5_batch_inverse_ffi", 5, 5, 1), ("ext5_batch_neg_ffi", 5, 5, 1), ("ext5_batch_square_ffi", 5, 5, 1),
    ("ext5_batch_frobenius_ffi", 5, 5, 1), ("gl_to_ext5_batch_ffi", 1, 5, 1), ("ext5_to_gl_batch_ffi", 5, 1, 1),
]
GL_SCALAR = [("gl_batch_mul_scalar", 1), ("ext2_batch_mul_scalar_ffi", 2), ("ext5_batch_mul_scalar_ffi", 5)]
GL_EXP = [("gl_batch_exp", 1), ("ext2_batch_exp_ffi", 2), ("ext5_batch_exp_ffi", 5)]

AGL_OPS = [
    ("agl_batch_add_ffi", 1, 1, 2), ("agl_batch_sub_ffi", 1, 1, 2), ("agl_batch_mul_ffi", 1, 1, 2), ("agl_batch_div_ffi", 1, 1, 2),
    ("agl_batch_inverse_ffi", 1, 1, 1), ("agl_batch_neg_ffi", 1, 1, 1), ("agl_batch_square_ffi", 1, 1, 1),
    ("agl_batch_double_ffi", 1, 1, 1),
    ("aext2_batch_add_ffi", 2, 2, 2), ("aext2_batch_sub_ffi", 2, 2, 2), ("aext2_batch_mul_ffi", 2, 2, 2),
    ("aext2_batch_inverse_ffi", 2, 2, 1), ("aext2_batch_neg_ffi", 2, 2, 1), ("aext2_batch_square_ffi", 2, 2, 1),
    ("aext2_batch_frobenius_ffi", 2, 2, 1), ("aext2_batch_conjugate_ffi", 2, 2, 1),
    ("agl_to_aext2_batch_ffi", 1, 2, 1), ("aext2_to_agl_batch_ffi", 2, 1, 1),
]
AGL_SCALAR = [("agl_batch_mul_scalar_ffi", 1), ("aext2_batch_mul_scalar_ffi", 2)]
AGL_EXP = [("agl_batch_exp_ffi", 1), ("aext2_batch_exp_ffi", 2)]


@pytest.fixture(scope="module")
def gl_libs():
    ours = load_gl()
    assert ours.goldilocks_cuda_init() == 0
    return ours, ref_gl()


@pytest.fixture(scope="module")
def agl_libs():
    ours = load_agl()
    assert ours.almost_goldilocks_cuda_init() == 0
    return ours, ref_agl()


@pytest.mark.parametrize("name,win,wout,arity", GL_OPS, ids=[o[0] for o in GL_OPS])
def test_goldilocks_batch_ops(gl_libs, name, win, wout, arity):
    _compare(*gl_libs, name, win, wout, GL_P, arity)


@pytest.mark.parametrize("name,width", GL_SCALAR, ids=[o[0] for o in GL_SCALAR])
@pytest.mark.parametrize("scalar", [1, 5, GL_P - 1, 0x0123456789ABCDEF])
def test_goldilocks_scalar_products(gl_libs, name, width, scalar):
    _compare(*gl_libs, name, width, width, GL_P, 1, scalar=scalar)


@pytest.mark.parametrize("name,width", GL_EXP, ids=[o[0] for o in GL_EXP])
@pytest.mark.parametrize("exponent", [1, 5, 2**40 + 3])
def test_goldilocks_powers(gl_libs, name, width, exponent):
    _compare(*gl_libs, name, width, width, GL_P, 1, exponent=exponent)


@pytest.mark.parametrize("name,win,wout,arity", AGL_OPS, ids=[o[0] for o in AGL_OPS])
def test_almost_goldilocks_batch_ops(agl_libs, name, win, wout, arity):
    _compare(*agl_libs, name, win, wout, AGL_Q, arity)


@pytest.mark.parametrize("name,width", AGL_SCALAR, ids=[o[0] for o in AGL_SCALAR])
@pytest.mark.parametrize("scalar", [1, 5, AGL_Q - 1, 0x0123456789ABCDEF])
def test_almost_goldilocks_scalar_products(agl_libs, name, width, scalar):
    _compare(*agl_libs, name, width, width, AGL_Q, 1, scalar=scalar)


@pytest.mark.parametrize("name,width", AGL_EXP, ids=[o[0] for o in AGL_EXP])
@pytest.mark.parametrize("exponent", [1, 5, 2**40 + 3])
def test_almost_goldilocks_powers(agl_libs, name, width, exponent):
    _compare(*agl_libs, name, width, width, AGL_Q, 1, exponent=exponent)
