"""Element-wise batch operations of both libraries against Python integers (bit-exact), including
non-canonical inputs, zero divisors, the empty batch and argument errors; stream and copy helpers."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl, load_gl
from matrix_b200.inputs import AGL_Q, GL_P, splitmix64

pytestmark = pytest.mark.gpu
N = 1000


def _inputs(seed, words, p):
    v = splitmix64(seed, words)  # raw 64-bit words: representatives at or above the modulus occur
    v[:6] = [0, 1, p - 1, p, 2**64 - 1, p + 1]
    return v


def _ext_mul(a, b, p, w):
    return ((a[0] * b[0] + w * a[1] * b[1]) % p, (a[0] * b[1] + a[1] * b[0]) % p)


def _ext_pow(a, e, p, w):
    r, b = (1, 0), a
    while e:
        if e & 1:
            r = _ext_mul(r, b, p, w)
        b = _ext_mul(b, b, p, w)
        e >>= 1
    return r


def _ext_inv(a, p, w):
    n = (a[0] * a[0] - w * a[1] * a[1]) % p
    ni = pow(n, p - 2, p)
    return (a[0] * ni % p, (-a[1]) * ni % p)


CASES = [
    ("gl", load_gl, GL_P, 7,
     dict(add="gl_batch_add", sub="gl_batch_sub", mul="gl_batch_mul", div="gl_batch_div", inv="gl_batch_inverse",
          neg="gl_batch_neg", sq="gl_batch_square", dbl="gl_batch_double", muls="gl_batch_mul_scalar", exp="gl_batch_exp",
          eadd="ext2_batch_add_ffi", esub="ext2_batch_sub_ffi", emul="ext2_batch_mul_ffi", einv="ext2_batch_inverse_ffi",
          eneg="ext2_batch_neg_ffi", esq="ext2_batch_square_ffi", efrob="ext2_batch_frobenius_ffi",
          econj="ext2_batch_conjugate_ffi", emuls="ext2_batch_mul_scalar_ffi", eexp="ext2_batch_exp_ffi",
          eacc="ext2_scale_accumulate_ffi", lift="gl_to_ext2_batch_ffi", proj="ext2_to_gl_batch_ffi",
          zero="gl_zero_buffer", perm="bit_permute_gl_ffi")),
    ("agl", load_agl, AGL_Q, 3,
     dict(add="agl_batch_add_ffi", sub="agl_batch_sub_ffi", mul="agl_batch_mul_ffi", div="agl_batch_div_ffi",
          inv="agl_batch_inverse_ffi", neg="agl_batch_neg_ffi", sq="agl_batch_square_ffi", dbl="agl_batch_double_ffi",
          muls="agl_batch_mul_scalar_ffi", exp="agl_batch_exp_ffi",
          eadd="aext2_batch_add_ffi", esub="aext2_batch_sub_ffi", emul="aext2_batch_mul_ffi", einv="aext2_batch_inverse_ffi",
          eneg="aext2_batch_neg_ffi", esq="aext2_batch_square_ffi", efrob="aext2_batch_frobenius_ffi",
          econj="aext2_batch_conjugate_ffi", emuls="aext2_batch_mul_scalar_ffi", eexp="aext2_batch_exp_ffi",
          eacc="aext2_scale_accumulate_ffi", lift="agl_to_aext2_batch_ffi", proj="aext2_to_agl_batch_ffi",
          zero="agl_zero_buffer_ffi", perm="agl_bit_permute_ffi")),
]


@pytest.mark.parametrize("name,loader,p,w,fn", CASES, ids=[c[0] for c in CASES])
def test_base_field_ops(name, loader, p, w, fn):
    lib = loader()
    a, b = _inputs(1, N, p), _inputs(2, N, p)
    b[10] = 0
    da, db, dr = DeviceBuffer.from_numpy(lib, a), DeviceBuffer.from_numpy(lib, b), DeviceBuffer(lib, 8 * N)
    A, B = [int(x) for x in a], [int(x) for x in b]
    run2 = lambda f: (getattr(lib, fn[f])(da.ptr, db.ptr, dr.ptr, N), lib.cuda_device_synchronize(), [int(x) for x in dr.to_numpy()])
    run1 = lambda f: (getattr(lib, fn[f])(da.ptr, dr.ptr, N), lib.cuda_device_synchronize(), [int(x) for x in dr.to_numpy()])
    rc, _, got = run2("add"); assert rc == 0 and got == [(x + y) % p for x, y in zip(A, B)]
    rc, _, got = run2("sub"); assert rc == 0 and got == [(x - y) % p for x, y in zip(A, B)]
    rc, _, got = run2("mul"); assert rc == 0 and got == [(x * y) % p for x, y in zip(A, B)]
    rc, _, got = run2("div"); assert rc == 0 and got == [(x * pow(y % p, p - 2, p)) % p for x, y in zip(A, B)]
    rc, _, got = run1("inv"); assert rc == 0 and got == [pow(x % p, p - 2, p) for x in A]
    rc, _, got = run1("neg"); assert rc == 0 and got == [(-x) % p for x in A]
    rc, _, got = run1("sq"); assert rc == 0 and got == [(x * x) % p for x in A]
    rc, _, got = run1("dbl"); assert rc == 0 and got == [(2 * x) % p for x in A]
    for s in (0, 1, p - 1, 2**64 - 1, 0x123456789ABCDEF):
        assert getattr(lib, fn["muls"])(s, da.ptr, dr.ptr, N) == 0
        lib.cuda_device_synchronize()
        assert [int(x) for x in dr.to_numpy()] == [(s * x) % p for x in A]
    for e in (0, 1, 2, 7, 2**64 - 1):
        assert getattr(lib, fn["exp"])(da.ptr, e, dr.ptr, N) == 0
        lib.cuda_device_synchronize()
        assert [int(x) for x in dr.to_numpy()] == [pow(x % p, e, p) for x in A]
    # empty batch and bad arguments
    assert getattr(lib, fn["add"])(da.ptr, db.ptr, dr.ptr, 0) == 0
    assert getattr(lib, fn["add"])(da.ptr, None, dr.ptr, 4) != 0
    assert getattr(lib, fn["neg"])(da.ptr, dr.ptr, -1) != 0


@pytest.mark.parametrize("name,loader,p,w,fn", CASES, ids=[c[0] for c in CASES])
def test_extension_ops(name, loader, p, w, fn):
    lib = loader()
    a, b = _inputs(3, 2 * N, p), _inputs(4, 2 * N, p)
    a[20:22] = 0
    da, db, dr = DeviceBuffer.from_numpy(lib, a), DeviceBuffer.from_numpy(lib, b), DeviceBuffer(lib, 16 * N)
    A = [(int(a[2 * i]) % p, int(a[2 * i + 1]) % p) for i in range(N)]
    B = [(int(b[2 * i]) % p, int(b[2 * i + 1]) % p) for i in range(N)]
    pairs = lambda arr: [(int(arr[2 * i]), int(arr[2 * i + 1])) for i in range(N)]

    def run(f, *args):
        assert getattr(lib, fn[f])(*args) == 0
        lib.cuda_device_synchronize()
        return pairs(dr.to_numpy())

    assert run("eadd", da.ptr, db.ptr, dr.ptr, N) == [((x[0] + y[0]) % p, (x[1] + y[1]) % p) for x, y in zip(A, B)]
    assert run("esub", da.ptr, db.ptr, dr.ptr, N) == [((x[0] - y[0]) % p, (x[1] - y[1]) % p) for x, y in zip(A, B)]
    assert run("emul", da.ptr, db.ptr, dr.ptr, N) == [_ext_mul(x, y, p, w) for x, y in zip(A, B)]
    assert run("einv", da.ptr, dr.ptr, N) == [_ext_inv(x, p, w) for x in A]
    assert run("eneg", da.ptr, dr.ptr, N) == [((-x[0]) % p, (-x[1]) % p) for x in A]
    assert run("esq", da.ptr, dr.ptr, N) == [_ext_mul(x, x, p, w) for x in A]
    conj = [(x[0], (-x[1]) % p) for x in A]
    assert run("econj", da.ptr, dr.ptr, N) == conj
    assert run("efrob", da.ptr, dr.ptr, N) == conj
    assert conj[:8] == [_ext_pow(x, p, p, w) for x in A[:8]]  # Frobenius is x -> x^p
    for s in (0, 5, p - 1, 2**64 - 1):
        assert run("emuls", s, da.ptr, dr.ptr, N) == [((s * x[0]) % p, (s * x[1]) % p) for x in A]
    for e in (0, 1, 5, 2**40 + 3):
        assert run("eexp", da.ptr, e, dr.ptr, N) == [_ext_pow(x, e, p, w) for x in A]
    # acc += scalar * src
    assert lib.cuda_memcpy_dtod(dr.ptr, db.ptr, 16 * N) == 0
    s = (0xDEADBEEFCAFE, p - 2)
    got = run("eacc", s[0], s[1], da.ptr, dr.ptr, N)
    assert got == [tuple((y[i] + _ext_mul(s, x, p, w)[i]) % p for i in range(2)) for x, y in zip(A, B)]
    # lift and projection
    assert getattr(lib, fn["lift"])(da.ptr, dr.ptr, N) == 0
    lib.cuda_device_synchronize()
    assert pairs(dr.to_numpy()) == [(int(a[i]) % p, 0) for i in range(N)]
    d1 = DeviceBuffer(lib, 8 * N)
    assert getattr(lib, fn["proj"])(da.ptr, d1.ptr, N) == 0
    lib.cuda_device_synchronize()
    assert [int(x) for x in d1.to_numpy()] == [x[0] for x in A]
    assert getattr(lib, fn["zero"])(d1.ptr, N) == 0
    lib.cuda_device_synchronize()
    assert not d1.to_numpy().any()


@pytest.mark.parametrize("name,loader,p,w,fn", CASES, ids=[c[0] for c in CASES])
def test_bit_permute(name, loader, p, w, fn):
    lib = loader()
    n_bits = 11
    total = 1 << n_bits
    data = splitmix64(9, total)
    perm = np.random.default_rng(3).permutation(n_bits).astype(np.int32)
    d_in, d_out = DeviceBuffer.from_numpy(lib, data), DeviceBuffer(lib, 8 * total)
    d_perm = DeviceBuffer.from_numpy(lib, perm.view(np.uint32).astype(np.uint32))
    assert getattr(lib, fn["perm"])(d_in.ptr, d_out.ptr, d_perm.ptr, n_bits, total) == 0
    lib.cuda_device_synchronize()
    exp = np.empty_like(data)
    for new in range(total):
        old = 0
        for b in range(n_bits):
            if (new >> b) & 1:
                old |= 1 << int(perm[b])
        exp[new] = data[old]
    assert np.array_equal(d_out.to_numpy(), exp)
    assert getattr(lib, fn["perm"])(d_in.ptr, d_out.ptr, d_perm.ptr, 40, total) != 0


def test_streams_copies_and_pool():
    lib = load_agl()
    n = 1 << 16
    data = splitmix64(17, n)
    d0, d1 = DeviceBuffer.from_numpy(lib, data), DeviceBuffer(lib, 8 * n)
    st = ctypes.c_void_p()
    assert lib.cuda_stream_create(ctypes.byref(st)) == 0
    assert lib.cuda_memcpy_dtod_async(d1.ptr, d0.ptr, 8 * n, st) == 0
    assert lib.cuda_stream_synchronize(st) == 0
    assert np.array_equal(d1.to_numpy(), data)
    assert lib.cuda_memset(d1.ptr, 0, 8 * n) == 0
    assert not d1.to_numpy().any()
    host = np.ascontiguousarray(data[::-1])
    assert lib.cuda_memcpy_htod_async(d1.ptr, host.ctypes.data, 8 * n, st) == 0
    assert lib.cuda_stream_synchronize(st) == 0
    assert np.array_equal(d1.to_numpy(), host)
    assert lib.cuda_stream_destroy(st) == 0
    dev = ctypes.c_int()
    assert lib.cuda_get_device(ctypes.byref(dev)) == 0
    assert lib.cuda_memcpy_peer(d1.ptr, dev.value, d0.ptr, dev.value, 8 * n) == 0  # same device: a plain copy
    assert lib.cuda_sync_mine() == 0
    assert np.array_equal(d1.to_numpy(), data)
    # staged copies: larger than one 64 MiB chunk, ragged tail
    words = (80 << 20) // 8 + 5
    big = splitmix64(23, words)
    dbig = DeviceBuffer(lib, 8 * words)
    assert lib.agl_h2d_staged(dbig.ptr, big.ctypes.data, 8 * words) == 0
    back = np.zeros(words, dtype=np.uint64)
    assert lib.agl_d2h_staged(back.ctypes.data, dbig.ptr, 8 * words) == 0
    assert np.array_equal(back, big)
    assert lib.agl_h2d_staged(dbig.ptr, big.ctypes.data, 0) == 0
    assert lib.agl_cached_bytes() >= 0
    assert lib.cuda_pool_trim(0) == 0
    assert b"no error" in lib.agl_cuda_error_string(0)


def test_ext5_ops():
    """Degree-5 extension of Goldilocks (five words per element): products, inverses, powers and the
    Frobenius map against the CPU oracle; coefficient-wise operations against Python integers."""
    from oracle import pyoracle
    lib, p, n = load_gl(), GL_P, 300
    a, b = _inputs(11, 5 * n, p), _inputs(12, 5 * n, p)
    a[10:15] = 0            # a zero element
    a[15:20] = p            # zero as a non-canonical representative
    a[20:25] = [9, 0, 0, 0, 0]
    da, db, dr = DeviceBuffer.from_numpy(lib, a), DeviceBuffer.from_numpy(lib, b), DeviceBuffer(lib, 40 * n)
    A = [[int(x) for x in a[5 * i:5 * i + 5]] for i in range(n)]
    B = [[int(x) for x in b[5 * i:5 * i + 5]] for i in range(n)]
    elems = lambda arr: [[int(x) for x in arr[5 * i:5 * i + 5]] for i in range(n)]

    def run(f, *args):
        assert getattr(lib, f)(*args) == 0
        lib.cuda_device_synchronize()
        return elems(dr.to_numpy())

    assert run("ext5_batch_add_ffi", da.ptr, db.ptr, dr.ptr, n) == [[(x + y) % p for x, y in zip(u, v)] for u, v in zip(A, B)]
    assert run("ext5_batch_sub_ffi", da.ptr, db.ptr, dr.ptr, n) == [[(x - y) % p for x, y in zip(u, v)] for u, v in zip(A, B)]
    assert run("ext5_batch_neg_ffi", da.ptr, dr.ptr, n) == [[(-x) % p for x in u] for u in A]
    for s in (0, 3, p - 1, 2**64 - 1):
        assert run("ext5_batch_mul_scalar_ffi", s, da.ptr, dr.ptr, n) == [[(s * x) % p for x in u] for u in A]
    assert run("ext5_batch_mul_ffi", da.ptr, db.ptr, dr.ptr, n) == [pyoracle.e5_op("mul", u, v) for u, v in zip(A, B)]
    assert run("ext5_batch_square_ffi", da.ptr, dr.ptr, n) == [pyoracle.e5_op("mul", u, u) for u in A]
    assert run("ext5_batch_frobenius_ffi", da.ptr, dr.ptr, n) == [pyoracle.e5_op("frobenius", u) for u in A]
    inv = run("ext5_batch_inverse_ffi", da.ptr, dr.ptr, n)
    assert inv == [pyoracle.e5_op("inv", u) for u in A]
    assert inv[2] == inv[3] == [0] * 5 and inv[4] == [pow(9, p - 2, p), 0, 0, 0, 0]
    for e in (0, 1, 5, 2**40 + 3, 2**64 - 1):
        assert run("ext5_batch_exp_ffi", da.ptr, e, dr.ptr, n) == [pyoracle.e5_op("pow", u, e=e) for u in A]
    # in place: result over the first operand
    dc = DeviceBuffer.from_numpy(lib, a)
    assert lib.ext5_batch_mul_ffi(dc.ptr, db.ptr, dc.ptr, n) == 0
    lib.cuda_device_synchronize()
    assert elems(dc.to_numpy()) == [pyoracle.e5_op("mul", u, v) for u, v in zip(A, B)]
    # lift and projection
    assert run("gl_to_ext5_batch_ffi", da.ptr, dr.ptr, n) == [[int(a[i]) % p, 0, 0, 0, 0] for i in range(n)]
    d1 = DeviceBuffer(lib, 8 * n)
    assert lib.ext5_to_gl_batch_ffi(da.ptr, d1.ptr, n) == 0
    lib.cuda_device_synchronize()
    assert [int(x) for x in d1.to_numpy()] == [u[0] % p for u in A]
    # empty batch and bad arguments
    assert lib.ext5_batch_mul_ffi(da.ptr, db.ptr, dr.ptr, 0) == 0
    assert lib.ext5_batch_mul_ffi(da.ptr, None, dr.ptr, 4) != 0
    assert lib.ext5_batch_inverse_ffi(da.ptr, dr.ptr, -1) != 0
