"""Module commitment over F_q[Y]/(Y^4096 + 1): the oracle's SHAKE256 key expansion against the
reference's known answer and hashlib, and the library's host-compiled expansion against the oracle."""
import ctypes
import hashlib
import random
import struct

import numpy as np

from oracle import pyoracle as po

Q = 2**64 - 2**32 - 31
TAG = b"MORPHEUS/KEY/SHAKE256/v2\0"


def _shake_words(seed, counter, nonce):
    msg = TAG + struct.pack("<12I", *seed, counter, *nonce)
    return list(struct.unpack("<16I", hashlib.shake_256(msg).digest(64)))


def test_shake_block_known_answer():
    # zk-torch-4/src/morpheus/keys.rs:133-135
    want = [1718816192, 2174491696, 1665938734, 997474263, 3934092271, 384552652, 1770842527, 2550189609,
            2315274332, 1133808957, 1818681556, 3465089802, 714274959, 3351567657, 2489001337, 1454658246]
    got = po.mcommit_shake_block([1, 2, 3, 4, 5, 6, 7, 8], 513, [0x10005, 0xDEAD, 0xBEEF])
    assert [int(v) for v in got] == want


def test_shake_block_against_hashlib():
    rnd = random.Random(5)
    for _ in range(50):
        seed = [rnd.randrange(2**32) for _ in range(8)]
        ctr = rnd.randrange(2**32)
        nonce = [rnd.randrange(2**32) for _ in range(3)]
        assert [int(v) for v in po.mcommit_shake_block(seed, ctr, nonce)] == _shake_words(seed, ctr, nonce)


def test_key_element_properties():
    # zk-torch-4/src/morpheus/keys.rs:113-127: canonical, deterministic, separated by kind / row / column
    seed = [1, 2, 3, 4, 5, 6, 7, 8]
    a = po.mcommit_key_element(seed, 1, 0, 5)
    assert (a == po.mcommit_key_element(seed, 1, 0, 5)).all()
    assert all(int(v) < Q for v in a)
    for other in (po.mcommit_key_element(seed, 2, 0, 5), po.mcommit_key_element(seed, 1, 1, 5), po.mcommit_key_element(seed, 1, 0, 6)):
        assert (a != other).any()
    hi = int((a >> np.uint64(63)).sum())
    assert 1700 <= hi <= 2400
    # block 3 by hand from hashlib (no rejection expected at 2^-31 per word)
    w = _shake_words(seed, 3, [(1 << 16) | 0, 5, 0])
    vals = [w[2 * t] | (w[2 * t + 1] << 32) for t in range(8)]
    assert all(v < Q for v in vals)
    assert [int(v) for v in a[24:32]] == vals


def test_library_key_expansion_on_the_host(hostcheck):
    hc = hostcheck
    hc.hc_mcm_shake.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]
    hc.hc_mcm_key_block.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p]
    rnd = random.Random(6)
    for _ in range(30):
        seed = np.array([rnd.randrange(2**32) for _ in range(8)], dtype=np.uint32)
        nonce = np.array([rnd.randrange(2**32) for _ in range(3)], dtype=np.uint32)
        ctr = rnd.randrange(2**32)
        out = np.zeros(16, dtype=np.uint32)
        hc.hc_mcm_shake(seed.ctypes.data, ctr, nonce.ctypes.data, out.ctypes.data)
        assert [int(v) for v in out] == _shake_words(seed, ctr, nonce)
    seed = np.array([9, 8, 7, 6, 5, 4, 3, 2], dtype=np.uint32)
    for kind, row, col in ((1, 0, 0), (2, 15, 12345), (3, 7, 2**33 + 5)):
        want = po.mcommit_key_element(seed, kind, row, col)
        for b in (0, 1, 255, 511):
            vals = np.zeros(8, dtype=np.uint64)
            hc.hc_mcm_key_block(seed.ctypes.data, kind, row, col, b, vals.ctypes.data)
            assert (vals == want[8 * b:8 * b + 8]).all()


def test_commit_oracle_is_linear_and_matches_python_integers():
    """One row, two columns with a handful of nonzero coefficients: exact integers in Python."""
    seed = [4, 4, 2, 2, 1, 1, 0, 9]
    rnd = random.Random(7)
    cols = [3, 11]
    x = np.zeros((2, 4096), dtype=np.int64)
    for c in range(2):
        for _ in range(6):
            x[c, rnd.randrange(4096)] = rnd.randrange(-(1 << 36), 1 << 36)
    err = np.zeros((1, 4096), dtype=np.int64)
    err[0, 17] = -1
    err[0, 4095] = 1
    got = po.mcommit_commit(seed, 2, 1, cols, x, err)[0]
    acc = [0] * 4096
    for c, col in enumerate(cols):
        key = [int(v) for v in po.mcommit_key_element(seed, 2, 0, col)]
        key = [v - Q if v > (Q - 1) // 2 else v for v in key]
        for i in np.nonzero(x[c])[0]:
            xi = int(x[c, i])
            for j in range(4096):
                if i + j < 4096:
                    acc[i + j] += xi * key[j]
                else:
                    acc[i + j - 4096] -= xi * key[j]
    acc[17] -= 1
    acc[4095] += 1
    assert [int(v) for v in got] == [a % Q for a in acc]
    # linearity in the witness
    x2 = np.zeros_like(x)
    x2[0, 5] = 1
    x2[1, 4000] = -1
    a = po.mcommit_commit(seed, 2, 1, cols, x)[0]
    b = po.mcommit_commit(seed, 2, 1, cols, x2)[0]
    s = po.mcommit_commit(seed, 2, 1, cols, x + x2)[0]
    assert [int(v) for v in s] == [(int(u) + int(v)) % Q for u, v in zip(a, b)]
