"""The whole same-point sumcheck on the GPU (agl_same_point_prove_device_ffi) against the oracle's restatement of
zk-torch-4's prove_same_point, bit for bit, for every witness kind; the library's host verifier against the
oracle's; and the reference's own deterministic case of uniform arity (same_point_sumcheck.rs:1709-1730)."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_agl
from matrix_b200.inputs import AGL_Q
from oracle import pyoracle
from .test_oracle_same_point import binary_instance, lift, random_instance

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = load_agl()
    assert lib.almost_goldilocks_cuda_init() == 0
    return lib


def transcript(lib, label):
    h = ctypes.c_void_p()
    assert lib.agl_transcript_create(label, len(label), ctypes.byref(h)) == 0
    return h


def gpu_prove(lib, instances, label):
    M, arity, kind = len(instances), instances[0]["arity"], instances[0]["kind"]
    assert all(i["arity"] == arity and i["kind"] == kind for i in instances)
    pts = np.concatenate([np.asarray(i["point"], dtype=np.uint64).reshape(-1) for i in instances])
    vals = np.concatenate([np.asarray(i["value"], dtype=np.uint64).reshape(-1) for i in instances])
    n = 1 << arity
    words = max(1, n >> 6)
    keep = []
    if kind == 0:
        w0 = DeviceBuffer.from_numpy(lib, np.concatenate([i["witness"] for i in instances]))
        w1 = None
    elif kind == 1:
        w0 = DeviceBuffer.from_numpy(lib, np.concatenate([i["witness"][:words] for i in instances]))
        w1 = DeviceBuffer.from_numpy(lib, np.concatenate([i["witness"][words:] for i in instances]))
    else:
        dense = np.zeros((M, n, 2), dtype=np.uint64)
        for k, i in enumerate(instances):
            dense[k, :, 0] = i["witness"]
        w0, w1 = DeviceBuffer.from_numpy(lib, dense), None
    keep += [w0, w1]
    out = dict(round_msgs=np.zeros((arity, 3, 2), dtype=np.uint64), challenges=np.zeros((arity, 2), dtype=np.uint64),
               f_evals=np.zeros((M, 2), dtype=np.uint64), final_eval=np.zeros(2, dtype=np.uint64), state=np.zeros(12, dtype=np.uint64))
    t = transcript(lib, label)
    rc = lib.agl_same_point_prove_device_ffi(M, arity, pts.ctypes.data, vals.ctypes.data, kind, w0.ptr, w1.ptr if w1 else None, t,
                                             out["round_msgs"].ctypes.data, out["challenges"].ctypes.data,
                                             out["f_evals"].ctypes.data, out["final_eval"].ctypes.data)
    assert rc == 0
    assert lib.agl_transcript_state(t, out["state"].ctypes.data) == 0
    lib.agl_transcript_destroy(t)
    return out


def lib_verify(lib, instances, n, proof, label):
    arity = np.array([i["arity"] for i in instances], dtype=np.int32)
    pts = np.concatenate([np.asarray(i["point"], dtype=np.uint64).reshape(-1) for i in instances])
    vals = np.concatenate([np.asarray(i["value"], dtype=np.uint64).reshape(-1) for i in instances])
    ch = np.zeros((n, 2), dtype=np.uint64)
    ok = ctypes.c_int(0)
    t = transcript(lib, label)
    rc = lib.agl_same_point_verify_ffi(len(instances), n, arity.ctypes.data, pts.ctypes.data, vals.ctypes.data,
                                       np.ascontiguousarray(proof["round_msgs"]).ctypes.data,
                                       np.ascontiguousarray(proof["f_evals"]).ctypes.data,
                                       np.ascontiguousarray(proof["final_eval"]).ctypes.data, t, ch.ctypes.data, ctypes.byref(ok))
    lib.agl_transcript_destroy(t)
    assert rc == 0
    return bool(ok.value), ch


@pytest.mark.parametrize("kind,arity,leaves", [(0, 1, 1), (0, 4, 2), (0, 6, 3), (0, 7, 1), (0, 11, 5), (0, 16, 4), (0, 13, 42),
                                               (1, 6, 2), (1, 9, 3), (1, 14, 4), (2, 1, 2), (2, 5, 3), (2, 12, 2), (2, 15, 6)])
def test_gpu_proof_equals_the_cpu_prover(lib, kind, arity, leaves):
    insts = [random_instance(300 + 17 * i, kind, arity) for i in range(leaves)]
    exp = pyoracle.agl_same_point_prove(insts, arity, b"sp-gpu")
    got = gpu_prove(lib, insts, b"sp-gpu")
    for key in ("round_msgs", "challenges", "f_evals", "final_eval", "state"):
        assert np.array_equal(got[key], exp[key]), key
    ok, ch = lib_verify(lib, insts, arity, got, b"sp-gpu")
    assert ok and np.array_equal(ch, got["challenges"])
    assert pyoracle.agl_same_point_verify(insts, arity, got, b"sp-gpu")[0]


@pytest.mark.parametrize("kind,arity,leaves", [(0, 3, 2), (0, 12, 5), (1, 10, 3), (2, 9, 4)])
def test_claims_on_the_device(lib, kind, arity, leaves):
    insts = [random_instance(900 + 13 * i, kind, arity) for i in range(leaves)]
    pts = np.concatenate([np.asarray(i["point"], dtype=np.uint64).reshape(-1) for i in insts])
    n = 1 << arity
    words = max(1, n >> 6)
    if kind == 0:
        w0, w1 = DeviceBuffer.from_numpy(lib, np.concatenate([i["witness"] for i in insts])), None
    elif kind == 1:
        w0 = DeviceBuffer.from_numpy(lib, np.concatenate([i["witness"][:words] for i in insts]))
        w1 = DeviceBuffer.from_numpy(lib, np.concatenate([i["witness"][words:] for i in insts]))
    else:
        dense = np.zeros((leaves, n, 2), dtype=np.uint64)
        for k, i in enumerate(insts):
            dense[k, :, 0] = i["witness"]
        w0, w1 = DeviceBuffer.from_numpy(lib, dense), None
    vals = np.zeros((leaves, 2), dtype=np.uint64)
    assert lib.agl_same_point_claims_device_ffi(leaves, arity, pts.ctypes.data, kind, w0.ptr, w1.ptr if w1 else None, vals.ctypes.data) == 0
    for k, i in enumerate(insts):
        assert np.array_equal(vals[k], i["value"])


def test_reference_case_single_instance(lib):
    n = 4
    inst = binary_instance([0b10101100 ^ (0b11110000 << 8)], n, [lift(i * 7 + 3) for i in range(n)])
    got = gpu_prove(lib, [inst], b"sp-single")
    assert np.array_equal(got["f_evals"][0], pyoracle.agl_witness_eval(0, inst["witness"], n, got["challenges"]))
    assert lib_verify(lib, [inst], n, got, b"sp-single")[0]


def test_host_verifier_matches_the_oracle_on_mixed_arities_and_rejects_tampering(lib):
    insts = [random_instance(50, 0, 3), random_instance(60, 1, 9), random_instance(70, 2, 6)]
    proof = pyoracle.agl_same_point_prove(insts, 9, b"sp-mixed")
    ok, ch = lib_verify(lib, insts, 9, proof, b"sp-mixed")
    assert ok and np.array_equal(ch, proof["challenges"])
    for key, idx in (("f_evals", (1, 0)), ("round_msgs", (4, 1, 1)), ("final_eval", (0,))):
        bad = {k: v.copy() for k, v in proof.items()}
        bad[key][idx] = (int(bad[key][idx]) + 1) % AGL_Q
        assert not lib_verify(lib, insts, 9, bad, b"sp-mixed")[0], key


def test_bad_arguments(lib):
    t = transcript(lib, b"x")
    z = np.zeros(64, dtype=np.uint64)
    d = DeviceBuffer.from_numpy(lib, z)
    assert lib.agl_same_point_prove_device_ffi(0, 4, z.ctypes.data, z.ctypes.data, 0, d.ptr, None, t, z.ctypes.data, None,
                                               z.ctypes.data, z.ctypes.data) != 0
    assert lib.agl_same_point_prove_device_ffi(1, 4, z.ctypes.data, z.ctypes.data, 1, d.ptr, None, t, z.ctypes.data, None,
                                               z.ctypes.data, z.ctypes.data) != 0   # ternary needs both masks
    assert lib.agl_same_point_prove_device_ffi(1, 4, z.ctypes.data, z.ctypes.data, 3, d.ptr, None, t, z.ctypes.data, None,
                                               z.ctypes.data, z.ctypes.data) != 0
    lib.agl_transcript_destroy(t)


@pytest.mark.parametrize("log_n,leaves,binary", [(2, 1, False), (5, 3, False), (12, 4, False), (2, 2, True), (7, 3, True), (13, 2, True)])
def test_fused_fold_and_message_equals_fold_then_message(lib, log_n, leaves, binary):
    """aext2_sumcheck_batched_fold_message_ffi (and the binary round-0 form) against the two separate calls."""
    from matrix_b200.inputs import splitmix64
    n, half, blocks = 1 << log_n, 1 << (log_n - 1), 3
    polys = (splitmix64(5, leaves * 4 * n) % np.uint64(AGL_Q))
    words = max(1, n >> 6)
    packed = splitmix64(6, leaves * words)
    d_in = DeviceBuffer.from_numpy(lib, polys)
    d_bits = DeviceBuffer.from_numpy(lib, packed)
    d_a, d_b = DeviceBuffer(lib, polys.nbytes), DeviceBuffer(lib, polys.nbytes)
    d_p1, d_p2 = DeviceBuffer(lib, 8 * blocks * leaves * 6), DeviceBuffer(lib, 8 * blocks * leaves * 6)
    r = (0x123456789ABCDEF, 0xFEDCBA987654321)
    if binary:
        assert lib.aext2_sumcheck_batched_round0_binary_fold_ffi(d_in.ptr, d_bits.ptr, d_a.ptr, r[0], r[1], n, half, leaves, words) == 0
        assert lib.aext2_sumcheck_batched_round0_binary_fold_message_ffi(d_in.ptr, d_bits.ptr, d_b.ptr, r[0], r[1], n, half, leaves,
                                                                         blocks, words, d_p2.ptr) == 0
    else:
        assert lib.aext2_sumcheck_batched_fold_ffi(d_in.ptr, d_a.ptr, r[0], r[1], n, half, leaves) == 0
        assert lib.aext2_sumcheck_batched_fold_message_ffi(d_in.ptr, d_b.ptr, r[0], r[1], n, half, leaves, blocks, d_p2.ptr) == 0
    assert lib.aext2_sumcheck_batched_round_message_ffi(d_a.ptr, d_p1.ptr, n, half // 2, leaves, blocks) == 0
    lib.cuda_device_synchronize()
    a, b = d_a.to_numpy().view(np.uint64).reshape(leaves, 2, n, 2), d_b.to_numpy().view(np.uint64).reshape(leaves, 2, n, 2)
    assert np.array_equal(a[:, :, :half], b[:, :, :half])

    def total(buf):
        p = buf.to_numpy().view(np.uint64).reshape(blocks, leaves * 6)
        return [sum(int(x) for x in p[:, k]) % AGL_Q for k in range(leaves * 6)]
    assert total(d_p1) == total(d_p2)
