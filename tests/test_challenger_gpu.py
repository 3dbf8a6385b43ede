"""The device challenger against the CPU transcript of the oracle: same
absorb / squeeze scripts must give the same outputs and the same state."""
import ctypes

import numpy as np
import pytest

from matrix_b200.ffi import DeviceBuffer, load_gl
from .conftest import GL_P, field_elems

pytestmark = pytest.mark.gpu
u64 = ctypes.c_uint64


class T(ctypes.Structure):
    _fields_ = [("sponge", u64 * 8), ("in_buf", u64 * 4), ("out_buf", u64 * 4),
                ("in_count", ctypes.c_int), ("out_count", ctypes.c_int), ("perms", u64)]


def test_batched_transcripts_match_cpu(oracle):
    lib = load_gl()
    assert lib.goldilocks_cuda_init() == 0
    assert lib.challenger_state_size() == 136
    oracle.gl_transcript_squeeze.restype = u64
    oracle.gl_transcript_absorb.argtypes = [ctypes.c_void_p, u64]
    n = 300
    states = ctypes.c_void_p()
    assert lib.challenger_alloc_states(ctypes.byref(states), n) == 0
    assert lib.challenger_init_states(states, n) == 0
    cpu = [T() for _ in range(n)]
    for t in cpu:
        oracle.gl_transcript_new(ctypes.byref(t), b"", 0)
    script = [("obs", 1), ("obs", 5), ("smp", 1), ("smp", 2), ("obs2", 2), ("smp", 5), ("obs", 3), ("smp", 7), ("obs", 4), ("smp", 1)]
    for step, (kind, count) in enumerate(script):
        if kind.startswith("obs"):
            vals = field_elems(700 + step, n * count)
            d_v = DeviceBuffer.from_numpy(lib, vals)
            if kind == "obs2":
                assert lib.challenger_observe_ext2_ffi(states, d_v.ptr, n) == 0
            elif count == 1:
                assert lib.challenger_observe_ffi(states, d_v.ptr, n) == 0
            else:
                assert lib.challenger_observe_slice_ffi(states, d_v.ptr, count, n) == 0
            for i, t in enumerate(cpu):
                for k in range(count):
                    oracle.gl_transcript_absorb(ctypes.byref(t), int(vals[i * count + k]))
        else:
            d_o = DeviceBuffer(lib, 8 * n * count)
            fn = {1: lib.challenger_sample_ffi, 2: lib.challenger_sample_ext2_ffi, 5: lib.challenger_sample_ext5_ffi}.get(count)
            if fn is not None:
                assert fn(states, d_o.ptr, n) == 0
            else:
                assert lib.challenger_sample_array_ffi(states, d_o.ptr, count, n) == 0
            got = d_o.to_numpy().reshape(n, count)
            for i, t in enumerate(cpu):
                exp = [oracle.gl_transcript_squeeze(ctypes.byref(t)) for _ in range(count)]
                assert list(got[i]) == exp, "transcript %d step %d" % (i, step)
    # state round trip
    h = (ctypes.c_uint8 * 136)()
    assert lib.challenger_copy_state_to_host(h, states.value + 136 * 7) == 0
    words = np.frombuffer(bytes(h), dtype=np.uint64, count=8)
    assert list(words) == list(cpu[7].sponge)
    assert lib.challenger_copy_state_to_device(states.value, h) == 0
    d_o = DeviceBuffer(lib, 8)
    assert lib.challenger_sample_ffi(states, d_o.ptr, 1) == 0
    assert int(d_o.to_numpy()[0]) == oracle.gl_transcript_squeeze(ctypes.byref(cpu[7]))
    lib.cuda_free(states)
