"""The on-disk commitment store: byte layout (zk-torch-4/src/commit/mod.rs:199-238, 302-310) and round trip."""
import struct

import numpy as np
import pytest

from matrix_b200.store import AjtaiStore, EdgeCommitment, KAPPA, RING_DIM


def _store():
    rng = np.random.default_rng(1)
    planes = lambda n: rng.integers(0, 2**63, size=(n, KAPPA, RING_DIM), dtype=np.uint64)
    return AjtaiStore(24, 21, range(1, 9), [EdgeCommitment(planes(3), False, 20), None, EdgeCommitment(planes(1), True, 7), None])


def test_byte_layout(tmp_path):
    st = _store()
    p = tmp_path / "store.bin"
    st.save(p)
    data = p.read_bytes()
    assert data[:8] == b"ZKAJTAI1"
    assert struct.unpack_from("<II", data, 8) == (24, 21)
    assert struct.unpack_from("<8I", data, 16) == tuple(range(1, 9))
    assert struct.unpack_from("<I", data, 48) == (4,)
    assert data[52] == 1 and data[53] == 0 and struct.unpack_from("<II", data, 54) == (20, 3)
    first = struct.unpack_from("<Q", data, 62)[0]
    assert first == int(st.commitments[0].planes[0, 0, 0])
    plane_bytes = KAPPA * RING_DIM * 8
    assert struct.unpack_from("<Q", data, 62 + plane_bytes + 8 * (5 * RING_DIM + 9))[0] == int(st.commitments[0].planes[1, 5, 9])
    after = 62 + 3 * plane_bytes
    assert data[after] == 0 and data[after + 1] == 1 and data[after + 2] == 1
    assert len(data) == after + 2 + 9 + plane_bytes + 1


def test_round_trip_and_errors(tmp_path):
    st = _store()
    p = tmp_path / "store.bin"
    st.save(p)
    back = AjtaiStore.load(p)
    assert (back.max_num_vars, back.b, back.seed) == (24, 21, list(range(1, 9)))
    assert back.commitments == st.commitments
    assert back.commitments[0].base == 2 and back.commitments[2].base == 1
    data = bytearray(p.read_bytes())
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"ZKAJTAI0" + bytes(data[8:]))
    with pytest.raises(ValueError):
        AjtaiStore.load(bad)
    data[52] = 2
    bad.write_bytes(bytes(data))
    with pytest.raises(ValueError):
        AjtaiStore.load(bad)
    bad.write_bytes(p.read_bytes()[:-5])
    with pytest.raises(ValueError):
        AjtaiStore.load(bad)
