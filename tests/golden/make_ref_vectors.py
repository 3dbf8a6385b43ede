"""Generates golden vectors by running the reference's OWN code, compiled
host-side where it lies (needs the reference tree; run in the build container):

    python tests/golden/make_ref_vectors.py

Builds oracle/_ref (see oracle/Makefile) and writes tests/golden/*.json. The
inputs are fixed or drawn from Python's random.Random with the seeds below.
"""
import ctypes
import json
import os
import random
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
P = 0xFFFFFFFF00000001


def main():
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "ref"])
    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libgl_ref.so"))
    rnd = random.Random(20240601)
    cases = [list(range(8)), [0] * 8, [P - 1] * 8] + [[rnd.randrange(P) for _ in range(8)] for _ in range(13)]
    out = []
    for c in cases:
        s = (ctypes.c_uint64 * 8)(*c)
        ref.ref_poseidon2_permute_8(s)
        out.append({"in": c, "out": list(s)})
    json.dump({"source": "cuda/poseidon2.cuh:322-358 poseidon2_permute_8, host build", "permute": out},
              open(os.path.join(HERE, "gl_poseidon2.json"), "w"), indent=1)
    print("wrote gl_poseidon2.json")

    # Ajtai: the reference's own cpu_ajtai_commit_batched / cpu_prg_ring_elem / cpu_ring_mul
    import hashlib
    import numpy as np
    aj = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libajtai_ref.so"))
    vp, u64 = ctypes.c_void_p, ctypes.c_uint64
    aj.ref_ajtai_commit_dense.argtypes = [vp, vp, u64, ctypes.c_int, vp]
    aj.ref_ajtai_ring_elem.argtypes = [vp, ctypes.c_int, u64, vp]
    key = np.arange(1, 9, dtype=np.uint32)
    cases = []
    rng = np.random.default_rng(20240602)
    for (n, b) in ((4, 1), (16, 2), (33, 4)):
        if n == 4:
            z = np.array([0x123456789abcdef0, 0xFFFFFFFFFFFFFFFF, 0, 1], dtype=np.uint64)
        else:
            z = rng.integers(0, 2**63, size=n * b, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=n * b, dtype=np.uint64)
        out = np.zeros(b * 42 * 64, dtype=np.uint64)
        aj.ref_ajtai_commit_dense(key.ctypes.data, z.ctypes.data, n, b, out.ctypes.data)
        cases.append({"N": n, "B": b, "z": [int(x) for x in z], "first": int(out[0]), "last": int(out[-1]),
                      "sha256": hashlib.sha256(out.tobytes()).hexdigest()})
    elems = []
    for (row, j) in ((0, 0), (41, 5), (7, (1 << 32) + 3)):
        e = np.zeros(64, dtype=np.uint64)
        aj.ref_ajtai_ring_elem(key.ctypes.data, row, j, e.ctypes.data)
        elems.append({"row": row, "j": j, "coeffs": [int(x) for x in e]})
    # sparse commit over a seeded position list (repeated columns, unsorted order)
    aj.ref_ajtai_commit_sparse.argtypes = [vp, vp, u64, vp]
    pos = rng.integers(0, 64 * 40, size=200, dtype=np.uint64)
    pos[:4] = [0, 63, 64, 64 * 39 + 63]
    sp = np.zeros(42 * 64, dtype=np.uint64)
    aj.ref_ajtai_commit_sparse(key.ctypes.data, pos.ctypes.data, len(pos), sp.ctypes.data)
    sparse = {"positions": [int(x) for x in pos], "first": int(sp[0]), "last": int(sp[-1]),
              "sha256": hashlib.sha256(sp.tobytes()).hexdigest()}
    json.dump({"source": "cuda_almost_goldilocks/ajtai_cpu_reference.cuh cpu_ajtai_commit_batched<64,42>, cpu_prg_ring_elem<64>, "
                         "cpu_ajtai_commit_sparse<64,42>; key = 1..8",
               "key": [int(k) for k in key], "dense": cases, "ring_elems": elems, "sparse": sparse},
              open(os.path.join(HERE, "ajtai_ref.json"), "w"), indent=1)
    print("wrote ajtai_ref.json")


if __name__ == "__main__":
    main()
