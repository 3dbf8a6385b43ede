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


if __name__ == "__main__":
    main()
