"""Seeded synthetic inputs: splitmix64 outputs reduced into the field.

The reference's tests draw inputs from Rust's StdRng, which cannot be
reproduced without its toolchain; every test and benchmark here uses this
generator instead and states the seed.
"""
import numpy as np

GL_P = 0xFFFFFFFF00000001   # Goldilocks, cuda/goldilocks.cuh:27
AGL_Q = 0xFFFFFFFEFFFFFFE1  # almost-Goldilocks 2^64 - 2^32 - 31, cuda_almost_goldilocks/almost_goldilocks.cuh:32


def splitmix64(seed, n):
    """n successive outputs of splitmix64 started at `seed`, as uint64."""
    idx = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def field_elems(seed, n, p=GL_P):
    """n canonical field elements."""
    return splitmix64(seed, n) % np.uint64(p)
