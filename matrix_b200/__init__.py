"""B200-native field-arithmetic hot path of a zero-knowledge prover.

The product is the pair of CUDA shared libraries under ``matrix_b200/lib``
(built by ``python -m matrix_b200.build``) with the C-ABI declared in
``include/``. This package only loads them through ctypes for tests and
benchmarks; it contains no CPU implementation of any kernel and raises if a
library is missing.
"""
from .ffi import load_gl, load_agl, LibraryMissing  # noqa: F401
