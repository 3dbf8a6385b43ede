"""ctypes loader for the CPU oracle (test infrastructure, not the product).

Only tests, the smoke check and the benchmark's cpu_baseline / reference arm
may import this module.
"""
import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "liboracle.so")

u64 = ctypes.c_uint64
vp = ctypes.c_void_p
ci = ctypes.c_int
sz = ctypes.c_size_t


def build(ref=True):
    """Compile the oracle (and, if the reference tree is present, oracle/_ref)."""
    subprocess.check_call(["make", "-s", "-C", HERE])
    if ref:
        subprocess.call(["make", "-s", "-C", HERE, "ref"])


_SIGS = {
    "gl_pow": (u64, [u64, u64]),
    "gl_inv": (u64, [u64]),
    "gl_poseidon2_permute": (None, [vp]),
    "oracle_gl_round_message": (None, [vp, ci, sz, sz, vp]),
    "oracle_gl_fold": (None, [vp, vp, u64, ci, sz, sz]),
    "oracle_gl_round_message_ext2": (None, [vp, ci, sz, sz, vp]),
    "oracle_gl_fold_ext2": (None, [vp, vp, u64, u64, ci, sz, sz]),
    "oracle_gl_sumcheck_prove": (ci, [vp, ci, ci, ci, ctypes.c_char_p, sz, vp, vp, vp, vp, vp]),
    "oracle_gl_sumcheck_verify": (ci, [ci, ci, ctypes.c_char_p, sz, vp, vp, vp]),
}

_LIB = None


def load():
    global _LIB
    if _LIB is None:
        srcs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".c", ".h"))]
        stale = not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in srcs)
        if stale:
            build(ref=False)
        lib = ctypes.CDLL(LIB)
        for name, (res, args) in _SIGS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB


def sumcheck_prove(polys, d, num_var, base_field, label=b"bench"):
    """Runs the oracle's sumcheck prover. `polys`: uint64 array, poly-major.
    Returns dict(round_msgs[num_var, d+1, 2], challenges[num_var, 2], final_evals[d, 2], final_eval[2], state[8])."""
    import numpy as np
    lib = load()
    polys = np.ascontiguousarray(polys, dtype=np.uint64)
    rm = np.zeros((num_var, d + 1, 2), dtype=np.uint64)
    ch = np.zeros((num_var, 2), dtype=np.uint64)
    fes = np.zeros((d, 2), dtype=np.uint64)
    fe = np.zeros(2, dtype=np.uint64)
    st = np.zeros(8, dtype=np.uint64)
    rc = lib.oracle_gl_sumcheck_prove(polys.ctypes.data, d, num_var, 1 if base_field else 0, label, len(label),
                                      rm.ctypes.data, ch.ctypes.data, fes.ctypes.data, fe.ctypes.data, st.ctypes.data)
    if rc != 0:
        raise RuntimeError("oracle_gl_sumcheck_prove: %d" % rc)
    return dict(round_msgs=rm, challenges=ch, final_evals=fes, final_eval=fe, state=st)
