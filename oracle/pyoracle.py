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
    """Compile the oracle and, when the reference tree is where the Makefile's REF points, oracle/_ref:
    the reference's host-only code (target ref) and its CUDA wrappers for sm_100a (target refcuda)."""
    subprocess.check_call(["make", "-s", "-C", HERE])
    if ref and subprocess.call(["make", "-s", "-C", HERE, "have-ref"]) == 0:
        subprocess.call(["make", "-s", "-C", HERE, "ref", "refcuda"])


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


# ---- Basefold -------------------------------------------------------------
_SIGS.update({
    "oracle_bf_query_words": (sz, [ci, ci]),
    "oracle_bf_proof_words": (sz, [ci, ci, ci]),
    "oracle_bf_table_entries": (sz, [ci, ci, ci]),
    "oracle_bf_table_generate": (None, [ci, ci, ci, u64, vp]),
    "oracle_bf_bit_reverse_gl": (None, [vp, ci]),
    "oracle_bf_bit_reverse_ext2": (None, [vp, ci]),
    "oracle_bf_bhc_interpolate": (None, [vp, vp, vp, ci]),
    "oracle_bf_encode": (None, [vp, vp, ci, ci]),
    "oracle_bf_merkle_tree": (None, [vp, sz, ci, vp]),
    "oracle_bf_commit": (None, [vp, ci, ci, vp, vp, vp]),
    "oracle_gl_eq_ext2": (None, [vp, ci, vp]),
    "oracle_gl_eq_base": (None, [vp, ci, vp]),
    "oracle_bf_open_ext2": (ci, [vp, vp, vp, ci, ci, vp, vp, ctypes.c_char_p, sz, ci, vp, vp]),
    "oracle_bf_verify_ext2": (ci, [vp, ci, ci, vp, vp, ctypes.c_char_p, sz, ci, vp]),
})


def bf_table(nv, lr, seed=42):
    """(point, weight) entries of the folding table, levels back to back."""
    import numpy as np
    lib = load()
    total = lib.oracle_bf_table_entries(nv, lr, nv)
    out = np.zeros(2 * total, dtype=np.uint64)
    lib.oracle_bf_table_generate(nv, lr, nv, seed, out.ctypes.data)
    return out


def bf_commit(evals, nv, lr):
    """Returns (codeword, bh_evals, tree) as uint64 arrays."""
    import numpy as np
    lib = load()
    evals = np.ascontiguousarray(evals, dtype=np.uint64)
    cw = np.zeros(1 << (nv + lr), dtype=np.uint64)
    bh = np.zeros(1 << nv, dtype=np.uint64)
    tree = np.zeros(4 * ((1 << (nv + lr)) - 1), dtype=np.uint64)
    lib.oracle_bf_commit(evals.ctypes.data, nv, lr, cw.ctypes.data, bh.ctypes.data, tree.ctypes.data)
    return cw, bh, tree


def bf_open(cw, bh, tree, nv, lr, point, table, num_queries, label=b"bench"):
    """Returns (proof words, transcript state)."""
    import numpy as np
    lib = load()
    proof = np.zeros(lib.oracle_bf_proof_words(nv, lr, num_queries), dtype=np.uint64)
    st = np.zeros(8, dtype=np.uint64)
    point = np.ascontiguousarray(point, dtype=np.uint64)
    rc = lib.oracle_bf_open_ext2(cw.ctypes.data, bh.ctypes.data, tree.ctypes.data, nv, lr, point.ctypes.data,
                                 table.ctypes.data, label, len(label), num_queries, proof.ctypes.data, st.ctypes.data)
    if rc != 0:
        raise RuntimeError("oracle_bf_open_ext2: %d" % rc)
    return proof, st


def bf_verify(root, nv, lr, point, table, num_queries, proof, label=b"bench"):
    import numpy as np
    lib = load()
    root = np.ascontiguousarray(root, dtype=np.uint64)
    point = np.ascontiguousarray(point, dtype=np.uint64)
    return lib.oracle_bf_verify_ext2(root.ctypes.data, nv, lr, point.ctypes.data, table.ctypes.data, label, len(label),
                                     num_queries, proof.ctypes.data)


# ---- almost-Goldilocks and partial evaluation ------------------------------------
_SIGS.update({
    "oracle_agl_mul": (u64, [u64, u64]),
    "oracle_agl_inv": (u64, [u64]),
    "oracle_aext2_mul": (None, [vp, vp, vp]),
    "oracle_agl_round_message": (None, [vp, ci, sz, sz, vp]),
    "oracle_agl_fold": (None, [vp, vp, u64, ci, sz, sz]),
    "oracle_aext2_round_message": (None, [vp, ci, sz, sz, vp]),
    "oracle_aext2_fold": (None, [vp, vp, u64, u64, ci, sz, sz]),
    "oracle_aext2_fold_mixed": (None, [vp, vp, u64, u64, ci, sz, sz, sz]),
    "oracle_agl_eq_base": (None, [vp, ci, vp]),
    "oracle_agl_eq_ext2": (None, [vp, ci, vp]),
    "oracle_agl_partial_eval": (None, [vp, vp, vp, ci, ci]),
    "oracle_agl_partial_eval_ext2_from_base": (None, [vp, vp, vp, ci, ci]),
    "oracle_gl_partial_eval": (None, [vp, vp, vp, ci, ci]),
    "oracle_gl_partial_eval_ext2_from_base": (None, [vp, vp, vp, ci, ci]),
})


# ---- Ajtai ------------------------------------------------------------------------
_SIGS.update({
    "oracle_chacha8_block": (None, [vp, ctypes.c_uint32, vp, vp]),
    "oracle_ajtai_ring_elem": (None, [vp, ctypes.c_uint32, u64, vp]),
    "oracle_ajtai_commit": (None, [vp, vp, ci, u64, ci, u64, vp]),
    "oracle_ajtai_commit_sparse": (None, [vp, vp, u64, vp]),
})

AJTAI_KAPPA, AJTAI_D = 42, 64


def ajtai_commit(key, z, kind, n_ring, planes, col_offset=0):
    """out[planes][42][64]; kind 0 = u64 bit planes, 1 = int8 digits, 2 = u64 field coefficients."""
    import numpy as np
    lib = load()
    key = np.ascontiguousarray(key, dtype=np.uint32)
    z = np.ascontiguousarray(z)
    out = np.zeros(planes * AJTAI_KAPPA * AJTAI_D, dtype=np.uint64)
    lib.oracle_ajtai_commit(key.ctypes.data, z.ctypes.data, kind, n_ring, planes, col_offset, out.ctypes.data)
    return out


def load_ref(name):
    """A library built from the reference's own sources (oracle/_ref), or None if absent."""
    path = os.path.join(HERE, "_ref", name)
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    if name == "libajtai_ref.so":
        lib.ref_ajtai_commit_dense.argtypes = [vp, vp, u64, ci, vp]
        lib.ref_ajtai_ring_elem.argtypes = [vp, ci, u64, vp]
        lib.ref_ring_mul.argtypes = [vp, vp, vp]
        lib.ref_chacha8_block.argtypes = [vp, ctypes.c_uint32, vp, vp]
        lib.ref_agl_mul.argtypes = [u64, u64]
        lib.ref_agl_mul.restype = u64
    return lib


# ---- batched eq * a * b sumcheck ---------------------------------------------------
_SIGS.update({
    "oracle_gl_batched_message": (None, [vp, vp, vp, ci, sz, sz, vp]),
    "oracle_gl_batched_fold": (None, [vp, vp, u64, u64, ci, sz, sz]),
    "oracle_gl_batched_claims": (None, [vp, vp, ci, sz, sz, vp]),
    "oracle_gl_batched_prove": (ci, [vp, vp, vp, ci, ci, ctypes.c_char_p, sz, vp, vp, vp, vp, vp, vp, vp]),
    "oracle_gl_e2_inv": (None, [vp, vp]),
    "oracle_gl_e5_mul": (None, [vp, vp, vp]),
    "oracle_gl_e5_frobenius": (None, [vp, vp]),
    "oracle_gl_e5_inv": (None, [vp, vp]),
    "oracle_gl_e5_pow": (None, [vp, u64, vp]),
})


_SIGS.update({
    "oracle_set_threads": (None, [ci]),
    "oracle_max_threads": (ci, []),
    "oracle_agl_sumcheck_prove": (ci, [vp, ci, ci, ci, ctypes.c_char_p, sz, vp, vp, vp, vp, vp]),
    "oracle_agl_sumcheck_verify": (ci, [vp, vp, vp, ci, ci, ctypes.c_char_p, sz, vp]),
})


def agl_sumcheck_prove(polys, d, num_var, base_field, label=b"bench"):
    """zk-torch-4's linear sumcheck prover (Monolith transcript) on a numpy array of d poly-major tables.
    Returns (round_msgs, challenges, final_evals, final_eval, sponge_state) as numpy arrays."""
    import numpy as np
    lib = load()
    polys = np.ascontiguousarray(polys, dtype=np.uint64)
    msgs = np.zeros(max(num_var, 1) * (d + 1) * 2, dtype=np.uint64)
    ch = np.zeros(max(num_var, 1) * 2, dtype=np.uint64)
    fe = np.zeros(2 * d, dtype=np.uint64)
    fin = np.zeros(2, dtype=np.uint64)
    st = np.zeros(12, dtype=np.uint64)
    rc = lib.oracle_agl_sumcheck_prove(polys.ctypes.data, d, num_var, int(base_field), label, len(label), msgs.ctypes.data,
                                       ch.ctypes.data, fe.ctypes.data, fin.ctypes.data, st.ctypes.data)
    assert rc == 0
    return msgs[:num_var * (d + 1) * 2], ch[:2 * num_var], fe, fin, st


def agl_sumcheck_verify(msgs, final_eval, claimed, d, num_var, label=b"bench"):
    """zk-torch-4's SumcheckVerifier::verify; returns (accepted, challenges)."""
    import numpy as np
    lib = load()
    msgs = np.ascontiguousarray(msgs, dtype=np.uint64)
    fin = np.ascontiguousarray(final_eval, dtype=np.uint64)
    cl = np.ascontiguousarray(claimed, dtype=np.uint64)
    ch = np.zeros(max(num_var, 1) * 2, dtype=np.uint64)
    ok = lib.oracle_agl_sumcheck_verify(msgs.ctypes.data, fin.ctypes.data, cl.ctypes.data, d, num_var, label, len(label),
                                        ch.ctypes.data)
    return bool(ok), ch[:2 * num_var]


_SIGS.update({
    "oracle_agl_witness_eval": (None, [ci, vp, ci, vp, vp]),
    "oracle_agl_same_point_prove": (ci, [ci, ci, vp, vp, vp, vp, vp, vp, vp, ctypes.c_char_p, sz, vp, vp, vp, vp, vp]),
    "oracle_agl_same_point_verify": (ci, [ci, ci, vp, vp, vp, vp, vp, vp, vp, ctypes.c_char_p, sz, vp]),
})


def _sp_pack(instances):
    """Flattens same-point instances: each is a dict with arity, point (arity x 2 words), kind (0 binary packed,
    1 ternary single chunk: pos words then neg words, 2 dense base-field table) and witness (uint64 words)."""
    import numpy as np
    arity = np.array([i["arity"] for i in instances], dtype=np.int32)
    kind = np.array([i["kind"] for i in instances], dtype=np.int32)
    pts = [np.ascontiguousarray(i["point"], dtype=np.uint64).reshape(-1) for i in instances]
    wit = [np.ascontiguousarray(i["witness"], dtype=np.uint64).reshape(-1) for i in instances]
    pt_off = np.cumsum([0] + [len(x) for x in pts[:-1]]).astype(np.uint64)
    wit_off = np.cumsum([0] + [len(x) for x in wit[:-1]]).astype(np.uint64)
    return arity, kind, np.concatenate(pts), pt_off, np.concatenate(wit), wit_off


def agl_witness_eval(kind, witness, arity, point):
    """FoldData::evaluate_at_ext2: the multilinear extension of a same-point witness at `point` -> (c0, c1)."""
    import numpy as np
    lib = load()
    w = np.ascontiguousarray(witness, dtype=np.uint64)
    pt = np.ascontiguousarray(point, dtype=np.uint64).reshape(-1)
    out = np.zeros(2, dtype=np.uint64)
    lib.oracle_agl_witness_eval(int(kind), w.ctypes.data, int(arity), pt.ctypes.data, out.ctypes.data)
    return out


def agl_same_point_prove(instances, num_vars, label):
    """zk-torch-4's prove_same_point (dense CPU states, Monolith transcript). `instances`: see _sp_pack, plus
    "value" (2 words) per instance. Returns a dict of numpy arrays: round_msgs [N][3][2], challenges [N][2],
    f_evals [M][2], final_eval [2], state [12]."""
    import numpy as np
    lib = load()
    M = len(instances)
    arity, kind, pts, pt_off, wit, wit_off = _sp_pack(instances)
    vals = np.ascontiguousarray([i["value"] for i in instances], dtype=np.uint64).reshape(-1)
    out = dict(round_msgs=np.zeros((num_vars, 3, 2), dtype=np.uint64), challenges=np.zeros((num_vars, 2), dtype=np.uint64),
               f_evals=np.zeros((M, 2), dtype=np.uint64), final_eval=np.zeros(2, dtype=np.uint64),
               state=np.zeros(12, dtype=np.uint64))
    rc = lib.oracle_agl_same_point_prove(M, num_vars, arity.ctypes.data, pts.ctypes.data, pt_off.ctypes.data, vals.ctypes.data,
                                         kind.ctypes.data, wit.ctypes.data, wit_off.ctypes.data, label, len(label),
                                         out["round_msgs"].ctypes.data, out["challenges"].ctypes.data,
                                         out["f_evals"].ctypes.data, out["final_eval"].ctypes.data, out["state"].ctypes.data)
    assert rc == 0, rc
    return out


def agl_same_point_verify(instances, num_vars, proof, label):
    """zk-torch-4's verify_same_point on (arity, point, value) of every instance; returns (accepted, challenges)."""
    import numpy as np
    lib = load()
    M = len(instances)
    arity = np.array([i["arity"] for i in instances], dtype=np.int32)
    pts = [np.ascontiguousarray(i["point"], dtype=np.uint64).reshape(-1) for i in instances]
    pt_off = np.cumsum([0] + [len(x) for x in pts[:-1]]).astype(np.uint64)
    pts = np.concatenate(pts)
    vals = np.ascontiguousarray([i["value"] for i in instances], dtype=np.uint64).reshape(-1)
    msgs = np.ascontiguousarray(proof["round_msgs"], dtype=np.uint64)
    fe = np.ascontiguousarray(proof["f_evals"], dtype=np.uint64)
    fin = np.ascontiguousarray(proof["final_eval"], dtype=np.uint64)
    ch = np.zeros((num_vars, 2), dtype=np.uint64)
    ok = lib.oracle_agl_same_point_verify(M, num_vars, arity.ctypes.data, pts.ctypes.data, pt_off.ctypes.data, vals.ctypes.data,
                                          msgs.ctypes.data, fe.ctypes.data, fin.ctypes.data, label, len(label), ch.ctypes.data)
    return bool(ok), ch


def e5_op(name, a, b=None, e=None):
    """One Ext5 operation of the oracle on lists of five words: name in mul / frobenius / inv / pow."""
    lib = load()
    A, O = (u64 * 5)(*a), (u64 * 5)()
    if name == "mul":
        lib.oracle_gl_e5_mul(A, (u64 * 5)(*b), O)
    elif name == "pow":
        lib.oracle_gl_e5_pow(A, e, O)
    else:
        getattr(lib, "oracle_gl_e5_" + name)(A, O)
    return [int(x) for x in O]


def batched_prove(a, b, point, K, nv, label=b"bench"):
    """Whole batched eq*a*b sumcheck on the CPU; a, b: [K * 2^nv] base field."""
    import numpy as np
    lib = load()
    a, b, point = (np.ascontiguousarray(x, dtype=np.uint64) for x in (a, b, point))
    out = dict(claims=np.zeros((K, 2), dtype=np.uint64), alpha=np.zeros(2, dtype=np.uint64),
               round_msgs=np.zeros((nv, 4, 2), dtype=np.uint64), challenges=np.zeros((nv, 2), dtype=np.uint64),
               finals=np.zeros((2 * K + 1, 2), dtype=np.uint64), final_eval=np.zeros(2, dtype=np.uint64),
               state=np.zeros(8, dtype=np.uint64))
    rc = lib.oracle_gl_batched_prove(a.ctypes.data, b.ctypes.data, point.ctypes.data, K, nv, label, len(label),
                                     out["claims"].ctypes.data, out["alpha"].ctypes.data, out["round_msgs"].ctypes.data,
                                     out["challenges"].ctypes.data, out["finals"].ctypes.data,
                                     out["final_eval"].ctypes.data, out["state"].ctypes.data)
    if rc != 0:
        raise RuntimeError("oracle_gl_batched_prove: %d" % rc)
    return out


# ---- Monolith (both fields) and the almost-Goldilocks transcript ---------------------
_SIGS.update({
    "oracle_gl_monolith_permute": (None, [vp]),
    "oracle_agl_monolith_permute": (None, [vp]),
    "oracle_agl_monolith_rc": (None, [vp]),
    "oracle_set_merkle_hash": (None, [ci]),
    "oracle_get_merkle_hash": (ci, []),
    "oracle_sha256": (None, [ctypes.c_char_p, sz, vp]),
    "oracle_agl_transcript_run": (sz, [ctypes.c_char_p, sz, sz, vp, ctypes.c_char_p, vp, vp, vp, vp, vp]),
})

APPEND, CHALLENGE, FORK = 0, 1, 2


def agl_transcript_run(init_label, ops):
    """Runs a scripted almost-Goldilocks transcript: ops = [(APPEND | CHALLENGE | FORK, label, value)].
    Returns (challenges in order, final 12-word sponge state)."""
    import numpy as np
    lib = load()
    kinds = np.array([o[0] for o in ops], dtype=np.int32)
    labels = b"".join(o[1] for o in ops)
    lens = np.array([len(o[1]) for o in ops], dtype=np.uint64)
    offs = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.uint64) if len(ops) else np.zeros(0, dtype=np.uint64)
    vals = np.array([o[2] for o in ops], dtype=np.uint64)
    out = np.zeros(max(1, len(ops)), dtype=np.uint64)
    state = np.zeros(12, dtype=np.uint64)
    n = lib.oracle_agl_transcript_run(init_label, len(init_label), len(ops), kinds.ctypes.data, labels,
                                      offs.ctypes.data, lens.ctypes.data, vals.ctypes.data, out.ctypes.data,
                                      state.ctypes.data)
    return out[:n].copy(), state


class merkle_hash:
    """Context manager: the oracle's Merkle hash (0 Poseidon2, 1 Monolith) inside the block."""

    def __init__(self, h):
        self.h = h

    def __enter__(self):
        lib = load()
        self.prev = lib.oracle_get_merkle_hash()
        lib.oracle_set_merkle_hash(self.h)

    def __exit__(self, *a):
        load().oracle_set_merkle_hash(self.prev)


# ---- K = F_q[Theta]/(Theta^8 - 3) and its product sumcheck -----------------------------
_SIGS.update({
    "oracle_k8_add": (None, [vp, vp, vp]),
    "oracle_k8_sub": (None, [vp, vp, vp]),
    "oracle_k8_mul": (None, [vp, vp, vp]),
    "oracle_k8_eq_table": (None, [vp, ci, vp]),
    "oracle_k8_sc_round": (None, [vp, ci, sz, ci, vp]),
    "oracle_k8_sc_fold": (None, [vp, sz, vp, vp]),
    "oracle_k8_axpy": (None, [vp, vp, sz, vp]),
})


def k8_sc_round(tabs, d):
    """tabs: list of uint64 arrays [len * 8]; returns the (d + 1) x 8 words of the round sums."""
    import numpy as np
    lib = load()
    ptrs = (ctypes.c_void_p * len(tabs))(*[t.ctypes.data for t in tabs])
    out = np.zeros((d + 1) * 8, dtype=np.uint64)
    lib.oracle_k8_sc_round(ptrs, len(tabs), len(tabs[0]) // 8, d, out.ctypes.data)
    return out


def k8_sc_fold(tab, r):
    import numpy as np
    lib = load()
    out = np.zeros(len(tab) // 2, dtype=np.uint64)
    lib.oracle_k8_sc_fold(tab.ctypes.data, len(tab) // 8, np.ascontiguousarray(r, dtype=np.uint64).ctypes.data, out.ctypes.data)
    return out


# ---- module commitment over F_q[Y]/(Y^4096 + 1) ----------------------------------------
_SIGS.update({
    "oracle_shake256_short": (None, [vp, sz, vp, sz]),
    "oracle_mcommit_shake_block": (None, [vp, ctypes.c_uint32, vp, vp]),
    "oracle_mcommit_key_element": (None, [vp, ctypes.c_uint32, ctypes.c_uint32, u64, vp]),
    "oracle_mcommit_commit": (None, [vp, ctypes.c_uint32, ci, vp, ci, vp, vp, vp]),
})


def mcommit_shake_block(seed, counter, nonce):
    import numpy as np
    s = np.ascontiguousarray(seed, dtype=np.uint32)
    n = np.ascontiguousarray(nonce, dtype=np.uint32)
    out = np.zeros(16, dtype=np.uint32)
    load().oracle_mcommit_shake_block(s.ctypes.data, counter, n.ctypes.data, out.ctypes.data)
    return out


def mcommit_key_element(seed, kind, row, col):
    import numpy as np
    s = np.ascontiguousarray(seed, dtype=np.uint32)
    out = np.zeros(4096, dtype=np.uint64)
    load().oracle_mcommit_key_element(s.ctypes.data, kind, row, col, out.ctypes.data)
    return out


def mcommit_commit(seed, kind, rows, cols, x, err=None):
    """x: int64 [len(cols)][4096]; err: int64 [rows][4096] or None; returns uint64 [rows][4096]."""
    import numpy as np
    s = np.ascontiguousarray(seed, dtype=np.uint32)
    c = np.ascontiguousarray(cols, dtype=np.uint64)
    xx = np.ascontiguousarray(x, dtype=np.int64).reshape(len(c), 4096)
    e = None if err is None else np.ascontiguousarray(err, dtype=np.int64).reshape(rows, 4096)
    out = np.zeros((rows, 4096), dtype=np.uint64)
    load().oracle_mcommit_commit(s.ctypes.data, kind, rows, c.ctypes.data, len(c), xx.ctypes.data,
                                 None if e is None else e.ctypes.data, out.ctypes.data)
    return out


# ---- packed link sumcheck ---------------------------------------------------------------
u32 = ctypes.c_uint32
_SIGS.update({
    "oracle_link_round": (None, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, u64, u32, ci, ci, ci, ci, vp]),
    "oracle_link_fold_rows": (None, [vp, u64, u64, u64, vp, vp, vp, u64, u64]),
    "oracle_link_fold_w": (None, [vp, vp, vp, u64, u64, u64, u64, u64, u64, u64]),
    "oracle_link_eq_expand": (None, [vp, u64, u64, u64]),
    "oracle_link_expand_bits": (None, [vp, vp, u64]),
    "oracle_link_eq_gather": (None, [vp, u64, vp, vp, u64]),
})


def _p(a):
    return None if a is None else a.ctypes.data


def link_round(eq, tags, half, n_commit, first_round, bits=None, w=None, omega=None, pts=None, scale=None, lists=None,
               w_stride=0, bits_stride_words=0, omega_stride=0, block_mask=0, block_bits=0, leaf_arity=0, rnd=0):
    """lists: (list u32, off u64, len u64) or None. Returns the 14 words [S(0..3), E(0..2)]."""
    import numpy as np
    out = np.zeros(14, dtype=np.uint64)
    l, lo, ll = lists if lists is not None else (None, None, None)
    load().oracle_link_round(_p(bits), _p(w), _p(omega), _p(pts), _p(scale), _p(eq), _p(tags), _p(l), _p(lo), _p(ll), w_stride,
                             bits_stride_words, omega_stride, half, n_commit, block_mask, block_bits, leaf_arity, rnd,
                             first_round, out.ctypes.data)
    return out


def link_fold_rows(tab, stride, half, n_commit, r, lists=None):
    import numpy as np
    t = np.array(tab, dtype=np.uint64, copy=True)
    l, lo, ll = lists if lists is not None else (None, None, None)
    load().oracle_link_fold_rows(t.ctypes.data, stride, half, n_commit, _p(l), _p(lo), _p(ll), int(r[0]), int(r[1]))
    return t


def link_fold_w(bits, w_in, in_stride, bits_stride_words, out_stride, half, n_commit, r):
    import numpy as np
    out = np.zeros(2 * n_commit * out_stride, dtype=np.uint64)
    load().oracle_link_fold_w(_p(bits), _p(w_in), out.ctypes.data, in_stride, bits_stride_words, out_stride, half, n_commit,
                              int(r[0]), int(r[1]))
    return out


def link_eq_expand(table, span, r):
    import numpy as np
    t = np.array(table, dtype=np.uint64, copy=True)
    load().oracle_link_eq_expand(t.ctypes.data, span, int(r[0]), int(r[1]))
    return t


def link_expand_bits(bits):
    import numpy as np
    out = np.zeros(len(bits) * 128, dtype=np.uint64)
    load().oracle_link_expand_bits(bits.ctypes.data, out.ctypes.data, len(bits))
    return out


def link_eq_gather(alpha, n_vars, lst):
    import numpy as np
    out = np.zeros(2 * len(lst), dtype=np.uint64)
    load().oracle_link_eq_gather(alpha.ctypes.data, n_vars, lst.ctypes.data, out.ctypes.data, len(lst))
    return out


# ---- sparse boolean-check sumcheck ------------------------------------------------------
_SIGS.update({
    "oracle_bool_round": (u32, [vp, vp, vp, vp, vp, ci, u32, vp, vp, vp]),
    "oracle_bool_fold": (None, [vp, vp, vp, vp, vp, ci, u32, u64, u64, u32, vp, vp, vp]),
})


def bool_round(idx, val, term_off, w, eq):
    """Returns (flags, gid, msg[8], total)."""
    import numpy as np
    n, n_terms = len(idx), len(term_off) - 1
    flags, gid = np.zeros(max(n, 1), dtype=np.uint32), np.zeros(max(n, 1), dtype=np.uint32)
    msg = np.zeros(8, dtype=np.uint64)
    total = load().oracle_bool_round(idx.ctypes.data, val.ctypes.data, term_off.ctypes.data, w.ctypes.data, eq.ctypes.data, n_terms, n,
                                     flags.ctypes.data, gid.ctypes.data, msg.ctypes.data)
    return flags[:n], gid[:n], msg, int(total)


def bool_fold(idx, val, flags, gid, term_off, r, total):
    """Returns (out_idx, out_val, new_off)."""
    import numpy as np
    n, n_terms = len(idx), len(term_off) - 1
    out_idx, out_val = np.zeros(max(total, 1), dtype=np.uint32), np.zeros(2 * max(total, 1), dtype=np.uint64)
    new_off = np.zeros(n_terms + 1, dtype=np.uint32)
    load().oracle_bool_fold(idx.ctypes.data, val.ctypes.data, flags.ctypes.data, gid.ctypes.data, term_off.ctypes.data, n_terms, n,
                            int(r[0]), int(r[1]), total, out_idx.ctypes.data, out_val.ctypes.data, new_off.ctypes.data)
    return out_idx[:total], out_val[:2 * total], new_off
