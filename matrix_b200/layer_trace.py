"""Shape trace of one Llama-2-7B decoder layer, replayed as the GPU calls its einsum blocks make.

What is replayed: for every einsum of the layer (the projections, the two attention products, the
scaling and the SwiGLU products of `zk-torch-4/src/dag/llama.rs:399-485`), the device sequence of
`Einsum::prove_gpu` (`zk-torch-4/src/basicblock/einsum.rs:1168-1310`):

  1. each operand is partially evaluated at the output point's challenges for the variables only that
     operand shares with the output (plain partial evaluation when those variables are its low bits,
     fused bit-permutation + partial evaluation otherwise, base-field to extension lift when none);
  2. the eq table of the variables shared by several operands and the output is built and tiled over
     the summation variables (a table of ones when there are none);
  3. one linear sumcheck over (shared + summation) variables with (operands + 1) tables, on the
     caller's transcript.

Operand values are synthetic (seeded 16-bit fixed-point integers as field elements). Variable
placement inside the tables is this module's own convention (shared variables in the low bits,
summation variables above, each in equation order), so proofs are checked by the sumcheck verifier
against the directly computed claim, not against the reference's bytes. Not replayed: the lookup /
range arguments of the non-linear blocks (sigmoid, softmax, RMS reciprocal, RoPE tables) and the
fold tree above the blocks.

No CPU path: everything runs through the C-ABI of the almost-Goldilocks library.
"""
import ctypes

import numpy as np

from .ffi import DeviceBuffer
from .inputs import AGL_Q, splitmix64


def llama_layer_ops(seq_log=7, hidden_log=12, heads_log=5, ffn_shard_log=10, ffn_shards=16):
    """(name, equation, {letter: log2 size}) for the einsums of one decoder layer. Llama-2-7B:
    hidden 4096, 32 heads of 128, FFN 11008 padded to 16 shards of 1024 (dag/llama.rs:395-398), seq 128."""
    hd = hidden_log - heads_log
    proj = dict(s=seq_log, i=hidden_log, j=hidden_log)
    att = dict(h=heads_log, s=seq_log, t=seq_log, d=hd)
    ops = [("attn_q", "si,ij->sj", proj), ("attn_k", "si,ij->sj", proj), ("attn_v", "si,ij->sj", proj),
           ("attn_scores", "hsd,htd->hst", att), ("attn_scale", "hst,z->hst", dict(att, z=0)),
           ("attn_out", "hst,htd->hsd", att), ("attn_o", "si,ij->sj", proj)]
    up = dict(s=seq_log, i=hidden_log, j=ffn_shard_log)
    ew = dict(s=seq_log, i=ffn_shard_log)
    down = dict(s=seq_log, i=ffn_shard_log, j=hidden_log)
    for k in range(ffn_shards):
        ops += [("ffn%d_gate" % k, "si,ij->sj", up), ("ffn%d_swish" % k, "si,si->si", ew), ("ffn%d_up" % k, "si,ij->sj", up),
                ("ffn%d_mul" % k, "si,si->si", ew), ("ffn%d_down" % k, "si,ij->sj", down)]
    return ops


def _bits(letters, dims):
    """[(letter, bit)] of a tensor's index, low variable first: the last letter varies fastest."""
    return [(c, b) for c in reversed(letters) for b in range(dims[c])]


class EinsumPlan:
    """Which variables of an equation are fixed per operand, shared, or summed, and the tables' layout."""

    def __init__(self, equation, dims):
        lhs, out = equation.split("->")
        self.inputs, self.out, self.dims = lhs.split(","), out, dims
        count = {c: sum(c in t for t in self.inputs) for c in set("".join(self.inputs))}
        for c, k in count.items():
            if c not in out and k < 2 and dims[c]:
                raise ValueError("reduction of a single operand is not part of this trace: " + equation)
        self.shared = [v for v in _bits(out, dims) if count.get(v[0], 0) >= 2]           # first rounds (eq table)
        summed = []
        for t in self.inputs:
            summed += [v for v in _bits(t, dims) if v[0] not in out and v not in summed]
        self.summed = summed                                                               # second rounds
        self.table_vars = self.shared + self.summed
        self.rounds = len(self.table_vars)
        self.fixed = [[v for v in _bits(t, dims) if v[0] in out and count[v[0]] == 1] for t in self.inputs]

    def operand_order(self, k):
        """New variable order of operand k (old positions, new low bit first): fixed, then its table variables."""
        old = _bits(self.inputs[k], self.dims)
        mine = [v for v in self.table_vars if v in old]
        return [old.index(v) for v in self.fixed[k] + mine], len(mine)


def split_luts(n, new_var_order, half):
    """Index tables of the fused kernel (almost-goldilocks-cuda-rs/src/partial_eval.rs:283-321)."""
    lo = np.zeros(1 << half, dtype=np.uint32)
    hi = np.zeros(1 << (n - half), dtype=np.uint32)
    for bit in range(half):
        lo[(np.arange(1 << half) >> bit) & 1 == 1] |= np.uint32(1 << new_var_order[bit])
    for bit in range(n - half):
        hi[(np.arange(1 << (n - half)) >> bit) & 1 == 1] |= np.uint32(1 << new_var_order[half + bit])
    return lo, hi


class LayerProver:
    """Runs einsum proofs of a trace on one device through the almost-Goldilocks C-ABI."""

    def __init__(self, lib):
        self.lib = lib
        self._cache = {}

    def _dev(self, arr):
        return DeviceBuffer.from_numpy(self.lib, np.ascontiguousarray(arr))

    def _eq_table(self, r):
        """eq(r, x) over {0,1}^len(r) as (buffer holding it, device pointer); bit k of x goes with r[k]."""
        lib, log_n = self.lib, len(r)
        a, b = DeviceBuffer(lib, 16 << log_n), DeviceBuffer(lib, 16 << log_n)
        d_r, res = self._dev(r), ctypes.c_void_p()
        rc = lib.aext2_eq_dp_all_ffi(d_r.ptr, a.ptr, b.ptr, log_n, ctypes.byref(res))
        if rc != 0:
            raise RuntimeError("aext2_eq_dp_all_ffi failed: %d" % rc)
        return (a, b, d_r), res.value

    def _tile(self, ptr, have_log, want_log):
        """Repeat the first 2^have_log extension elements up to 2^want_log (new high variables)."""
        for k in range(have_log, want_log):
            if self.lib.cuda_memcpy_dtod(ptr + (16 << k), ptr, 16 << k) != 0:
                raise RuntimeError("cuda_memcpy_dtod failed")

    def plan(self, equation, dims):
        key = (equation, tuple(sorted(dims.items())))
        if key not in self._cache:
            pl = EinsumPlan(equation, dims)
            pl.luts = []
            for k in range(len(pl.inputs)):
                order, nmine = pl.operand_order(k)
                n = len(order)
                if order == list(range(n)) or n == 0:
                    pl.luts.append(None)
                else:   # index tables live on the device for the life of the prover
                    lo, hi = split_luts(n, order, n // 2)
                    pl.luts.append((self._dev(lo), self._dev(hi)))
            self._cache[key] = pl
        return self._cache[key]

    def prove_einsum(self, equation, dims, operands, point, transcript):
        """operands: device pointers of base-field tables (index order = the equation's letters, last fastest);
        point: uint64 array [output variables][2], low variable first; transcript: agl_transcript handle.
        Returns (round_msgs, challenges, final_evals, final_eval) as numpy arrays."""
        lib, pl = self.lib, self.plan(equation, dims)
        out_bits = _bits(pl.out, pl.dims)
        point = np.asarray(point, dtype=np.uint64).reshape(len(out_bits), 2)
        rounds, d = pl.rounds, len(pl.inputs) + 1
        size = 1 << rounds
        tables, keep = DeviceBuffer(lib, d * size * 16), []
        for k, src in enumerate(operands):
            order, nmine = pl.operand_order(k)
            n, m = len(order), len(pl.fixed[k])
            if pl.table_vars[:nmine] != [v for v in pl.table_vars if v in _bits(pl.inputs[k], pl.dims)]:
                raise ValueError("operand lacks an inner table variable: " + equation)
            dst = tables.ptr + k * size * 16
            r = np.array([point[out_bits.index(v)] for v in pl.fixed[k]], dtype=np.uint64).reshape(m, 2)
            if pl.luts[k] is None and m == 0:
                rc = lib.agl_to_aext2_batch_ffi(src, dst, 1 << n)
            elif pl.luts[k] is None:
                scratch, d_r = DeviceBuffer(lib, 16 << max(n - 1, 0)), self._dev(r)
                keep += [scratch, d_r]
                rc = lib.agl_partial_eval_ext2_from_base_ffi(src, scratch.ptr, d_r.ptr, n, m)
                rc |= lib.cuda_memcpy_dtod(dst, scratch.ptr, 16 << (n - m))
            else:
                if m:
                    bufs, eq_ptr = self._eq_table(r)
                else:
                    bufs = self._dev(np.array([1, 0], dtype=np.uint64))
                    eq_ptr = bufs.ptr
                keep.append(bufs)
                lo, hi = pl.luts[k]
                rc = lib.agl_fused_permute_partial_eval_ffi(src, dst, eq_ptr, lo.ptr, hi.ptr, n, m, n // 2, 1 << (n - m), 0)
            if rc != 0:
                raise RuntimeError("operand %d of %s failed: %d" % (k, equation, rc))
            self._tile(dst, nmine, rounds)
        dst = tables.ptr + (d - 1) * size * 16
        if pl.shared:
            r = np.array([point[out_bits.index(v)] for v in pl.shared], dtype=np.uint64)
            bufs, eq_ptr = self._eq_table(r)
            keep.append(bufs)
            if lib.cuda_memcpy_dtod(dst, eq_ptr, 16 << len(pl.shared)) != 0:
                raise RuntimeError("cuda_memcpy_dtod failed")
            self._tile(dst, len(pl.shared), rounds)
        else:
            ones = np.zeros(2 * size, dtype=np.uint64)
            ones[0::2] = 1
            if lib.cuda_memcpy_htod(dst, ones.ctypes.data, ones.nbytes) != 0:
                raise RuntimeError("cuda_memcpy_htod failed")
        msgs = np.zeros(max(rounds, 1) * (d + 1) * 2, dtype=np.uint64)
        ch = np.zeros(max(rounds, 1) * 2, dtype=np.uint64)
        fe, fin = np.zeros(2 * d, dtype=np.uint64), np.zeros(2, dtype=np.uint64)
        rc = lib.agl_sumcheck_prove_device_ffi(tables.ptr, d, rounds, 0, transcript, msgs.ctypes.data, ch.ctypes.data,
                                               fe.ctypes.data, fin.ctypes.data)
        if rc != 0:
            raise RuntimeError("sumcheck of %s failed: %d" % (equation, rc))
        return msgs[:rounds * (d + 1) * 2], ch[:2 * rounds], fe, fin


class _EinsumOperand(ctypes.Structure):
    """mb_einsum_operand of include/almost_goldilocks_cuda_wrapper.h."""
    _fields_ = [("d_src", ctypes.c_void_p), ("d_lut_lo", ctypes.c_void_p), ("d_lut_hi", ctypes.c_void_p),
                ("n", ctypes.c_int), ("m", ctypes.c_int), ("fixed_off", ctypes.c_int), ("reserved", ctypes.c_int)]


def _native_plan(prover, equation, dims):
    """The flat form of a plan that agl_einsum_prove_device_ffi takes: operand records (sources filled per call),
    the indices of every operand's fixed output variables and of the shared ones. Cached on the plan."""
    pl = prover.plan(equation, dims)
    if getattr(pl, "native", None) is None:
        out_bits = _bits(pl.out, pl.dims)
        ops = (_EinsumOperand * len(pl.inputs))()
        fixed = []
        for k in range(len(pl.inputs)):
            order, nmine = pl.operand_order(k)
            if pl.table_vars[:nmine] != [v for v in pl.table_vars if v in _bits(pl.inputs[k], pl.dims)]:
                raise ValueError("operand lacks an inner table variable: " + equation)
            ops[k].n, ops[k].m, ops[k].fixed_off = len(order), len(pl.fixed[k]), len(fixed)
            if pl.luts[k] is not None:
                ops[k].d_lut_lo, ops[k].d_lut_hi = pl.luts[k][0].ptr, pl.luts[k][1].ptr
            fixed += [out_bits.index(v) for v in pl.fixed[k]]
        pl.native = (ops, (ctypes.c_int * max(len(fixed), 1))(*fixed),
                     (ctypes.c_int * max(len(pl.shared), 1))(*[out_bits.index(v) for v in pl.shared]), len(out_bits))
    return pl


def prove_einsum_native(prover, equation, dims, operands, point, transcript):
    """LayerProver.prove_einsum with the whole device sequence inside the library (agl_einsum_prove_device_ffi):
    one call per einsum block, nothing synchronises before the sumcheck's first message. Same outputs."""
    lib = prover.lib
    pl = _native_plan(prover, equation, dims)
    ops, fixed, shared, nvars = pl.native
    for k, src in enumerate(operands):
        ops[k].d_src = src
    point = np.ascontiguousarray(point, dtype=np.uint64).reshape(nvars, 2)
    rounds, d = pl.rounds, len(pl.inputs) + 1
    msgs = np.zeros(max(rounds, 1) * (d + 1) * 2, dtype=np.uint64)
    ch = np.zeros(max(rounds, 1) * 2, dtype=np.uint64)
    fe, fin = np.zeros(2 * d, dtype=np.uint64), np.zeros(2, dtype=np.uint64)
    rc = lib.agl_einsum_prove_device_ffi(len(pl.inputs), ops, fixed, rounds, len(pl.shared), shared, point.ctypes.data, nvars,
                                         transcript, msgs.ctypes.data, ch.ctypes.data, fe.ctypes.data, fin.ctypes.data)
    if rc != 0:
        raise RuntimeError("agl_einsum_prove_device_ffi of %s failed: %d" % (equation, rc))
    return msgs[:rounds * (d + 1) * 2], ch[:2 * rounds], fe, fin


def synthetic_operand(seed, n_log):
    """2^n_log fixed-point values in [-2^15, 2^15) as canonical field elements (negatives as q - |v|)."""
    v = (splitmix64(seed, 1 << n_log) & np.uint64(0xFFFF)).astype(np.int64) - (1 << 15)
    return np.where(v < 0, np.uint64(AGL_Q) - (-v).astype(np.uint64), v.astype(np.uint64)).astype(np.uint64)
