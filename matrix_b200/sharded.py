"""Batched degree-3 sumcheck (shared eq table, K instances combined with powers
of alpha) sharded over the top hypercube variables, one shard per rank.

    S = sum_k alpha^k sum_x eq(t, x) a_k(x) b_k(x),   x in {0,1}^nv

Rank g of G = 2^g_bits holds the slices of a_k, b_k whose top g_bits index bits
equal g. The sumcheck binds the low variable first, so the first nv - g_bits
rounds are local: every rank computes its share of the round polynomial on its
GPU, the shares (4 extension elements = 64 bytes per rank) are exchanged with
one all-gather and added mod p, every rank runs the same transcript and folds
on the same challenge. After the local rounds each rank is left with one value
per table; these are all-gathered and the last g_bits rounds are finished on the
host, identically on every rank. There is no other data-path communication.

The reference runs this kernel family on one GPU per task and adds partial sums
on the host (almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:351-385); sharding
one sumcheck over several GPUs has no reference counterpart.
"""
import ctypes

import numpy as np

GL_P = 0xFFFFFFFF00000001
W = 7  # X^2 = 7


# ---- extension-field helpers on Python integers (a few dozen values per round) ----
def e2_add(a, b):
    return ((a[0] + b[0]) % GL_P, (a[1] + b[1]) % GL_P)


def e2_sub(a, b):
    return ((a[0] - b[0]) % GL_P, (a[1] - b[1]) % GL_P)


def e2_mul(a, b):
    return ((a[0] * b[0] + W * a[1] * b[1]) % GL_P, (a[0] * b[1] + a[1] * b[0]) % GL_P)


def e2_inv(a):
    n = (a[0] * a[0] - W * a[1] * a[1]) % GL_P
    ni = pow(n, GL_P - 2, GL_P)
    return (a[0] * ni % GL_P, (-a[1]) * ni % GL_P)


def eq_scale(point_top, shard):
    """eq(t_top, bits of shard): bit i of the shard index pairs with point_top[i]."""
    s = (1, 0)
    for i, t in enumerate(point_top):
        s = e2_mul(s, t if (shard >> i) & 1 else e2_sub((1, 0), t))
    return s


class SingleComm:
    """All `world` shards live in this process (one GPU simulating several ranks, or world = 1)."""

    def __init__(self, world=1):
        self.world = world
        self.local_ranks = list(range(world))

    def allgather(self, arrs):
        return [np.array(a, dtype=np.uint64) for a in arrs]


class TorchComm:
    """All-gather of small uint64 arrays over torch.distributed (NCCL between GPUs, gloo on CPU)."""

    def __init__(self, device=None):
        import torch.distributed as dist
        self.dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.local_ranks = [self.rank]
        self.device = device
        self._bufs = {}

    def allgather(self, arrs):
        """Every rank's array, in rank order. Staging buffers (pinned host, device) are kept per length."""
        import torch
        a = np.ascontiguousarray(arrs[0], dtype=np.uint64)
        n = a.size
        buf = self._bufs.get(n)
        if buf is None:
            pin = self.device is not None
            h_in = torch.empty(n, dtype=torch.int64, pin_memory=pin)
            h_out = torch.empty(n * self.world, dtype=torch.int64, pin_memory=pin)
            d_in = torch.empty(n, dtype=torch.int64, device=self.device) if pin else h_in
            d_out = torch.empty(n * self.world, dtype=torch.int64, device=self.device) if pin else h_out
            buf = self._bufs[n] = (h_in, h_out, d_in, d_out)
        h_in, h_out, d_in, d_out = buf
        h_in.numpy()[:] = a.view(np.int64)
        if self.device is not None:
            d_in.copy_(h_in, non_blocking=True)
        self.dist.all_gather_into_tensor(d_out, d_in)
        if self.device is not None:
            h_out.copy_(d_out, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
        res = h_out.numpy().view(np.uint64).reshape(self.world, n)
        return [res[g].copy() for g in range(self.world)]


class ShmComm:
    """All-gather of small uint64 arrays between the processes of one node through a file in shared memory
    (a mailbox per rank and call parity: sequence number, then payload). A round message is a few dozen
    bytes that already sit on the host, so a host-side exchange costs microseconds where a collective
    through the GPUs costs a launch, two copies and a synchronisation per round. Waits are bounded."""

    MAX_WORDS = 1024

    def __init__(self, path, rank, world, timeout_s=120.0):
        import mmap
        import os
        self.rank, self.world, self.timeout = rank, world, timeout_s
        self.local_ranks = [rank]
        self.row = 1 + self.MAX_WORDS
        size = 8 * world * 2 * self.row
        if rank == 0:
            with open(path + ".tmp", "wb") as f:
                f.write(b"\0" * size)
            os.replace(path + ".tmp", path)  # appears fully zeroed
        import time
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > timeout_s:
                raise TimeoutError("mailbox file %s did not appear" % path)
            time.sleep(0.001)
        self.f = open(path, "r+b")
        self.mm = mmap.mmap(self.f.fileno(), size)
        self.box = np.frombuffer(self.mm, dtype=np.uint64).reshape(world, 2, self.row)
        self.seq = 0

    def allgather(self, arrs):
        import time
        a = np.ascontiguousarray(arrs[0], dtype=np.uint64)
        assert a.size <= self.MAX_WORDS
        self.seq += 1
        slot = self.seq & 1
        mine = self.box[self.rank, slot]
        mine[1:1 + a.size] = a
        mine[0] = self.seq  # published after the payload
        out = []
        t0 = None
        for g in range(self.world):
            spins = 0
            while int(self.box[g, slot, 0]) != self.seq:
                spins += 1
                if spins & 0xFFF == 0:
                    t0 = t0 or time.time()
                    if time.time() - t0 > self.timeout:
                        raise TimeoutError("rank %d did not publish call %d" % (g, self.seq))
            out.append(self.box[g, slot, 1:1 + a.size].copy())
        return out


class LibTranscript:
    """The library's host transcript (zk-torch-3/src/transcript.rs semantics) through the C-ABI."""

    def __init__(self, lib, label):
        self.lib = lib
        self.h = ctypes.c_void_p()
        assert lib.gl_transcript_create(label, len(label), ctypes.byref(self.h)) == 0

    def append_u64(self, label, v):
        self.lib.gl_transcript_append_u64(self.h, label, int(v))

    def append_ext2(self, label, v):
        self.lib.gl_transcript_append_ext2(self.h, label, int(v[0]), int(v[1]))

    def challenge_ext2(self, label):
        out = (ctypes.c_uint64 * 2)()
        self.lib.gl_transcript_challenge_ext2(self.h, label, out)
        return (int(out[0]), int(out[1]))

    def state(self):
        out = np.zeros(8, dtype=np.uint64)
        self.lib.gl_transcript_state(self.h, out.ctypes.data)
        return out

    def __del__(self):
        try:
            self.lib.gl_transcript_destroy(self.h)
        except Exception:
            pass


class GpuShard:
    """One shard on the current CUDA device through the C-ABI (gl_batched_state_*)."""

    def __init__(self, lib, d_a_ptr, d_b_ptr, point_low, scale, K, n_loc):
        self.lib, self.K = lib, K
        self.h = ctypes.c_void_p()
        pl = np.array([c for t in point_low for c in t], dtype=np.uint64)
        sc = np.array(scale, dtype=np.uint64)
        rc = lib.gl_batched_state_create(d_a_ptr, d_b_ptr, pl.ctypes.data, sc.ctypes.data, K, n_loc, ctypes.byref(self.h))
        if rc != 0:
            raise RuntimeError("gl_batched_state_create: %d" % rc)

    def claims(self):
        out = np.zeros(2 * self.K, dtype=np.uint64)
        assert self.lib.gl_batched_state_claims(self.h, out.ctypes.data) == 0
        return out

    def set_alpha(self, alpha):
        assert self.lib.gl_batched_state_set_alpha(self.h, alpha[0], alpha[1]) == 0

    def round_message(self):
        out = np.zeros(8, dtype=np.uint64)
        assert self.lib.gl_batched_state_round_message(self.h, out.ctypes.data) == 0
        return out

    def fold(self, r):
        assert self.lib.gl_batched_state_fold(self.h, r[0], r[1]) == 0

    def finals(self):
        out = np.zeros(2 * (2 * self.K + 1), dtype=np.uint64)
        assert self.lib.gl_batched_state_finals(self.h, out.ctypes.data) == 0
        return out

    def close(self):
        if self.h:
            self.lib.gl_batched_state_destroy(self.h)
            self.h = None


def _sum_shares(shares, width):
    """Adds the ranks' arrays of `width` extension elements mod p."""
    tot = [(0, 0)] * width
    for s in shares:
        tot = [e2_add(t, (int(s[2 * i]), int(s[2 * i + 1]))) for i, t in enumerate(tot)]
    return tot


def prove_sharded(make_shard, transcript, comm, point, K, nv, g_bits):
    """Runs the protocol. `make_shard(rank, point_low, scale)` builds the shard object of a
    rank this process owns (GpuShard or a test double with the same methods); `transcript`
    follows LibTranscript; `point` is a list of nv (c0, c1) pairs. Returns the same
    dictionary on every process."""
    assert comm.world == 1 << g_bits and nv - g_bits >= 1
    n_loc = nv - g_bits
    shards = [make_shard(g, point[:n_loc], eq_scale(point[n_loc:], g)) for g in comm.local_ranks]
    transcript.append_u64(b"sp_num_var", nv)
    transcript.append_u64(b"sp_num_inst", K)
    claims = _sum_shares(comm.allgather([s.claims() for s in shards]), K)
    for c in claims:
        transcript.append_ext2(b"sp_y_i", c)
    alpha = transcript.challenge_ext2(b"sp_alpha")
    for s in shards:
        s.set_alpha(alpha)
    round_msgs, challenges = [], []
    for _ in range(n_loc):
        msg = _sum_shares(comm.allgather([s.round_message() for s in shards]), 4)
        for m in msg:
            transcript.append_ext2(b"sp_round_msg", m)
        r = transcript.challenge_ext2(b"sp_round_challenge")
        round_msgs.append(msg)
        challenges.append(r)
        for s in shards:
            s.fold(r)
    # one value per table and rank: eq, alpha^k a_k, b_k; finish the top variables on the host
    gathered = comm.allgather([s.finals() for s in shards])
    T = 2 * K + 1
    tables = [[(int(g[2 * i]), int(g[2 * i + 1])) for g in gathered] for i in range(T)]
    size = comm.world
    while size > 1:
        half = size // 2
        msg = []
        for c in range(4):
            tot = (0, 0)
            cc = (c, 0)
            for y in range(half):
                def at(tab):
                    lo, hi = tab[2 * y], tab[2 * y + 1]
                    return e2_add(lo, e2_mul(cc, e2_sub(hi, lo)))
                inner = (0, 0)
                for k in range(K):
                    inner = e2_add(inner, e2_mul(at(tables[1 + k]), at(tables[1 + K + k])))
                tot = e2_add(tot, e2_mul(at(tables[0]), inner))
            msg.append(tot)
        for m in msg:
            transcript.append_ext2(b"sp_round_msg", m)
        r = transcript.challenge_ext2(b"sp_round_challenge")
        round_msgs.append(msg)
        challenges.append(r)
        tables = [[e2_add(t[2 * y], e2_mul(r, e2_sub(t[2 * y + 1], t[2 * y]))) for y in range(half)] for t in tables]
        size = half
    # report a_k(R) without the alpha^k factor the shards carry
    finals = [tables[0][0]]
    pw, acc = (1, 0), (0, 0)
    for k in range(K):
        finals.append(e2_mul(tables[1 + k][0], e2_inv(pw)))
        acc = e2_add(acc, e2_mul(tables[1 + k][0], tables[1 + K + k][0]))
        pw = e2_mul(pw, alpha)
    finals += [tables[1 + K + k][0] for k in range(K)]
    for f in finals:
        transcript.append_ext2(b"sp_f_eval", f)
    final_eval = e2_mul(tables[0][0], acc)
    for s in shards:
        if hasattr(s, "close"):
            s.close()
    return dict(claims=np.array(claims, dtype=np.uint64), alpha=np.array(alpha, dtype=np.uint64),
                round_msgs=np.array(round_msgs, dtype=np.uint64), challenges=np.array(challenges, dtype=np.uint64),
                finals=np.array(finals, dtype=np.uint64), final_eval=np.array(final_eval, dtype=np.uint64),
                state=transcript.state())


def prove_batched_native(lib, exchange, d_a_ptr, d_b_ptr, K, nv, point, label, timing=False):
    """The same protocol as prove_sharded with the whole round loop inside the library
    (gl_batched_prove_sharded): one call per rank, the ranks' shares exchanged through `exchange` (an
    mb_exchange handle: mb_exchange_local_create for threads of one process, MailboxExchange /
    ProcessExchange for one process per GPU). `d_a_ptr`, `d_b_ptr`: this rank's slices [K][2^(nv - log2 world)]
    on the current device. Returns the dictionary prove_sharded returns; with `timing` (and MB_SHARD_TIMING set
    in the environment) also `round_us` = microseconds per local round in (kernel wait, exchange, host)."""
    pt = np.array([c for t in point for c in t], dtype=np.uint64)
    out = dict(claims=np.zeros((K, 2), dtype=np.uint64), alpha=np.zeros(2, dtype=np.uint64),
               round_msgs=np.zeros((nv, 4, 2), dtype=np.uint64), challenges=np.zeros((nv, 2), dtype=np.uint64),
               finals=np.zeros((2 * K + 1, 2), dtype=np.uint64), final_eval=np.zeros(2, dtype=np.uint64),
               state=np.zeros(8, dtype=np.uint64))
    us = np.zeros(3, dtype=np.float64)
    rc = lib.gl_batched_prove_sharded(exchange, d_a_ptr, d_b_ptr, K, nv, pt.ctypes.data, label, len(label),
                                      out["claims"].ctypes.data, out["alpha"].ctypes.data, out["round_msgs"].ctypes.data,
                                      out["challenges"].ctypes.data, out["finals"].ctypes.data, out["final_eval"].ctypes.data,
                                      out["state"].ctypes.data, us.ctypes.data)
    if rc != 0:
        raise RuntimeError("gl_batched_prove_sharded: %d" % rc)
    if timing:
        out["round_us"] = us
    return out


class MailboxExchange:
    """An mb_exchange for one process per GPU on one machine whose provers exchange host words only (the batched
    sumcheck): the library's mailbox in POSIX shared memory, no device all-to-all. `name` must be the same on
    every rank and unused by any other run."""

    def __init__(self, lib, name, rank, world, slot_words=1024):
        self.lib = lib
        h = ctypes.c_void_p()
        rc = lib.mb_exchange_shm_create(name.encode(), rank, world, slot_words, None, None, ctypes.byref(h))
        if rc != 0:
            raise RuntimeError("mb_exchange_shm_create: %d" % rc)
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mb_exchange_destroy(self.handle)
            self.handle = None


# ---- Ajtai commitment sharded by column ranges -------------------------------------------------
AGL_Q = 0xFFFFFFFEFFFFFFE1


def column_range(n_ring, world, rank):
    """Ring columns [lo, hi) of `rank`: contiguous, as even as possible."""
    base, extra = divmod(n_ring, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _add_mod_q(a, b):
    """(a + b) mod q on uint64 arrays of canonical residues, without leaving 64-bit arithmetic."""
    q = np.uint64(AGL_Q)
    b = np.where(b >= q, b - q, b)
    s = a + b                      # wraps mod 2^64
    wrapped = s < a
    return np.where(wrapped | (s >= q), s - q, s)   # after a wrap s - q wraps back to the true a + b - q


def _sum_column_shards(commit_columns, comm, ncols, words):
    """All-gathers the ranks' partial results over their column ranges and adds them mod q."""
    parts = []
    for g in comm.local_ranks:
        lo, hi = column_range(ncols, comm.world, g)
        part = np.ascontiguousarray(commit_columns(lo, hi), dtype=np.uint64).reshape(-1)
        assert part.size == words
        parts.append(part)
    gathered = comm.allgather(parts)
    total = np.zeros(words, dtype=np.uint64)
    for p in gathered:
        total = _add_mod_q(total, np.asarray(p, dtype=np.uint64).reshape(-1))
    return total


def link_round_sharded(round_commitments, comm, n_commit):
    """The link round message is a sum over commitments (cuda_almost_goldilocks/link_sumcheck.cuh:16-19: a
    partition of the commitment axis with a 7-element all-reduce): every rank forms the message of its own
    range of commitments, the 14 words per rank are all-gathered and added mod q. `round_commitments(lo, hi)`
    returns [S(0..3), E(0..2)] over commitments lo..hi (zeros for an empty range). Same array everywhere;
    the ranks then fold their own tables with the same challenge, no further exchange."""
    return _sum_column_shards(round_commitments, comm, n_commit, 14)


def module_commit_sharded(commit_columns, comm, ncols, vectors, rows):
    """The module commitment over F_q[Y]/(Y^4096 + 1) is a sum over key columns
    (zk-torch-4/src/morpheus/commit_gpu.rs:1-8: partial per column range and GPU, then add): every rank
    builds the key cache of its own column range (`col0` of agl_mcommit_keygen), commits its columns and
    finishes; each shard's integer is exact on its own, so the finished words (vectors x rows x 4096) add
    mod q. `commit_columns(lo, hi)` returns this rank's finished partial commitment (zeros for an empty
    range, without the identity error, which the caller adds once). Same array on every process."""
    return _sum_column_shards(commit_columns, comm, ncols, vectors * rows * 4096)


def commit_sharded(commit_columns, comm, n_ring, planes):
    """c = sum_j M[:, j] z_j is a sum over columns: every rank commits its own column range against the
    matching window of the matrix (`col_offset`, the reference's ajtai_commit_dense_batched_at_ffi,
    almost-goldilocks-cuda-rs/src/ffi.rs:500-508; sharding design almost-goldilocks-cuda-rs tests
    ajtai_integration.rs:296-328), the partial commitments (planes x 42 x 64 words) are all-gathered and added
    mod q. `commit_columns(lo, hi)` returns this rank's partial commitment as a uint64 array (zeros for an
    empty range). Returns the same array on every process."""
    return _sum_column_shards(commit_columns, comm, n_ring, planes * 42 * 64)


# ---- one Basefold proof over several processes ------------------------------------------------------
class _RawDeviceWords:
    """A view of `words` 64-bit words of device memory for torch.as_tensor (CUDA array interface, no copy)."""

    def __init__(self, ptr, words):
        self.__cuda_array_interface__ = {"shape": (int(words),), "typestr": "<i8", "data": (int(ptr), False), "version": 2}


class ProcessExchange:
    """The exchange object of the sharded Basefold prover for one process per GPU on one machine: the host words of
    every round go through the library's mailbox in POSIX shared memory, the device all-to-all of the commit phase
    is one torch.distributed all_to_all_single (NCCL) on the caller's process group.

    `name` must be the same on every rank and unused by any other run (e.g. derived from MASTER_PORT); `device` is
    this rank's torch device. Keep the object alive while the exchange is in use: it owns the callback."""

    A2A = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t)

    def __init__(self, lib, name, rank, world, device, slot_words=1 << 17):
        import torch
        import torch.distributed as dist
        self.lib, self.rank, self.world = lib, rank, world
        self.calls = 0

        def all_to_all(_ctx, d_send, d_recv, words_per_rank):
            try:
                total = words_per_rank * world
                send = torch.as_tensor(_RawDeviceWords(d_send, total), device=device)
                recv = torch.as_tensor(_RawDeviceWords(d_recv, total), device=device)
                dist.all_to_all_single(recv, send)
                torch.cuda.synchronize(device)
                self.calls += 1
                return 0
            except Exception as exc:  # an exception must not cross the C boundary
                import sys
                sys.stderr.write("ProcessExchange.all_to_all failed: %r\n" % (exc,))
                return -4

        self._cb = self.A2A(all_to_all)
        h = ctypes.c_void_p()
        rc = lib.mb_exchange_shm_create(name.encode(), rank, world, slot_words, ctypes.cast(self._cb, ctypes.c_void_p), None,
                                        ctypes.byref(h))
        if rc != 0:
            raise RuntimeError("mb_exchange_shm_create: %d" % rc)
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mb_exchange_destroy(self.handle)
            self.handle = None
