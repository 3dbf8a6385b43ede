#!/usr/bin/env python
"""Benchmark of the Basefold commit + opening path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--num-vars NV]

Workload (one "step"): commit to one multilinear polynomial of 2^24
uniform-random Goldilocks evaluations (seed 3 + rank) at code rate 1/2
(codeword 2^25), Poseidon2 Merkle trees, then the extension-field opening at a
seeded point (24 fold rounds, Poseidon2 Fiat-Shamir transcript, 100 queries).
The folding table (seed 42) is key material: built once, outside the timed
region, as in the reference. Synthetic seeded inputs (splitmix64 mod p).

Printed on one JSON line:
  value    field elements committed and opened per second, evaluations already
           resident in HBM when the timed region starts;
  e2e      the same through the host-buffer entry point basefold_prove_host:
           host->device copy of the evaluations and device->host copy of the
           proof inside the timed region;
  roofline the dominant kernel by device time (CUDA events around every launch
           of the timed region) against the measured HBM peak;
  cpu_baseline  the CPU oracle (a C restatement of the reference's CPU
           prover) on a bounded sample, all host cores.
The N = 1 line also carries `parts`: the linear sumcheck of f * g at 2^24 and
the Ajtai ring commit at 2^18 ring columns, each with its own roofline, e2e and
CPU figure (the metric names all three paths).
With N > 1 (launched by torch.distributed.run) the SAME single polynomial is
partitioned over the N GPUs (strong scaling: contiguous ranges of the
evaluations and of every codeword, one device all-to-all per proof, one gather
of 10 words per rank and round); `replicas` beside it is N independent provers.
Timed regions run without per-kernel events; kernel times come from a separate
pass. `--impl reference` times the CPU oracle alone on the host cores, at the
full size.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "field-elems/s: Basefold commit+open (Poseidon2 Merkle, rate 1/2, 100 queries), Goldilocks"
UNIT = "field-elems/s"
LOG_RATE = 1
NUM_QUERIES = 100
LABEL = b"bench"


def pinned_copy(lib, arr):
    """The array's bytes in page-locked host memory (what a step's inputs are copied from in the end-to-end legs)."""
    p = ctypes.c_void_p()
    assert lib.mb_host_alloc(ctypes.byref(p), arr.nbytes) == 0
    ctypes.memmove(p.value, arr.ctypes.data, arr.nbytes)
    return p.value


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi. It is started before the warm-up (nvidia-smi takes
    a while to print its first line) and asked for the samples that fall inside the timed region; when the region
    was shorter than the sampling period, the samples taken under the same load just before it are used and the
    answer says so."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.t_load = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        self.t_load = time.time()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.06)   # let the sample that covers the end of the region arrive
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        for t, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                rows.append((t, float(parts[2]), float(parts[3]), parts[6:10]))
            except ValueError:
                continue
        t0 = self.t0 if self.t0 is not None else self.t_load
        t1 = (self.t1 if self.t1 is not None else time.time()) + 0.06
        inside = [r for r in rows if t0 <= r[0] <= t1]
        window = "timed region"
        if not inside:
            inside = [r for r in rows if r[0] >= (self.t_load or 0)]
            window = "warm-up and timed region (the timed region is shorter than the sampling period)"
        reasons = set()
        for r in inside:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median([r[1] for r in inside])) if inside else None,
                "sm_max_mhz": max(r[2] for r in inside) if inside else None,
                "reasons": sorted(reasons), "samples": len(inside), "window": window}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def cpu_oracle_sample(num_vars, threads=None, merkle_hash="poseidon2"):
    """One commit + open of the CPU oracle at 2^num_vars; returns seconds and thread count."""
    from matrix_b200.inputs import field_elems
    from oracle import pyoracle
    # every host core, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1 for N > 1)
    pyoracle.load().oracle_set_threads(threads or os.cpu_count() or 1)
    pyoracle.load().oracle_set_merkle_hash(1 if merkle_hash == "monolith" else 0)
    evals = field_elems(3, 1 << num_vars)
    point = field_elems(4, 2 * num_vars)
    table = pyoracle.bf_table(num_vars, LOG_RATE)  # key material, untimed
    t0 = time.perf_counter()
    cw, bh, tree = pyoracle.bf_commit(evals, num_vars, LOG_RATE)
    proof, _ = pyoracle.bf_open(cw, bh, tree, num_vars, LOG_RATE, point, table, NUM_QUERIES, LABEL)
    dt = time.perf_counter() - t0
    return dt, proof


def run_reference(args):
    """The reference arm: the CPU prover (oracle port) on the host cores, rank 0 only. Steps run at the full size
    (2^num_vars) while a time budget lasts, at least one; a small sample is reported beside them."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    nv, snv = args.num_vars, min(args.ref_num_vars, args.num_vars)
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_sample(min(snv, 16), merkle_hash=args.hash)
    dt_small, _ = cpu_oracle_sample(snv, merkle_hash=args.hash)
    budget = float(os.environ.get("MB_REFERENCE_BUDGET_S", "150"))
    times = []
    t_begin = time.perf_counter()
    while len(times) < args.steps:
        dt, _ = cpu_oracle_sample(nv, merkle_hash=args.hash)
        times.append(dt)
        if time.perf_counter() - t_begin + dt > budget:
            break
    total = sum(times)
    value = (1 << nv) * len(times) / total
    line = {
        "impl": "reference",
        "metric": METRIC if args.hash == "poseidon2" else METRIC.replace("Poseidon2 Merkle", "Monolith Merkle"),
        "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "steps_run_at_full_size": len(times),
        "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "u64",
        "data": "synthetic",
        "config": basefold_config(nv, args.hash, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "CPU oracle (C restatement of the reference's CPU prover, OpenMP on %d cores) commit+open at the "
                                   "full 2^%d evaluations, %d step(s) of %.1f s each inside a %.0f s budget; table generation "
                                   "excluded; a 2^%d sample ran at %.3e elements/s" %
                                   (cores, nv, len(times), total / len(times), budget, snv, (1 << snv) / dt_small)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_batched(args):
    """Config 4: K instances of eq*a*b over 2^nv points, combined with powers of alpha, one proof sharded over
    the top log2(N) variables (strong scaling). Default driver: the whole round loop inside the library
    (gl_batched_prove_sharded), the ranks' 64-byte shares of every round polynomial exchanged through the
    library's mailbox in POSIX shared memory. --exchange nccl / shm keep the Python round loop over an NCCL
    all-gather or a mailbox file."""
    rank, world, local = dist_env()
    from matrix_b200 import load_gl
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import GL_P, field_elems
    from matrix_b200.sharded import (GpuShard, LibTranscript, MailboxExchange, SingleComm, TorchComm, prove_batched_native,
                                     prove_sharded)
    lib = load_gl()
    assert lib.cuda_set_device(local) == 0
    nv = args.num_vars if args.num_vars != 24 else 26
    K = args.instances
    g_bits = world.bit_length() - 1
    assert world == 1 << g_bits, "the number of ranks must be a power of two"
    native = args.exchange == "mailbox"
    comm = SingleComm(1)
    dist, exch, handle = None, None, None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))   # timing barrier and max over ranks
        if native:
            token = [os.urandom(6).hex() if rank == 0 else None]   # a fresh name: a mailbox left by a killed run is never reused
            dist.broadcast_object_list(token, src=0)
            exch = MailboxExchange(lib, "/mb_batched_%s" % token[0], rank, world)
            handle = exch.handle
            dist.barrier()
        else:
            comm = TorchComm(device=torch.device("cuda", local))
            if args.exchange == "shm":
                from matrix_b200.sharded import ShmComm
                path = "/dev/shm/matrix_b200_mailbox_%s" % os.environ.get("MASTER_PORT", "0")
                if rank == 0 and os.path.exists(path):
                    os.remove(path)
                dist.barrier()
                comm = ShmComm(path, rank, world)
    elif native:
        exs = (ctypes.c_void_p * 1)()
        assert lib.mb_exchange_local_create(1, exs) == 0
        handle = exs[0]
    n_loc = nv - g_bits
    m = 1 << n_loc
    # this rank's slices, made on the device: instance k, table a / b, entries [rank * m, (rank + 1) * m)
    d_a, d_b = DeviceBuffer(lib, 8 * K * m), DeviceBuffer(lib, 8 * K * m)
    for k in range(K):
        # seeds 100 + k / 200 + k; the slice of a longer stream starts at element rank * m
        off = (rank * m * 0x9E3779B97F4A7C15) & (2**64 - 1)
        assert lib.mb_fill_splitmix(d_a.ptr + 8 * k * m, m, (100 + k + off) & (2**64 - 1), GL_P) == 0
        assert lib.mb_fill_splitmix(d_b.ptr + 8 * k * m, m, (200 + k + off) & (2**64 - 1), GL_P) == 0
    pt = field_elems(6, 2 * nv)
    point = [(int(pt[2 * i]), int(pt[2 * i + 1])) for i in range(nv)]

    def step(timing=False):
        if native:
            return prove_batched_native(lib, handle, d_a.ptr, d_b.ptr, K, nv, point, LABEL, timing=timing)
        return prove_sharded(lambda g, pl, sc: GpuShard(lib, d_a.ptr, d_b.ptr, pl, sc, K, n_loc),
                             LibTranscript(lib, LABEL), comm, point, K, nv, g_bits)

    def barrier():
        if dist is not None:
            dist.barrier()
        lib.cuda_device_synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    a, b = ctypes.c_void_p(), ctypes.c_void_p()
    lib.mb_event_create(ctypes.byref(a)); lib.mb_event_create(ctypes.byref(b))
    lib.mb_prof_enable(0)
    launches0 = lib.mb_launch_count()
    barrier()
    sampler.mark_begin()
    lib.mb_event_record(a)
    for _ in range(args.steps):
        proof = step()
    lib.mb_event_record(b); lib.mb_event_sync(b)
    sampler.mark_end()
    barrier()
    ms = ctypes.c_float(); lib.mb_event_elapsed_ms(a, b, ctypes.byref(ms))
    val = ms.value
    launches = lib.mb_launch_count() - launches0
    if dist is not None:
        import torch
        t = torch.tensor([val], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        val = float(t.item())
    # per-kernel times and per-round costs: a separate pass, outside the timed region
    psteps = min(args.steps, 3)
    os.environ["MB_SHARD_TIMING"] = "1"
    lib.mb_prof_reset(); lib.mb_prof_enable(1)
    barrier()
    for _ in range(psteps):
        timed_proof = step(timing=True)
    barrier()
    lib.mb_prof_enable(0)
    os.environ.pop("MB_SHARD_TIMING", None)
    clocks = sampler.stop()
    kernels = prof_report(lib)
    elems = 2 * K * (1 << nv)  # field elements of the 2K witness tables (eq is derived, not counted)
    peak, peak_kind = measured_peaks()
    # algorithmic bytes of the dominant pass (fold of round 0 fused with message 1): read 8 B, write 8 B per element
    roofline = None
    if "batched_fold_message" in kernels:
        cnt, kms = kernels["batched_fold_message"]
        # per step and rank: round 0 fold reads 2K*m*8 + eq m*16, writes (2K+1)*m/2*16; later rounds halve: read S, write S/2
        first = 2 * K * m * 8 + m * 16 + (2 * K + 1) * (m // 2) * 16
        later = sum((2 * K + 1) * (m >> r) * 16 * 1.5 for r in range(1, n_loc - 1))
        total_bytes = (first + later) * psteps
        ach = total_bytes / (kms * 1e-3) / 1e9
        roofline = {"kernel": "batched_fold_message", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "traffic": None, "peak_kind": peak_kind, "launches": cnt,
                    "avg_launch_ms": kms / cnt,
                    "timed_in": "a separate pass of %d steps with CUDA events around every launch (not the timed region)" % psteps,
                    "note": "per rank; all rounds' fold+message launches together"}
    kernel_ms = sum(x for _, x in kernels.values()) / psteps
    how = {"mailbox": "round loop inside the library; host mailbox in POSIX shared memory",
           "nccl": "Python round loop; NCCL all-gather", "shm": "Python round loop; mailbox file in /dev/shm"}[args.exchange]
    line = {"metric": "field-elems/s: batched degree-3 sumcheck eq*a*b, %d instances, 2^%d points" % (K, nv),
            "value": elems * args.steps / (val * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": val / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": "batched_sumcheck nv=%d instances=%d" % (nv, K), "sharding": "top %d variables" % g_bits,
                       "collective": "one all-gather of 64 B per rank and round (%s)" % how,
                       "l2": "tables larger than L2"},
            "roofline": roofline,
            "kernel_times_ms": {k: {"launches": c, "ms": round(x, 4)} for k, (c, x) in sorted(kernels.items())},
            "kernel_times_steps": psteps,
            "per_step": {"kernel_ms": kernel_ms, "other_ms": val / args.steps - kernel_ms,
                         "note": "other = launches, read-backs, exchange, transcript and the host rounds (rank 0's kernels)"},
            "gpu_launches": int(launches), "clocks": clocks,
            "final_eval": [int(x) for x in proof["final_eval"]]}
    if native and "round_us" in timed_proof:
        us = [float(x) for x in timed_proof["round_us"]]
        line["round_fixed_cost_us"] = {"kernel_wait": us[0], "exchange": us[1], "recombination_and_transcript": us[2],
                                       "note": "rank 0, microseconds per local round in the per-kernel pass (launch events on)"}
    if rank == 0:
        print(json.dumps(line))
    if exch is not None:
        dist.barrier()
        exch.close()
    elif native and handle is not None:
        lib.mb_exchange_destroy(handle)
    if dist is not None:
        dist.destroy_process_group()


def run_reference_batched(args):
    """CPU arm of the batched sumcheck: the oracle prover on a bounded sample (2^ref_num_vars points)."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from matrix_b200.inputs import field_elems
    from oracle import pyoracle
    pyoracle.load().oracle_set_threads(os.cpu_count() or 1)   # the launcher may have exported OMP_NUM_THREADS=1
    nv, K = args.ref_num_vars, args.instances
    n = 1 << nv
    a = np.concatenate([field_elems(100 + k, n) for k in range(K)])
    b = np.concatenate([field_elems(200 + k, n) for k in range(K)])
    pt = field_elems(6, 2 * nv)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        pyoracle.batched_prove(a, b, pt, K, nv, LABEL)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = 2 * K * n * args.steps / total
    cores = os.cpu_count() or 1
    print(json.dumps({"impl": "reference", "metric": "field-elems/s: batched degree-3 sumcheck eq*a*b, %d instances" % K,
                      "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "strong",
                      "vs_baseline": None, "dtype": "u64", "data": "synthetic",
                      "config": {"workload": "batched_sumcheck instances=%d (sampled at nv=%d)" % (K, nv)},
                      "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                                       "sample": "CPU oracle batched prover at 2^%d points per step" % nv},
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


def _event_timer(lib):
    a, b = ctypes.c_void_p(), ctypes.c_void_p()
    lib.mb_event_create(ctypes.byref(a)); lib.mb_event_create(ctypes.byref(b))

    def timed(fn, reps):
        lib.mb_event_record(a)
        for _ in range(reps):
            fn()
        lib.mb_event_record(b); lib.mb_event_sync(b)
        ms = ctypes.c_float(); lib.mb_event_elapsed_ms(a, b, ctypes.byref(ms))
        return ms.value
    return timed


def run_simple(args):
    """Single-GPU lines for the two other kernels of the path (parity cases in tests/, not the headline):
    sumcheck: one sumcheck of f * g over 2^20 points (base-field tables, extension challenges), tables resident;
    ajtai:    ring commit, 2^18 ring columns (2^24 coefficients), signed 8-bit digit planes on the tensor cores;
    mcommit:  exact module commitment over F_q[Y]/(Y^4096+1): 8192 ternary columns x 16 rows against a resident
              transform-domain key cache, three primes (the shape of the reference's own throughput test,
              zk-torch-4/src/morpheus/commit_gpu.rs:170-186); columns split across the ranks."""
    rank, world, local = dist_env()
    if args.workload == "sumcheck" and rank != 0:
        return
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import field_elems
    peak, peak_kind = measured_peaks()
    dist = None
    if args.workload == "sumcheck":
        from matrix_b200 import load_gl
        lib = load_gl()
        assert lib.cuda_set_device(local) == 0
        nv = args.num_vars if args.num_vars != 24 else 20
        d, n = 2, 1 << (args.num_vars if args.num_vars != 24 else 20)
        polys = np.concatenate([field_elems(1, n), field_elems(2, n)])
        d_t = DeviceBuffer.from_numpy(lib, polys)
        rm, ch = np.zeros((nv, d + 1, 2), dtype=np.uint64), np.zeros((nv, 2), dtype=np.uint64)
        fes, fe = np.zeros((d, 2), dtype=np.uint64), np.zeros(2, dtype=np.uint64)
        step = lambda: lib.gl_sumcheck_prove_device_ffi(d_t.ptr, d, nv, 1, LABEL, len(LABEL), rm.ctypes.data, ch.ctypes.data,
                                                        fes.ctypes.data, fe.ctypes.data, None)
        # end to end: the tables start in page-locked host memory
        h_polys = ctypes.c_void_p()
        assert lib.mb_host_alloc(ctypes.byref(h_polys), polys.nbytes) == 0
        ctypes.memmove(h_polys.value, polys.ctypes.data, polys.nbytes)
        step_e2e = lambda: lib.gl_sumcheck_prove_host_ffi(h_polys.value, d, nv, 1, LABEL, len(LABEL), rm.ctypes.data,
                                                          ch.ctypes.data, fes.ctypes.data, fe.ctypes.data, None)
        units, metric = d * n, "field-elems/s: sumcheck of f*g over 2^%d points, Goldilocks" % nv
        workload = "sumcheck nv=%d d=2" % nv
        alg_bytes = d * n * 8 * (1 + 1 + 1.5 * 2)  # round 0 read; fold read + half-size ext write; later rounds halve
        h2d, d2h = polys.nbytes, rm.nbytes + fe.nbytes
        scaling = "weak"
    elif args.workload == "mcommit":
        from matrix_b200 import load_agl
        from matrix_b200.sharded import SingleComm, TorchComm, column_range, module_commit_sharded
        lib = load_agl()
        assert lib.cuda_set_device(local) == 0
        comm = SingleComm(1)
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            comm = TorchComm(device=torch.device("cuda", local))
        ncols, rows, kp, NR = (args.num_vars if args.num_vars != 24 else 8192), 16, 3, 4096
        lo, hi = column_range(ncols, world, rank)
        cols = hi - lo
        seed = np.ones(8, dtype=np.uint32)
        d_key = DeviceBuffer(lib, kp * cols * rows * NR * 4)
        assert lib.agl_mcommit_keygen(seed.ctypes.data, 1, rows, lo, cols, kp, d_key.ptr) == 0   # key material: untimed
        x = np.random.default_rng(5 + rank).integers(-1, 2, size=cols * NR, dtype=np.int8)
        d_x = DeviceBuffer.from_numpy(lib, x)
        d_acc, d_o = DeviceBuffer(lib, kp * rows * NR * 4), DeviceBuffer(lib, rows * NR * 8)
        out = np.zeros(rows * NR, dtype=np.uint64)

        def device_commit():
            rc = lib.agl_mcommit_partial(d_key.ptr, cols, rows, kp, d_x.ptr, 1, 1, cols, 0, None, d_acc.ptr)
            return rc or lib.agl_mcommit_finish(d_acc.ptr, 1, kp, rows, None, d_o.ptr)

        def local_commit(a, b):
            assert device_commit() == 0
            lib.cuda_memcpy_dtoh(out.ctypes.data, d_o.ptr, out.nbytes)
            return out

        def step():
            if world == 1:
                return device_commit()
            module_commit_sharded(local_commit, comm, ncols, 1, rows)
            return 0

        h_x = pinned_copy(lib, x)

        def step_e2e():
            lib.cuda_memcpy_htod(d_x.ptr, h_x, x.nbytes)
            if world == 1:
                device_commit()
                lib.cuda_memcpy_dtoh(out.ctypes.data, d_o.ptr, out.nbytes)
            else:
                module_commit_sharded(local_commit, comm, ncols, 1, rows)
        units = ncols * NR
        metric = "field-elems/s: module commitment over F_q[Y]/(Y^4096+1), 16 rows, ternary columns, almost-Goldilocks"
        workload = "mcommit cols=%d rows=16 primes=3 int8" % ncols
        # the key cache is read once (16 KB per prime, column and row); the transformed inputs are written and read once
        alg_bytes = float(kp * cols * rows * NR * 4 + 2 * kp * cols * NR * 4 + cols * NR)
        h2d, d2h = x.nbytes, out.nbytes
        scaling = "strong"
    else:
        # the witness columns are split across the ranks (strong scaling); partial commitments are all-gathered
        # (planes x 42 x 64 words per rank) and added mod q
        from matrix_b200 import load_agl
        from matrix_b200.sharded import SingleComm, TorchComm, column_range, commit_sharded
        lib = load_agl()
        assert lib.cuda_set_device(local) == 0
        comm = SingleComm(1)
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            comm = TorchComm(device=torch.device("cuda", local))
        logn = args.num_vars if args.num_vars != 24 else 18
        n_ring, L = 1 << logn, args.planes
        lo, hi = column_range(n_ring, world, rank)
        cols = hi - lo
        key = np.arange(1, 9, dtype=np.uint32)
        dig = np.random.default_rng(5 + rank).integers(-127, 128, size=L * cols * 64, dtype=np.int8)
        d_k, d_z = DeviceBuffer.from_numpy(lib, key), DeviceBuffer.from_numpy(lib, dig)
        d_o = DeviceBuffer(lib, L * 42 * 64 * 8)
        out = np.zeros(L * 42 * 64, dtype=np.uint64)

        def local_commit(a, b):
            assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, b - a, L, a, d_o.ptr) == 0
            lib.cuda_memcpy_dtoh(out.ctypes.data, d_o.ptr, out.nbytes)
            return out

        d_tiled = None
        if args.matrix == "tiled":
            # the matrix as byte planes in operand order, built once (key material, untimed); one GPU only
            assert world == 1, "--matrix tiled runs on one GPU"
            d_tiled = DeviceBuffer(lib, lib.ajtai_tc_matrix_bytes(n_ring))
            assert lib.ajtai_materialize_tc_ffi(d_k.ptr, d_tiled.ptr, n_ring, 0) == 0

        def commit_all():
            if d_tiled is not None:
                return lib.ajtai_commit_s8_tiled_ffi(d_tiled.ptr, d_z.ptr, n_ring, L, d_o.ptr)
            return lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, n_ring, L, 0, d_o.ptr)

        def step():
            if world == 1:
                return commit_all()
            commit_sharded(local_commit, comm, n_ring, L)
            return 0

        h_dig = pinned_copy(lib, dig)

        def step_e2e():
            lib.cuda_memcpy_htod(d_z.ptr, h_dig, dig.nbytes)
            if world == 1:
                commit_all()
                lib.cuda_memcpy_dtoh(out.ctypes.data, d_o.ptr, out.nbytes)
            else:
                commit_sharded(local_commit, comm, n_ring, L)
        units = n_ring * 64
        metric = "field-elems/s: Ajtai ring commit (42 x 64 rows), %d signed 8-bit digit planes, almost-Goldilocks" % L
        workload = "ajtai_commit_s8 n_ring=2^%d planes=%d matrix=%s" % (logn, L, args.matrix)
        alg_bytes = None
        h2d, d2h = dig.nbytes, out.nbytes
        scaling = "strong"
    timed = _event_timer(lib)

    def barrier():
        if dist is not None:
            dist.barrier()
        lib.cuda_device_synchronize()

    def timed_max(fn, reps):
        barrier()
        v = timed(fn, reps)
        barrier()
        if dist is not None:
            import torch
            t = torch.tensor([v], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            v = float(t.item())
        return v

    for _ in range(max(args.warmup, 1)):
        assert step() == 0
    sampler = ClockSampler(local)
    launches0 = lib.mb_launch_count()
    sampler.start()
    ms = timed_max(step, args.steps)
    launches = lib.mb_launch_count() - launches0
    step_e2e()
    ms_e2e = timed_max(step_e2e, args.steps)
    # a timed region of a few milliseconds ends before nvidia-smi prints its first sample: keep the same
    # step running (untimed) until one has arrived, so that the clocks are read under this load
    if world == 1:
        t_end = time.perf_counter() + 2.0
        while not sampler.lines and time.perf_counter() < t_end:
            step()
    else:
        for _ in range(20):   # the same count on every rank: the steps hold collectives
            step()
    clocks = sampler.stop()
    line = {"metric": metric, "value": units * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None,
            "dtype": {"sumcheck": "u64", "mcommit": "u32 residues mod five 31-bit primes, u64 recombination"}.get(
                args.workload, "s8 x u8 -> s32, u64 recombination"),
            "data": "synthetic", "config": {"workload": workload},
            "e2e": {"value": units * args.steps / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "clocks": clocks}
    if alg_bytes is not None:
        ach = alg_bytes * args.steps / (ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                            "peak_kind": peak_kind,
                            "note": ("whole call (input transforms, streaming accumulate, finish) against the bytes of this "
                                     "rank's key cache and transformed inputs; the accumulate kernel alone runs near the copy peak")
                            if args.workload == "mcommit" else
                            "whole proof (all rounds, host transcript between them) against the bytes its passes must move; "
                            "small tables are latency bound"}
    else:
        macs = 2688.0 * units * 8 * args.planes   # 42 x 64 rows, 8 byte planes of the matrix, digit planes of the witness
        mac_rate = macs * args.steps / (ms * 1e-3)
        ipeak = int8_peak(lib) if rank == 0 else None
        line["roofline"] = {"bound": "tensor", "achieved": mac_rate / 1e12, "peak": ipeak / 1e12 if ipeak else None,
                            "unit": "int8 TMAC/s", "frac": mac_rate / (ipeak * world) if ipeak else None, "traffic": None,
                            "peak_kind": "measured in this run by the library's tcgen05 kind::i8 issue loop on resident "
                                         "operands (per GPU)" if ipeak else "unmeasured",
                            "note": "matrix byte planes read in operand order from HBM" if args.matrix == "tiled" else
                                    "the matrix is regenerated from the ChaCha8 stream in every pass; generation and the "
                                    "operand build bound the kernel before the tensor pipe does"}
    if args.workload == "mcommit" and rank == 0 and not args.no_cpu_baseline:
        # the oracle's schoolbook products (what the reference's CPU test compares with, commit.rs:92-131) on two columns
        from oracle import pyoracle
        xs = np.random.default_rng(1).integers(-1, 2, size=(2, 4096)).astype(np.int64)
        t0 = time.perf_counter()
        pyoracle.mcommit_commit([1] * 8, 1, 16, [0, 1], xs)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 2 * 4096 / dt, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                                "sample": "2 columns x 16 rows, schoolbook negacyclic products with key expansion (OpenMP over rows)"}
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_link(args):
    """The two largest rounds of the packed link sumcheck on one GPU: round 0 off the bit-packed witness
    (message, then fold to a half-size table with the weights folded in place) and round 1 on the tables
    (message, fold). 8 commitments of 2^24 coefficients, 5 % of the bits set (one-hot style advice is sparser,
    committed weights denser); weights, eq and tags are seeded field elements."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    from matrix_b200 import load_agl
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import AGL_Q, field_elems
    lib = load_agl()
    assert lib.cuda_set_device(local) == 0
    peak, peak_kind = measured_peaks()
    log_n, nc = (args.num_vars if args.num_vars != 24 else 24), 8
    n, half = 1 << log_n, 1 << (log_n - 1)
    rng = np.random.default_rng(7)
    bits = rng.random(nc * n) < 0.05
    words = np.ascontiguousarray(np.packbits(bits.reshape(-1, 64)[:, ::-1], axis=1).view(">u8").astype(np.uint64).reshape(-1))

    def dev_rand(seed, elems):   # seeded field elements tiled on the device (the host holds one 32 MB tile)
        buf, tile = DeviceBuffer(lib, elems * 16), field_elems(seed, 1 << 22, AGL_Q)
        for off in range(0, 2 * elems, 1 << 22):
            lib.cuda_memcpy_htod(buf.ptr + off * 8, tile.ctypes.data, min(1 << 22, 2 * elems - off) * 8)
        return buf
    d_bits, d_om0, d_eq, d_tags = DeviceBuffer.from_numpy(lib, words), dev_rand(1, nc * n), dev_rand(2, half), dev_rand(3, nc)
    d_om, d_w = DeviceBuffer(lib, nc * n * 16), DeviceBuffer(lib, nc * half * 16)
    chunks = 148 * 8 // nc
    d_part, d_out = DeviceBuffer(lib, nc * chunks * 7 * 16), DeviceBuffer(lib, 7 * 16)
    msg = np.zeros(14, dtype=np.uint64)

    def step():
        lib.cuda_memcpy_dtod(d_om.ptr, d_om0.ptr, nc * n * 16)   # the folds work in place: restore the weights
        rc = lib.link_round0_bits_ffi(d_bits.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, n, half, nc, d_part.ptr, chunks, d_out.ptr)
        rc |= lib.link_fold0_bits_ffi(d_bits.ptr, d_w.ptr, d_om.ptr, n, half, nc, 5, 7)
        rc |= lib.link_round_message_ffi(d_w.ptr, d_om.ptr, d_eq.ptr, d_tags.ptr, half, n, half // 2, nc, 0, d_part.ptr, chunks, d_out.ptr)
        rc |= lib.link_fold_ffi(d_w.ptr, d_om.ptr, half, n, half // 2, nc, 11, 13)
        return rc

    h_words = pinned_copy(lib, words)

    def step_e2e():
        lib.cuda_memcpy_htod(d_bits.ptr, h_words, words.nbytes)
        step()
        lib.cuda_memcpy_dtoh(msg.ctypes.data, d_out.ptr, msg.nbytes)
    timed = _event_timer(lib)
    for _ in range(max(args.warmup, 3)):
        assert step() == 0
    sampler = ClockSampler(local)
    launches0 = lib.mb_launch_count()
    sampler.start()
    lib.cuda_device_synchronize()
    ms = timed(step, args.steps)   # the timed region: no per-launch events
    launches = lib.mb_launch_count() - launches0
    lib.mb_prof_enable(1)          # per-kernel times: a separate pass
    lib.mb_prof_reset()
    for _ in range(args.steps):
        step()
    lib.cuda_device_synchronize()
    buf = ctypes.create_string_buffer(1 << 16)
    lib.mb_prof_report(buf, len(buf))
    kernels = {l.split()[0]: float(l.split()[2]) / args.steps for l in buf.value.decode().splitlines() if len(l.split()) == 3}
    lib.mb_prof_enable(0)
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    t_end = time.perf_counter() + 2.0
    while not sampler.lines and time.perf_counter() < t_end:
        step()
    clocks = sampler.stop()
    units = nc * n
    fold_bytes = 1.5 * nc * half * 32.0   # link_fold: both tables, read 2 halves, write 1
    ach = fold_bytes / (kernels.get("link_fold", float("nan")) * 1e-3) / 1e9
    line = {"metric": "field-elems/s: packed link sumcheck, rounds 0 and 1 (8 commitments x 2^%d bit-packed coefficients), "
                      "almost-Goldilocks" % log_n,
            "value": units * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic", "config": {"workload": "link rounds 0-1, n_commit=8, 2^%d coefficients, 5%% of bits set" % log_n,
                                            "l2": "tables larger than L2"},
            "e2e": {"value": units * args.steps / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(words.nbytes), "d2h_bytes_per_step": int(msg.nbytes)},
            "gpu_launches": int(launches), "clocks": clocks, "kernel_ms_per_step": kernels,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "peak_kind": peak_kind, "note": "link_fold (the streaming kernel of the step); the bit round is a gather "
                                                         "over live pairs, the table round is bound by the integer pipe"}}
    print(json.dumps(line))


def run_llama_layer(args):
    """Shape trace of one Llama-2-7B decoder layer (hidden 4096, 32 heads, FFN in 16 shards of 1024, seq 128):
    every einsum of the layer proved as its block does on the GPU (operand partial evaluations, eq table, one
    linear sumcheck on a shared transcript; matrix_b200/layer_trace.py) plus the Ajtai commit of every einsum
    output at three signed 8-bit digit planes (21-bit decomposition). Weights (2^28 coefficients) and inputs
    are resident: distinct buffers per einsum, unsigned 16-bit synthetic magnitudes. Not in the trace: lookup
    and range arguments of the non-linear blocks and the fold tree above the blocks."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    from matrix_b200 import load_agl
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import AGL_Q, field_elems
    from matrix_b200.layer_trace import EinsumPlan, LayerProver, llama_layer_ops
    lib = load_agl()
    assert lib.cuda_set_device(local) == 0
    prover = LayerProver(lib)
    ops = llama_layer_ops()
    work, n_in, n_out_total = [], 0, 0
    for k, (name, eq, dims) in enumerate(ops):
        pl = EinsumPlan(eq, dims)
        bufs = []
        for j, t in enumerate(pl.inputs):
            n = sum(dims[c] for c in t)
            b = DeviceBuffer(lib, 8 << n)
            assert lib.mb_fill_splitmix(b.ptr, 1 << n, 1000 + 8 * k + j, 1 << 16) == 0
            bufs.append(b)
            n_in += 1 << n
        n_out = sum(dims[c] for c in pl.out)
        n_out_total += 1 << n_out
        point = field_elems(5000 + k, 2 * max(n_out, 1), AGL_Q)[:2 * n_out].reshape(n_out, 2)
        work.append((eq, dims, bufs, point, n_out))
    L, max_out = 3, max(w[4] for w in work)
    key = np.arange(1, 9, dtype=np.uint32)
    dig = np.random.default_rng(5).integers(-127, 128, size=L << max_out, dtype=np.int8)
    d_k, d_z = DeviceBuffer.from_numpy(lib, key), DeviceBuffer.from_numpy(lib, dig)
    d_o = DeviceBuffer(lib, L * 42 * 64 * 8)
    finals = []

    from matrix_b200.layer_trace import prove_einsum_native

    def step(commit=True, native=True):
        h = ctypes.c_void_p()
        lib.agl_transcript_create(b"llama-layer", 11, ctypes.byref(h))
        for eq, dims, bufs, point, n_out in work:
            if native:   # the whole device sequence of the block in one library call
                finals.append(prove_einsum_native(prover, eq, dims, [b.ptr for b in bufs], point, h)[3])
            else:        # the same sequence issued call by call, as the reference's Rust issues it
                finals.append(prover.prove_einsum(eq, dims, [b.ptr for b in bufs], point, h)[3])
            if commit and n_out >= 6:   # the digit planes of a smaller tensor start at its own plane stride
                assert lib.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, 1 << (n_out - 6), L, 0, d_o.ptr) == 0
        lib.agl_transcript_destroy(h)
        del finals[:-1]
        return 0
    timed = _event_timer(lib)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local)
    launches0 = lib.mb_launch_count()
    sampler.start()
    lib.cuda_device_synchronize()
    ms = timed(lambda: step(), args.steps)   # the timed region: no per-launch events
    launches = lib.mb_launch_count() - launches0
    ms_prove = timed(lambda: step(False), args.steps)
    native_final = [int(x) for x in finals[-1]]
    step(True, False)
    ms_calls = timed(lambda: step(True, False), args.steps)
    # per-kernel times: a separate pass with events around every launch
    lib.mb_prof_enable(1)
    lib.mb_prof_reset()
    for _ in range(args.steps):
        step()
    lib.cuda_device_synchronize()
    buf = ctypes.create_string_buffer(1 << 16)
    lib.mb_prof_report(buf, len(buf))
    kernels = {l.split()[0]: round(float(l.split()[2]) / args.steps, 4) for l in buf.value.decode().splitlines() if len(l.split()) == 3}
    lib.mb_prof_enable(0)
    same = native_final == [int(x) for x in finals[-1]]
    t_end = time.perf_counter() + 2.0
    while not sampler.lines and time.perf_counter() < t_end:
        step()
    clocks = sampler.stop()
    peak, peak_kind = measured_peaks()
    # the operand passes read every weight and input once (8 B each): the part of the step that is bound by HBM
    pe_ms = sum(v for k, v in kernels.items() if "partial_eval" in k or "peval" in k)
    ach = 8.0 * n_in / (pe_ms * 1e-3) / 1e9 if pe_ms else float("nan")
    line = {"metric": "prove time: one Llama-2-7B-shaped decoder layer, einsum blocks + activation commits (shape trace)",
            "value": ms / args.steps, "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic",
            "config": {"workload": "llama_layer d=4096 heads=32 ffn=16x1024 seq=128: %d einsum proofs, %d activation commits of %d "
                                   "planes" % (len(work), sum(1 for w in work if w[4] >= 6), L),
                       "operand_elems": int(n_in), "committed_elems": int(n_out_total),
                       "l2": "2.2 GB of distinct operands per step, larger than L2"},
            "prove_only_ms_per_step": ms_prove / args.steps, "kernel_ms_per_step": kernels,
            "kernel_ms_total": sum(kernels.values()),
            "call_by_call_ms_per_step": ms_calls / args.steps,
            "call_by_call_note": "the same sequence issued one synchronising C-ABI call at a time (how the reference's Rust "
                                 "drives it); ms_per_step is one library call per einsum block; last final evaluation equal: %s" % same,
            "e2e": {"value": ms / args.steps, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "weights and activations are resident in the reference's prover too (device weight cache); "
                            "per proof only challenges go up and round messages come back, inside the timed step"},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "peak_kind": peak_kind, "note": "operand partial evaluations (all weights and inputs read once, 8 B per "
                                                         "element) over their summed kernel time; the rest of the step is "
                                                         "latency: 87 sumchecks of 10 to 17 rounds on small tables"}}
    print(json.dumps(line))


def run_peval(args):
    """Table preparation kernels of the sumcheck callers on one GPU, almost-Goldilocks: partial evaluation of the 12
    low variables of a 2^n base-field table (extension challenges), the fused bit-permutation + partial evaluation
    with the 12 high variables fixed, and the eq table of n variables. Event-timed per call; the partial evaluation
    is the headline of the line."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    from matrix_b200 import load_agl
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import AGL_Q, field_elems
    from matrix_b200.layer_trace import split_luts
    lib = load_agl()
    assert lib.cuda_set_device(local) == 0
    peak, peak_kind = measured_peaks()
    log_n, m = (args.num_vars if args.num_vars != 24 else 26), 12
    n = 1 << log_n
    src = DeviceBuffer(lib, 8 * n)
    assert lib.mb_fill_splitmix(src.ptr, n, 1, AGL_Q) == 0
    out, o2 = DeviceBuffer(lib, 16 * (n >> 1)), DeviceBuffer(lib, 16 * (n >> m))
    r = DeviceBuffer.from_numpy(lib, field_elems(3, 2 * log_n, AGL_Q))
    order = list(range(log_n - m, log_n)) + list(range(log_n - m))
    lo, hi = split_luts(log_n, order, log_n // 2)
    dlo, dhi = DeviceBuffer.from_numpy(lib, lo), DeviceBuffer.from_numpy(lib, hi)
    eq_a, eq_b, res = DeviceBuffer(lib, 16 * n), DeviceBuffer(lib, 16 * n), ctypes.c_void_p()
    eq_m = DeviceBuffer.from_numpy(lib, field_elems(4, 2 << m, AGL_Q))
    timed = _event_timer(lib)
    calls = {"partial_eval": lambda: lib.agl_partial_eval_ext2_from_base_ffi(src.ptr, out.ptr, r.ptr, log_n, m),
             "fused_permute_partial_eval": lambda: lib.agl_fused_permute_partial_eval_ffi(
                 src.ptr, o2.ptr, eq_m.ptr, dlo.ptr, dhi.ptr, log_n, m, log_n // 2, n >> m, 0),
             "eq_table": lambda: lib.aext2_eq_dp_all_ffi(r.ptr, eq_a.ptr, eq_b.ptr, log_n, ctypes.byref(res))}
    for fn in calls.values():
        for _ in range(max(args.warmup, 3)):
            assert fn() == 0
    sampler = ClockSampler(local)
    launches0 = lib.mb_launch_count()
    sampler.start()
    ms = {k: timed(fn, args.steps) / args.steps for k, fn in calls.items()}
    launches = lib.mb_launch_count() - launches0
    t_end = time.perf_counter() + 2.0
    while not sampler.lines and time.perf_counter() < t_end:
        calls["partial_eval"]()
    clocks = sampler.stop()
    alg = 8.0 * n + 16.0 * (n >> m)
    ach = alg / (ms["partial_eval"] * 1e-3) / 1e9
    line = {"metric": "field-elems/s: partial evaluation of %d variables of a 2^%d base-field table, almost-Goldilocks" % (m, log_n),
            "value": n / (ms["partial_eval"] * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms["partial_eval"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic", "config": {"workload": "peval n=%d m=%d" % (log_n, m), "l2": "table of %d MB, larger than L2" % (8 * n >> 20)},
            "ms_per_call": ms,
            "gbs": {"partial_eval": ach, "fused_permute_partial_eval": alg / (ms["fused_permute_partial_eval"] * 1e-3) / 1e9,
                    "eq_table": 16.0 * n / (ms["eq_table"] * 1e-3) / 1e9},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "peak_kind": peak_kind, "note": "whole call (three passes, the first reads the table once: 8 B per element)"}}
    print(json.dumps(line))


def basefold_config(nv, hash_name, world):
    """The `config` object of the headline line; the same for both arms so that the two lines describe one workload."""
    cfg = {"workload": "basefold_commit_open nv=%d lr=%d queries=%d %s" % (nv, LOG_RATE, NUM_QUERIES, hash_name),
           "num_vars": nv, "log_rate": LOG_RATE, "num_queries": NUM_QUERIES,
           "l2": "inputs larger than L2 (codeword 256 MiB, trees > 1 GiB per step)"}
    if world > 1:
        cfg["partition"] = ("one polynomial over %d GPUs: contiguous ranges of the evaluations and of every codeword; one "
                            "device all-to-all per proof, one gather of 10 words per rank and round" % world)
    return cfg


def prof_report(lib):
    need = lib.mb_prof_report(None, 0)
    buf = ctypes.create_string_buffer(need + 16)
    lib.mb_prof_report(buf, need + 16)
    kernels = {}
    for line in buf.value.decode().splitlines():
        name, cnt, ms = line.split()
        name = name[len("monolith_"):] if name.startswith("monolith_") else name
        kernels[name] = (int(cnt), float(ms))
    return kernels


def run_same_point(args):
    """The batched same-point sumcheck of zk-torch-4's fold tree (fold/same_point_sumcheck.rs) at the shape the
    reference publishes (zk-torch-4/PROVER_PERFORMANCE.md:466-493: arity 22, 42 leaves): binary packed witnesses,
    one claim point per leaf, whole protocol through agl_same_point_prove_device_ffi (eq tables built on the device,
    22 rounds, host Monolith transcript). Single GPU."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    from matrix_b200 import load_agl
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import AGL_Q, splitmix64
    lib = load_agl()
    assert lib.cuda_set_device(local) == 0 and lib.almost_goldilocks_cuda_init() == 0
    arity = args.num_vars if args.num_vars != 24 else 22
    M = args.instances if args.instances != 16 else 42
    n = 1 << arity
    words = max(1, n >> 6)
    packed = splitmix64(11, M * words)
    if n < 64:
        packed &= np.uint64((1 << n) - 1)
    pts = splitmix64(12, 2 * arity * M) % np.uint64(AGL_Q)
    h_packed = ctypes.c_void_p()
    assert lib.mb_host_alloc(ctypes.byref(h_packed), packed.nbytes) == 0
    ctypes.memmove(h_packed.value, packed.ctypes.data, packed.nbytes)
    d_w = DeviceBuffer.from_numpy(lib, packed)
    vals = np.zeros((M, 2), dtype=np.uint64)
    assert lib.agl_same_point_claims_device_ffi(M, arity, pts.ctypes.data, 0, d_w.ptr, None, vals.ctypes.data) == 0   # the claims: untimed
    msgs, ch = np.zeros((arity, 3, 2), dtype=np.uint64), np.zeros((arity, 2), dtype=np.uint64)
    fe, fin = np.zeros((M, 2), dtype=np.uint64), np.zeros(2, dtype=np.uint64)

    def step():
        t = ctypes.c_void_p()
        assert lib.agl_transcript_create(LABEL, len(LABEL), ctypes.byref(t)) == 0
        rc = lib.agl_same_point_prove_device_ffi(M, arity, pts.ctypes.data, vals.ctypes.data, 0, d_w.ptr, None, t, msgs.ctypes.data,
                                                 ch.ctypes.data, fe.ctypes.data, fin.ctypes.data)
        lib.agl_transcript_destroy(t)
        return rc

    def step_e2e():
        assert lib.mb_memcpy_htod_async(d_w.ptr, h_packed, packed.nbytes) == 0
        assert step() == 0

    timed = _event_timer(lib)
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 1)):
        assert step() == 0
    lib.mb_prof_enable(0)
    launches0 = lib.mb_launch_count()
    lib.cuda_device_synchronize()
    sampler.mark_begin()
    ms = timed(step, args.steps)
    sampler.mark_end()
    launches = lib.mb_launch_count() - launches0
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    psteps = min(args.steps, 3)
    lib.mb_prof_reset(); lib.mb_prof_enable(1)
    for _ in range(psteps):
        step()
    lib.mb_prof_enable(0)
    clocks = sampler.stop()
    kernels = prof_report(lib)
    # the proof must verify (host verifier of the library)
    ok = ctypes.c_int(0)
    t = ctypes.c_void_p()
    lib.agl_transcript_create(LABEL, len(LABEL), ctypes.byref(t))
    ar = np.full(M, arity, dtype=np.int32)
    assert lib.agl_same_point_verify_ffi(M, arity, ar.ctypes.data, pts.ctypes.data, vals.ctypes.data, msgs.ctypes.data, fe.ctypes.data,
                                         fin.ctypes.data, t, None, ctypes.byref(ok)) == 0
    lib.agl_transcript_destroy(t)
    peak, peak_kind = measured_peaks()
    per = ms / args.steps
    # bytes the proof must move (extension elements of 16 B): the eq tables are written once and read by the first
    # message and by the first fold (with the packed bits), which writes the half-size eq and f tables; every later
    # round is one pass that reads its eq and f tables and writes their halves
    alg = M * n * 16.0 * 3 + M * (n // 2) * 32.0 + sum(M * (n >> r) * 32.0 * 1.5 for r in range(1, arity))
    kernel_ms = sum(x for _, x in kernels.values()) / psteps
    ach = alg / (kernel_ms * 1e-3) / 1e9
    elems = M * n
    line = {"metric": "field-elems/s: batched same-point sumcheck (eq x f, degree 2), %d leaves of arity %d, almost-Goldilocks" % (M, arity),
            "value": elems * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": per, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": "same_point arity=%d leaves=%d binary" % (arity, M),
                       "l2": "tables larger than L2" if M * n * 32 > (256 << 20) else "tables fit L2",
                       "published": "26-27 ms for the 22 rounds on an A100 (zk-torch-4/PROVER_PERFORMANCE.md:466-493); "
                                    "ms_per_step here includes the eq tables and the reveals"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "peak_kind": peak_kind,
                         "timed_in": "a separate pass of %d steps with CUDA events around every launch" % psteps,
                         "note": "all kernels of a proof against the bytes its passes must move (one pass per round: fold and next "
                                 "message fused); the passes are bound by the integer pipe (extension products), not by HBM"},
            "kernel_times_ms": {k: {"launches": c, "ms": round(x, 4)} for k, (c, x) in sorted(kernels.items())},
            "kernel_times_steps": psteps,
            "per_step": {"kernel_ms": kernel_ms, "other_ms": per - kernel_ms},
            "e2e": {"value": elems * args.steps / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(packed.nbytes), "d2h_bytes_per_step": int(msgs.nbytes + fe.nbytes + 6 * M * 8 * arity)},
            "gpu_launches": int(launches), "clocks": clocks, "verified": bool(ok.value),
            "final_eval": [int(x) for x in fin]}
    if not args.no_cpu_baseline:
        from oracle import pyoracle
        sa = min(arity, 16)
        insts = []
        sw = max(1, (1 << sa) >> 6)
        for i in range(M):
            w = packed[i * words:i * words + sw].copy()
            pt = pts[2 * arity * i:2 * arity * i + 2 * sa].reshape(sa, 2)
            insts.append(dict(arity=sa, kind=0, witness=w, point=pt, value=pyoracle.agl_witness_eval(0, w, sa, pt)))
        pyoracle.load().oracle_set_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        pyoracle.agl_same_point_prove(insts, sa, LABEL)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": M * (1 << sa) / dt, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": "CPU oracle (restatement of prove_same_point's dense path, OpenMP over the leaves) on "
                                          "%d leaves of arity %d, %.2f s; the cost is linear in 2^arity" % (M, sa, dt)}
    print(json.dumps(line))
    lib.mb_host_free(h_packed)


def part_sumcheck(lib, args, peak, peak_kind):
    """The linear sumcheck of f * g over 2^24 points (base-field tables, extension challenges): whole proof through
    gl_sumcheck_prove_device_ffi (tables resident) and gl_sumcheck_prove_host_ffi (host tables, copy inside)."""
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import field_elems
    nv, d = min(args.num_vars, 24), 2
    n = 1 << nv
    polys = np.concatenate([field_elems(1, n), field_elems(2, n)])
    d_t = DeviceBuffer.from_numpy(lib, polys)
    h_p = ctypes.c_void_p()
    assert lib.mb_host_alloc(ctypes.byref(h_p), polys.nbytes) == 0
    ctypes.memmove(h_p.value, polys.ctypes.data, polys.nbytes)
    rm, ch = np.zeros((nv, d + 1, 2), dtype=np.uint64), np.zeros((nv, 2), dtype=np.uint64)
    fes, fe = np.zeros((d, 2), dtype=np.uint64), np.zeros(2, dtype=np.uint64)

    def step():
        assert lib.gl_sumcheck_prove_device_ffi(d_t.ptr, d, nv, 1, LABEL, len(LABEL), rm.ctypes.data, ch.ctypes.data,
                                                fes.ctypes.data, fe.ctypes.data, None) == 0

    def step_e2e():
        assert lib.gl_sumcheck_prove_host_ffi(h_p, d, nv, 1, LABEL, len(LABEL), rm.ctypes.data, ch.ctypes.data,
                                              fes.ctypes.data, fe.ctypes.data, None) == 0

    timed = _event_timer(lib)
    reps = max(args.steps, 5)
    for _ in range(3):
        step()
    lib.mb_prof_enable(0)
    ms = timed(step, reps) / reps
    step_e2e()
    ms_e2e = timed(step_e2e, reps) / reps
    lib.mb_prof_reset(); lib.mb_prof_enable(1)
    step()
    lib.mb_prof_enable(0)
    kernels = prof_report(lib)
    alg_bytes = d * n * 48.0   # round 0 reads 8 B per element, the first fold reads 8 and writes 8, later rounds halve
    # The dominant kernel alone, through the per-round entry point the reference's state object would call: the fold
    # of round 0 fused with the message of round 1 over the full tables (8 B read and 8 B written per element),
    # timed by the library's CUDA events around the launch.
    d_o = DeviceBuffer(lib, d * n * 16)
    nblk = 592
    d_pp = DeviceBuffer(lib, nblk * (d + 1) * 2 * 8)
    big_reps = 5
    lib.mb_prof_reset(); lib.mb_prof_enable(1)
    for _ in range(big_reps):
        assert lib.sumcheck_fold_round_mixed_ffi(d_t.ptr, d_o.ptr, 0x1234567, 0x7654321, d, n, n // 4, d_pp.ptr, nblk) == 0
    lib.mb_prof_enable(0)
    big_ms = sum(x for _, x in prof_report(lib).values()) / big_reps
    big_bytes = d * n * 16.0
    ach = big_bytes / (big_ms * 1e-3) / 1e9
    whole = alg_bytes / (ms * 1e-3) / 1e9
    out = {"metric": "field-elems/s: sumcheck of f*g over 2^%d points, Goldilocks" % nv, "value": d * n / (ms * 1e-3), "unit": UNIT,
           "ms": ms, "config": {"workload": "sumcheck nv=%d d=2" % nv},
           "roofline": {"kernel": "sumcheck_fold_message (fold of round 0 + message of round 1, 2^%d elements per table)" % nv,
                        "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                        "peak_kind": peak_kind, "avg_launch_ms": big_ms, "launches": big_reps,
                        "timed_in": "a separate pass of %d launches through sumcheck_fold_round_mixed_ffi with CUDA events "
                                    "around each (not the timed region)" % big_reps,
                        "whole_proof": {"achieved": whole, "frac": whole / peak,
                                        "note": "%d rounds with the host transcript between them against the %.2f GB the passes "
                                                "must move; the last rounds are latency bound" % (nv, alg_bytes / 1e9)}},
           "e2e": {"value": d * n / (ms_e2e * 1e-3), "unit": UNIT, "ms": ms_e2e, "h2d_bytes_per_step": int(polys.nbytes),
                   "d2h_bytes_per_step": int(rm.nbytes + fe.nbytes)},
           "kernel_times_ms": {k: {"launches": c, "ms": round(x, 4)} for k, (c, x) in sorted(kernels.items())}}
    if not args.no_cpu_baseline:
        from oracle import pyoracle
        snv = nv
        sp = np.concatenate([field_elems(1, 1 << snv), field_elems(2, 1 << snv)])
        pyoracle.load().oracle_set_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        pyoracle.sumcheck_prove(sp, d, snv, True, LABEL)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": d * (1 << snv) / dt, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                               "sample": "CPU oracle prover (restating cpu_ext2_prover.rs) at 2^%d points, %.2f s" % (snv, dt)}
    lib.mb_host_free(h_p)
    return out


def int8_peak(agl):
    """Sustained int8 multiply-accumulate rate of the tensor pipe as this library's own tcgen05 kind::i8 issue loop
    measures it (resident operands, no operand build); None when the library has no such probe."""
    fn = getattr(agl, "ajtai_tc_int8_peak_ffi", None)
    if fn is None:
        return None
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    best = 0.0
    for _ in range(3):
        v = ctypes.c_double()
        if fn(4096, ctypes.byref(v)) != 0:
            return None
        best = max(best, v.value)
    return best


def part_ajtai(args, local):
    """The Ajtai ring commit (42 x 64 rows) of 2^18 ring columns = 2^24 coefficients in three signed 8-bit digit
    planes on the tensor cores, matrix regenerated from the ChaCha8 stream."""
    from matrix_b200 import load_agl
    from matrix_b200.ffi import DeviceBuffer
    agl = load_agl()
    assert agl.cuda_set_device(local) == 0 and agl.almost_goldilocks_cuda_init() == 0
    logn, L = min(args.num_vars, 24) - 6, 3
    n_ring = 1 << logn
    key = np.arange(1, 9, dtype=np.uint32)
    dig = np.random.default_rng(5).integers(-127, 128, size=L * n_ring * 64, dtype=np.int8)
    d_k, d_z = DeviceBuffer.from_numpy(agl, key), DeviceBuffer.from_numpy(agl, dig)
    d_o = DeviceBuffer(agl, L * 42 * 64 * 8)
    out = np.zeros(L * 42 * 64, dtype=np.uint64)

    def step():
        assert agl.ajtai_commit_s8_ffi(d_k.ptr, d_z.ptr, n_ring, L, 0, d_o.ptr) == 0

    h_dig = pinned_copy(agl, dig)

    def step_e2e():
        agl.cuda_memcpy_htod(d_z.ptr, h_dig, dig.nbytes)
        step()
        agl.cuda_memcpy_dtoh(out.ctypes.data, d_o.ptr, out.nbytes)

    timed = _event_timer(agl)
    reps = max(args.steps, 5)
    for _ in range(3):
        step()
    ms = timed(step, reps) / reps
    step_e2e()
    ms_e2e = timed(step_e2e, reps) / reps
    macs = 2688.0 * n_ring * 64 * 8 * L      # 42 x 64 rows, 64 coefficients per column, 8 byte planes of the matrix, L digit planes
    mac_rate = macs / (ms * 1e-3)
    peak = int8_peak(agl)
    res = {"metric": "field-elems/s: Ajtai ring commit (42 x 64 rows), %d signed 8-bit digit planes, almost-Goldilocks" % L,
           "value": n_ring * 64 / (ms * 1e-3), "unit": UNIT, "ms": ms,
           "config": {"workload": "ajtai_commit_s8 n_ring=2^%d planes=%d" % (logn, L)},
           "roofline": {"bound": "tensor", "achieved": mac_rate / 1e12, "peak": peak / 1e12 if peak else None,
                        "unit": "int8 TMAC/s", "frac": mac_rate / peak if peak else None, "traffic": None,
                        "peak_kind": "measured in this run by the library's tcgen05 kind::i8 issue loop on resident operands"
                        if peak else "unmeasured",
                        "note": "the matrix is regenerated from the ChaCha8 stream in every pass; generation and the "
                                "operand build bound the kernel before the tensor pipe does"},
           "e2e": {"value": n_ring * 64 / (ms_e2e * 1e-3), "unit": UNIT, "ms": ms_e2e, "h2d_bytes_per_step": int(dig.nbytes),
                   "d2h_bytes_per_step": int(out.nbytes)}}
    if not args.no_cpu_baseline:
        from oracle import pyoracle
        cols = 8192
        pyoracle.load().oracle_set_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        pyoracle.ajtai_commit(key, dig[:L * cols * 64], 1, cols, L)
        dt = time.perf_counter() - t0
        res["cpu_baseline"] = {"value": cols * 64 / dt, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                               "sample": "CPU oracle (pinned to the reference's cpu_ajtai_commit) on %d ring columns x %d planes, "
                                         "%.2f s; the cost is linear in the columns" % (cols, L, dt)}
    return res


def run_basefold(args):
    """The headline. N = 1: one polynomial on one GPU. N > 1: the same single polynomial partitioned over the N
    GPUs (strong scaling); the figure for N independent provers is reported beside it as `replicas`."""
    rank, world, local = dist_env()
    from matrix_b200 import load_gl
    from matrix_b200.ffi import DeviceBuffer
    from matrix_b200.inputs import field_elems

    lib = load_gl()  # raises when the CUDA library is missing: there is no CPU path
    assert lib.basefold_set_merkle_hash(1 if args.hash == "monolith" else 0) == 0
    if lib.cuda_set_device(local) != 0:
        raise SystemExit("cuda_set_device(%d) failed" % local)

    dist, exch = None, None
    if world > 1:
        import torch
        import torch.distributed as dist
        from matrix_b200.sharded import ProcessExchange
        torch.cuda.set_device(local)
        lib.cuda_set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        token = [os.urandom(6).hex() if rank == 0 else None]
        dist.broadcast_object_list(token, src=0)
        exch = ProcessExchange(lib, "/mb_basefold_%s" % token[0], rank, world, torch.device("cuda", local))

    def barrier():
        if dist is not None:
            dist.barrier()
        lib.cuda_device_synchronize()

    nv, lr, nq = args.num_vars, LOG_RATE, NUM_QUERIES
    n = 1 << nv
    evals = field_elems(3, n)            # one polynomial, the same on every rank
    point = field_elems(4, 2 * nv)
    table = ctypes.c_void_p()
    rc = lib.basefold_table_create(nv, lr, nv, 42, ctypes.byref(table))   # key material, untimed
    assert rc == 0, "basefold_table_create: %d" % rc
    words = lib.basefold_proof_words(nv, lr, nq)
    n_loc = n // world
    shard = np.ascontiguousarray(evals[rank * n_loc:(rank + 1) * n_loc])

    # pinned host staging for the e2e path
    h_evals_p, h_proof_p = ctypes.c_void_p(), ctypes.c_void_p()
    assert lib.mb_host_alloc(ctypes.byref(h_evals_p), 8 * n_loc) == 0
    assert lib.mb_host_alloc(ctypes.byref(h_proof_p), 8 * words) == 0
    ctypes.memmove(h_evals_p.value, shard.ctypes.data, 8 * n_loc)
    h_proof = np.ctypeslib.as_array(ctypes.cast(h_proof_p.value, ctypes.POINTER(ctypes.c_uint64)), shape=(words,))
    root = np.zeros(4, dtype=np.uint64)
    d_evals = DeviceBuffer.from_numpy(lib, shard)

    if world == 1:
        def step_resident():
            c = ctypes.c_void_p()
            rc = lib.basefold_commit_device(d_evals.ptr, nv, lr, ctypes.byref(c), root.ctypes.data)
            assert rc == 0, "basefold_commit_device: %d" % rc
            rc = lib.basefold_open_ext2(c, point.ctypes.data, table, LABEL, len(LABEL), nq, h_proof_p, None)
            assert rc == 0, "basefold_open_ext2: %d" % rc
            lib.basefold_commitment_destroy(c)

        def step_e2e():
            rc = lib.basefold_prove_host(h_evals_p, nv, lr, point.ctypes.data, table, LABEL, len(LABEL), nq,
                                         root.ctypes.data, h_proof_p)
            assert rc == 0, "basefold_prove_host: %d" % rc
    else:
        def step_resident():
            rc = lib.basefold_prove_sharded_device(d_evals.ptr, nv, lr, point.ctypes.data, table, LABEL, len(LABEL), nq,
                                                   exch.handle, root.ctypes.data, h_proof_p)
            assert rc == 0, "basefold_prove_sharded_device: %d" % rc

        def step_e2e():
            rc = lib.basefold_prove_sharded_host(h_evals_p, nv, lr, point.ctypes.data, table, LABEL, len(LABEL), nq,
                                                 exch.handle, root.ctypes.data, h_proof_p)
            assert rc == 0, "basefold_prove_sharded_host: %d" % rc

    def ev():
        e = ctypes.c_void_p()
        assert lib.mb_event_create(ctypes.byref(e)) == 0
        return e

    def timed(fn, steps, sampler=None):
        """CUDA events on the library's stream around `steps` calls; returns max-over-ranks ms."""
        a, b = ev(), ev()
        barrier()
        if sampler:
            sampler.mark_begin()
        lib.mb_event_record(a)
        for _ in range(steps):
            fn()
        lib.mb_event_record(b)
        lib.mb_event_sync(b)
        if sampler:
            sampler.mark_end()
        barrier()
        ms = ctypes.c_float()
        lib.mb_event_elapsed_ms(a, b, ctypes.byref(ms))
        val = ms.value
        if dist is not None:
            import torch
            t = torch.tensor([val], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            val = float(t.item())
        return val

    sampler = ClockSampler(local)
    sampler.start()
    lib.mb_prof_enable(0)
    for _ in range(max(args.warmup, 3)):
        step_resident()
    launches0 = lib.mb_launch_count()
    ms_total = timed(step_resident, args.steps, sampler)      # clean: no per-kernel events in the timed region
    launches = lib.mb_launch_count() - launches0
    clocks = sampler.stop()
    proof_words_sum = int(h_proof.sum(dtype=np.uint64))     # a checksum of the proof, equal on every N

    # e2e: host buffers in, proof out
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)

    # per-kernel times: a separate, untimed pass with CUDA events around every launch
    prof_steps = min(args.steps, 3)
    lib.mb_prof_reset()
    lib.mb_prof_enable(1)
    for _ in range(prof_steps):
        step_resident()
    lib.cuda_device_synchronize()
    lib.mb_prof_enable(0)
    kernels = prof_report(lib)

    ms_step = ms_total / args.steps
    value = n * args.steps / (ms_total * 1e-3)
    e2e_value = n * args.steps / (ms_e2e * 1e-3)

    # Roofline of the dominant kernel by device time. Algorithmic bytes per unit:
    #   hash_leaves     base pair 16 B in + 32 B digest out (commit tree); extension pair 32 B + 32 B (folded trees)
    #   compress_layer  64 B in + 32 B out per node
    # Units per launch come from this rank's share of the work (1 / world of every tree before the gather).
    peak, peak_kind = measured_peaks()
    total_kernel_ms = sum(ms for _, ms in kernels.values()) or 1.0
    dom = max(kernels, key=lambda k: kernels[k][1]) if kernels else None
    cw_len = 1 << (nv + lr)
    leaves_commit = ((cw_len // 2) >> lr) // world
    leaves_folded = sum((cw_len >> (i + 2)) for i in range(nv - 1)) // world
    nodes_per_step = leaves_commit + sum(max((cw_len >> (i + 2)) - 1, 0) for i in range(nv - 1)) // world
    roofline = None
    hash_ms = sum(kernels.get(k, (0, 0))[1] for k in ("hash_leaves", "compress_layer", "tree_tail", "compress_layer_coop",
                                                       "hash_leaves_coop"))
    perms_per_s = (leaves_commit + leaves_folded + nodes_per_step) * prof_steps / (hash_ms * 1e-3) if hash_ms else 0.0
    inst_per_perm = 15550.0 if args.hash == "poseidon2" else 6900.0  # thread instructions per permutation (ncu)
    sm_hz = 1e6 * (clocks.get("sm_mhz") or 1965.0)
    if dom is not None:
        cnt, ms = kernels[dom]
        if dom == "hash_leaves":
            total_bytes = (leaves_commit * 48 + leaves_folded * 64) * prof_steps
        elif dom == "compress_layer":
            total_bytes = 96 * nodes_per_step * prof_steps
        else:
            total_bytes = None
        if total_bytes is not None:
            achieved = total_bytes / (ms * 1e-3) / 1e9
            # DRAM bytes per launch, scaled from an ncu capture of the 2^22 case by the units hashed (reads equal the
            # algorithmic reads; most digest writes are still in L2 when a kernel ends): 65.06 B per node,
            # 20.44 B per base leaf pair, extension leaf pairs taken as 32 B read + the same write share.
            if dom == "compress_layer":
                traffic = 65.06 * nodes_per_step * prof_steps / cnt
            else:
                traffic = (20.44 * leaves_commit + 36.4 * leaves_folded) * prof_steps / cnt
            roofline = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                        "traffic_note": "bytes per launch (average), scaled from the ncu capture in profiles/",
                        "launches": cnt, "avg_launch_ms": ms / cnt, "share_of_kernel_time": ms / total_kernel_ms,
                        "timed_in": "a separate pass of %d steps with CUDA events around every launch (not the timed region)" % prof_steps,
                        "note": ("Poseidon2 hashing: ~520 modular multiplications per 32-byte digest, bound by the "
                                 "integer pipes, not HBM; permutations/s is the meaningful rate") if args.hash == "poseidon2"
                        else "Monolith hashing: bound by the integer pipes, not HBM; permutations/s is the meaningful rate",
                        "permutations_per_s": perms_per_s,
                        # the bound that applies: warp instructions issued against the issue slots of the machine
                        # (instructions per permutation from the ncu capture in profiles/; 148 SMs x 4 schedulers)
                        "issue": {"warp_inst_per_permutation": inst_per_perm / 32.0,
                                  "achieved_warp_inst_per_s": perms_per_s * inst_per_perm / 32.0,
                                  "peak_warp_inst_per_s": 148 * 4 * sm_hz,
                                  "frac": perms_per_s * inst_per_perm / 32.0 / (148 * 4 * sm_hz),
                                  "note": "integer additions, logic and multiply-adds share one 16-lane datapath per "
                                          "scheduler: 0.57 of the issue slots is the measured ceiling for this mix"}}
    line = {
        "metric": METRIC if args.hash == "poseidon2" else METRIC.replace("Poseidon2 Merkle", "Monolith Merkle"),
        "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
        "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": basefold_config(nv, args.hash, world),
        "roofline": roofline,
        "kernel_times_ms": {k: {"launches": c, "ms": round(ms, 4)} for k, (c, ms) in sorted(kernels.items())},
        "kernel_times_steps": prof_steps,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": 8 * n_loc + 16 * nv, "d2h_bytes_per_step": 8 * words + 32},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "proof_checksum": proof_words_sum,
    }
    if world > 1:
        line["bounded_by"] = ("per-round fixed cost: %d rounds x (kernel launches, one stream synchronisation, one host gather of 10 "
                              "words per rank); the hashing itself splits evenly" % (nv - 1))
        line["exchange"] = {"device_all_to_all_calls": exch.calls, "host_gather": "POSIX shared-memory mailbox"}
        # N independent provers (what the reference does across devices): every rank proves its own polynomial
        own = DeviceBuffer.from_numpy(lib, field_elems(3 + rank, n))

        def step_replica():
            c = ctypes.c_void_p()
            assert lib.basefold_commit_device(own.ptr, nv, lr, ctypes.byref(c), root.ctypes.data) == 0
            assert lib.basefold_open_ext2(c, point.ctypes.data, table, LABEL, len(LABEL), nq, h_proof_p, None) == 0
            lib.basefold_commitment_destroy(c)
        step_replica()
        rsteps = min(args.steps, 5)
        ms_rep = timed(step_replica, rsteps)
        line["replicas"] = {"value": world * n * rsteps / (ms_rep * 1e-3), "unit": UNIT, "ms_per_step": ms_rep / rsteps,
                            "scaling": "weak", "note": "one polynomial per rank, no exchange"}
    if rank == 0 and world == 1:
        line["parts"] = {"sumcheck": part_sumcheck(lib, args, peak, peak_kind), "ajtai": part_ajtai(args, local)}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        snv = min(args.ref_num_vars, nv)
        dt, _ = cpu_oracle_sample(snv, merkle_hash=args.hash)
        line["cpu_baseline"] = {"value": (1 << snv) / dt, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": "CPU oracle commit+open at 2^%d evaluations (%.2f s), OpenMP on all cores; "
                                          "table generation excluded on both sides; the reference arm (--impl reference) "
                                          "times the full size" % (snv, dt)}
    if rank == 0:
        print(json.dumps(line))
    lib.basefold_table_destroy(table)
    if exch is not None:
        dist.barrier()
        exch.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--num-vars", type=int, default=24)
    ap.add_argument("--ref-num-vars", type=int, default=20, help="sample size of the CPU arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="basefold", choices=["basefold", "batched_sumcheck", "sumcheck", "ajtai", "mcommit", "link", "llama_layer", "peval", "same_point"],
                    help="basefold: the headline (commit + open, 2^24); batched_sumcheck: 16 instances of "
                         "eq*a*b over 2^26 points sharded on the top variables (strong scaling)")
    ap.add_argument("--instances", type=int, default=16)
    ap.add_argument("--planes", type=int, default=3, help="ajtai workload: signed 8-bit digit planes of the witness")
    ap.add_argument("--matrix", default="stream", choices=["stream", "tiled"],
                    help="ajtai workload: regenerate the matrix from the ChaCha8 stream in every pass, or read byte planes "
                         "in operand order built once")
    ap.add_argument("--exchange", default="mailbox", choices=["mailbox", "nccl", "shm"],
                    help="batched_sumcheck: mailbox = the round loop inside the library with the ranks' 64-byte shares "
                         "going through its mailbox in POSIX shared memory; nccl / shm = the Python round loop over an NCCL "
                         "all-gather or a mailbox file in /dev/shm")
    ap.add_argument("--hash", default="poseidon2", choices=["poseidon2", "monolith"],
                    help="Merkle hash of the basefold workload (the transcript is Poseidon2 either way); the headline "
                         "metric names Poseidon2, the reference's default cargo features select Monolith")
    args = ap.parse_args()
    if args.workload == "batched_sumcheck":
        if args.impl == "reference":
            run_reference_batched(args)
        else:
            run_batched(args)
        return
    if args.workload in ("sumcheck", "ajtai", "mcommit"):
        run_simple(args)
        return
    if args.workload == "link":
        run_link(args)
        return
    if args.workload == "llama_layer":
        run_llama_layer(args)
        return
    if args.workload == "peval":
        run_peval(args)
        return
    if args.workload == "same_point":
        run_same_point(args)
        return

    if args.impl == "reference":
        run_reference(args)
        return

    run_basefold(args)


if __name__ == "__main__":
    main()
