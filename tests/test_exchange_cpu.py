"""The exchange objects of the sharded provers, host side only (no GPU): ranks as threads of one process, and
ranks as processes over the mailbox in POSIX shared memory, with messages longer than a slot and many rounds."""
import ctypes
import multiprocessing as mp
import os
import threading

import numpy as np

from matrix_b200.ffi import load_gl


def _message(rank, rnd, words):
    return (np.arange(words, dtype=np.uint64) * np.uint64(1000003) + np.uint64(rank * 7919 + rnd * 104729)).astype(np.uint64)


def test_local_exchange_gathers_between_threads():
    lib = load_gl()
    world, rounds = 4, 50
    exs = (ctypes.c_void_p * world)()
    assert lib.mb_exchange_local_create(world, exs) == 0
    errors = []

    def run(r):
        for rnd in range(rounds):
            words = 1 + (rnd * 37) % 300
            mine = _message(r, rnd, words)
            out = np.zeros(world * words, dtype=np.uint64)
            if lib.mb_exchange_all_gather_host(exs[r], mine.ctypes.data, words, out.ctypes.data) != 0:
                errors.append((r, rnd, "rc"))
                return
            for g in range(world):
                if not np.array_equal(out[g * words:(g + 1) * words], _message(g, rnd, words)):
                    errors.append((r, rnd, g))

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
    for r in range(world):
        lib.mb_exchange_destroy(exs[r])


def _shm_worker(name, rank, world, rounds, slot_words, q):
    lib = load_gl()
    ex = ctypes.c_void_p()
    if lib.mb_exchange_shm_create(name.encode(), rank, world, slot_words, None, None, ctypes.byref(ex)) != 0:
        q.put((rank, "create failed"))
        return
    bad = None
    for rnd in range(rounds):
        words = 1 + (rnd * 53) % 500          # up to several slots per message
        mine = _message(rank, rnd, words)
        out = np.zeros(world * words, dtype=np.uint64)
        if lib.mb_exchange_all_gather_host(ex, mine.ctypes.data, words, out.ctypes.data) != 0:
            bad = "rc at round %d" % rnd
            break
        for g in range(world):
            if not np.array_equal(out[g * words:(g + 1) * words], _message(g, rnd, words)):
                bad = "round %d: piece of rank %d" % (rnd, g)
                break
        if bad:
            break
    # a device all-to-all without a supplied function is refused, not attempted
    if bad is None and lib.mb_exchange_all_to_all_device(ex, 8, 8, 1) != -4:
        bad = "all_to_all without a function"
    lib.mb_exchange_destroy(ex)
    q.put((rank, bad))


def test_shm_exchange_gathers_between_processes():
    world, rounds, slot_words = 3, 200, 64
    name = "/mb_test_exchange_%d" % os.getpid()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_shm_worker, args=(name, r, world, rounds, slot_words, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(bad is None for _, bad in results), results


def test_a_missing_rank_times_out_with_an_error_code(monkeypatch):
    """Two ranks expected, one shows up: the wait is bounded and the call returns -4."""
    monkeypatch.setenv("MB_EXCHANGE_TIMEOUT_S", "0.5")
    code = ("import ctypes, numpy as np\n"
            "from matrix_b200.ffi import load_gl\n"
            "lib = load_gl(); ex = ctypes.c_void_p()\n"
            "assert lib.mb_exchange_shm_create(b'/mb_test_timeout_%d', 0, 2, 64, None, None, ctypes.byref(ex)) == 0\n"
            "a = np.ones(4, dtype=np.uint64); o = np.zeros(8, dtype=np.uint64)\n"
            "print('RC', lib.mb_exchange_all_gather_host(ex, a.ctypes.data, 4, o.ctypes.data))\n"
            "lib.mb_exchange_destroy(ex)\n") % os.getpid()
    import subprocess
    import sys
    from .conftest import ROOT
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=60,
                         env=dict(os.environ, MB_EXCHANGE_TIMEOUT_S="0.5"))
    assert "RC -4" in out.stdout, out.stdout + out.stderr
