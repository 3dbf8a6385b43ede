"""Builds the CUDA libraries of this package in-tree with nvcc for sm_100a.

    python -m matrix_b200.build          # incremental
    python -m matrix_b200.build --force  # rebuild everything

Outputs (kept out of version control, shipped alongside the sources):
    matrix_b200/lib/libgoldilocks_cuda_wrapper.so         Goldilocks C-ABI
    matrix_b200/lib/libalmost_goldilocks_cuda_wrapper.so  almost-Goldilocks C-ABI
The library names are the ones the reference's Rust crates link
(goldilocks-cuda-rs/src/ffi.rs:5, almost-goldilocks-cuda-rs/src/ffi.rs).
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "_obj")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--default-stream", "per-thread",
         "-Xcompiler", "-fPIC", "-ccbin", "g++"]

LIBRARIES = {
    "libgoldilocks_cuda_wrapper.so": [
        "gl_memory.cu",
        "prof.cu",
        "gl_sumcheck.cu",
        "gl_noalloc.cu",
        "gl_merkle.cu",
        "gl_batch.cu",
        "gl_basefold.cu",
        "gl_challenger.cu",
        "gl_stubs.cu",
        "host/gl_sumcheck_prover.cu",
        "host/gl_basefold_prover.cu",
        "host/gl_basefold_sharded.cu",
        "host/gl_basefold_verifier.cu",
        "host/exchange.cu",
        "host/gl_batched_prover.cu",
    ],
    "libalmost_goldilocks_cuda_wrapper.so": [
        "gl_memory.cu",
        "prof.cu",
        "agl_wrapper.cu",
        "agl_ajtai.cu",
        "agl_batch.cu",
        "agl_k8.cu",
        "agl_mcommit.cu",
        "agl_link.cu",
        "agl_bool.cu",
        "agl_batched.cu",
        "agl_ajtai_fold.cu",
        "agl_stubs.cu",
        "host/agl_transcript.cu",
        "host/agl_sumcheck_prover.cu",
        "host/agl_same_point_prover.cu",
        "host/agl_einsum_prover.cu",
    ],
}


def _headers():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cuh", ".hpp", ".h")):
                out.append(os.path.join(root, f))
    return out


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, obj, verbose):
    cmd = [NVCC] + ARCH + FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return r.stderr


def build(force=False, verbose=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    jobs = []
    for lib, srcs in LIBRARIES.items():
        for s in srcs:
            src = os.path.join(CSRC, s)
            obj = os.path.join(OBJ, s.replace("/", "_") + ".o")
            if force or _newer(obj, [src] + headers):
                jobs.append((src, obj))
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda j: _compile(j[0], j[1], verbose), jobs))
    for lib, srcs in LIBRARIES.items():
        objs = [os.path.join(OBJ, s.replace("/", "_") + ".o") for s in srcs]
        out = os.path.join(LIB, lib)
        if force or _newer(out, objs):
            cmd = [NVCC] + ARCH + ["-shared", "-o", out] + objs + ["-ccbin", "g++"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("link failed for %s:\n%s\n%s" % (lib, r.stdout, r.stderr))
    return logs


if __name__ == "__main__":
    for log in build(force="--force" in sys.argv, verbose="-v" in sys.argv):
        if "-v" in sys.argv:
            sys.stderr.write(log)
    print("built:", ", ".join(sorted(os.listdir(LIB))))
