"""Writes tests/golden/ffi_symbols.json: the names of every extern "C" function the reference's two Rust crates
declare (goldilocks-cuda-rs/src/ffi.rs, almost-goldilocks-cuda-rs/src/ffi.rs). Names only; run where the
reference tree is present:  python tests/golden/make_ffi_symbols.py [reference root]"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def names(path):
    return re.findall(r"pub fn (\w+)\s*\(", open(path).read())


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    out = {"goldilocks_cuda_wrapper": names(os.path.join(ref, "goldilocks-cuda-rs", "src", "ffi.rs")),
           "almost_goldilocks_cuda_wrapper": names(os.path.join(ref, "almost-goldilocks-cuda-rs", "src", "ffi.rs"))}
    with open(os.path.join(HERE, "ffi_symbols.json"), "w") as f:
        json.dump(out, f, indent=0)
    print({k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
