// Builds the reference's OWN Goldilocks device headers for the host (g++ treats
// the CUDA function qualifiers as ignorable attributes), to pin the oracle
// against what the reference code actually computes. Compiled from the
// reference tree where it lies into oracle/_ref/ by `make ref`; no reference
// source is copied. Test infrastructure only.
#include <cuda_runtime.h>
#include <cstring>
#include "poseidon2.cuh"

static void load_tables() {
    memcpy(d_RC_EXT_8, h_RC_EXT_8, sizeof(h_RC_EXT_8));
    memcpy(d_RC_INT, h_RC_INT, sizeof(h_RC_INT));
    memcpy(d_DIAG_8, h_DIAG_8, sizeof(h_DIAG_8));
}

extern "C" void ref_poseidon2_permute_8(uint64_t* s) {
    load_tables();
    GoldilocksField st[8];
    for (int i = 0; i < 8; i++) st[i] = GoldilocksField(s[i]);
    poseidon2_permute_8(st);
    for (int i = 0; i < 8; i++) s[i] = canonicalize(st[i].value);
}

extern "C" uint64_t ref_gl_mul(uint64_t a, uint64_t b) {
    return canonicalize(gl_mul(GoldilocksField(a), GoldilocksField(b)).value);
}
