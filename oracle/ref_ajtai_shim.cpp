// Builds the reference's OWN host-side Ajtai code (ajtai_cpu_reference.cuh,
// ajtai_chacha8.cuh, almost_goldilocks.cuh are __host__ __device__ / host code)
// into oracle/_ref/libajtai_ref.so, to pin the oracle and the kernels against
// what the reference computes. Compiled from the reference tree where it lies by
// `make ref`; no reference source is copied. Test infrastructure only.
#include <cuda_runtime.h>
#include <cstdint>
#include <vector>
#include "almost_goldilocks.cuh"
#include "ajtai_chacha8.cuh"
#include "ajtai_cpu_reference.cuh"

extern "C" {

// out[b][i][r] for B dense binary planes z[b*N + j] (cpu_ajtai_commit_batched)
void ref_ajtai_commit_dense(const uint32_t* key, const uint64_t* z, uint64_t N, int B, uint64_t* out) {
    auto res = ajtai_cpu::cpu_ajtai_commit_batched<64, 42>(key, z, N, B);
    for (size_t k = 0; k < res.size(); k++)
        for (int r = 0; r < 64; r++) out[k * 64 + r] = res[k][r];
}

// cpu_ajtai_commit_sparse over a position list; out[i][r]
void ref_ajtai_commit_sparse(const uint32_t* key, const uint64_t* positions, uint64_t K, uint64_t* out) {
    auto res = ajtai_cpu::cpu_ajtai_commit_sparse<64, 42>(key, positions, K);
    for (size_t k = 0; k < res.size(); k++)
        for (int r = 0; r < 64; r++) out[k * 64 + r] = res[k][r];
}

void ref_ajtai_ring_elem(const uint32_t* key, int row, uint64_t j, uint64_t* out) {
    auto e = ajtai_cpu::cpu_prg_ring_elem<64>(key, row, j);
    for (int r = 0; r < 64; r++) out[r] = e[r];
}

// One negacyclic product with the reference's cpu_ring_mul.
void ref_ring_mul(const uint64_t* a, const uint64_t* b, uint64_t* out) {
    ajtai_cpu::Ring<64> ra, rb;
    for (int r = 0; r < 64; r++) { ra[r] = a[r]; rb[r] = b[r]; }
    auto c = ajtai_cpu::cpu_ring_mul<64>(ra, rb);
    for (int r = 0; r < 64; r++) out[r] = c[r];
}

void ref_chacha8_block(const uint32_t* key, uint32_t counter, const uint32_t* nonce, uint32_t* out) {
    chacha8_block(key, counter, nonce, out);
}

uint64_t ref_agl_mul(uint64_t a, uint64_t b) {
    return agl_canonicalize(agl_mul(AlmostGoldilocksField(a), AlmostGoldilocksField(b)).value);
}

}  // extern "C"
