// Folding of Ajtai witnesses and commitments by short ring challenges
// (reference: cuda_almost_goldilocks/ajtai.cuh:700-1255; Rust callers
// almost-goldilocks-cuda-rs/src/ajtai.rs:397-1497, zk-torch-4/src/fold/multifold.rs).
//
//   witness     z'[j] = sum_i r_i * z_i[j]   in Z[X]/(X^64 + 1), z_i binary (bit masks) or ternary (pos / neg masks),
//                                            r_i with coefficients in {-1, 0, 1, 2}; 16-bit result
//   commitment  c'[i] = sum_m r_m * c_m[i]   in F_q[X]/(X^64 + 1)
//   split       16-bit coefficients back to 13 ternary planes
//
// This file holds the scalar forms (one thread per output coefficient); the
// witness fold on the tensor cores lives in ajtai_fold_tc.cuh.
#pragma once
#include "common.cuh"
#include "agl_field.cuh"

namespace mb {
namespace aj {

struct Challenge64 {
    int8_t c[64];
};

// Negacyclic extension: coefficient of X^(k - l) in r, with the sign of the wrap.
__device__ __forceinline__ int r_at(const int8_t* r, int k, int l) {
    const int v = r[(k - l) & 63];
    return l <= k ? v : -v;
}

// out[j][k] = z_first[j]_k + sum over instances of (r_i * z_i[j])_k. Instances: num_binary masks in
// zbin[i * N + j], then num_ternary pairs pos / neg[t * N + j]; r_all holds their challenges in that order;
// z_first (may be null) is a binary witness with the implicit challenge 1 (the two-instance fold of the
// reference). OUT16: 16-bit result, otherwise the canonical field element.
template <bool OUT16>
__global__ void __launch_bounds__(64)
multifold_witness_scalar_kernel(const uint64_t* __restrict__ z_first, const uint64_t* __restrict__ zbin,
                                const uint64_t* __restrict__ pos, const uint64_t* __restrict__ neg,
                                const int8_t* __restrict__ r_all, void* __restrict__ out, int num_binary, int num_ternary,
                                uint64_t N) {
    extern __shared__ int8_t r_sh[];
    const int k = threadIdx.x, total = num_binary + num_ternary;
    for (int t = k; t < total * 64; t += 64) r_sh[t] = r_all[t];
    __syncthreads();
    for (uint64_t j = blockIdx.x; j < N; j += gridDim.x) {
        int acc = z_first ? (int)((z_first[j] >> k) & 1) : 0;
        for (int i = 0; i < total; i++) {
            uint64_t p = i < num_binary ? zbin[(uint64_t)i * N + j] : pos[(uint64_t)(i - num_binary) * N + j];
            uint64_t m = i < num_binary ? 0 : neg[(uint64_t)(i - num_binary) * N + j];
            const int8_t* r = r_sh + i * 64;
            while (p) {
                const int l = __ffsll((long long)p) - 1;
                p &= p - 1;
                acc += r_at(r, k, l);
            }
            while (m) {
                const int l = __ffsll((long long)m) - 1;
                m &= m - 1;
                acc -= r_at(r, k, l);
            }
        }
        if (OUT16) static_cast<int16_t*>(out)[j * 64 + k] = (int16_t)acc;
        else static_cast<uint64_t*>(out)[j * 64 + k] = acc >= 0 ? (uint64_t)acc : agl::P - (uint64_t)(-acc);
    }
}

// out[i][k] = base[i][k] + sum_m (r_m * c_m[i])_k, i < 42; block = (row i), 64 threads. The terms are small
// multiples (|r| <= 127) of field elements: positive and negative parts are summed exactly and reduced once.
static __global__ void __launch_bounds__(64)
multifold_commitment_kernel(const uint64_t* __restrict__ base, const uint64_t* __restrict__ c_all,
                            const int8_t* __restrict__ r_all, int num_instances, uint64_t* __restrict__ out) {
    extern __shared__ int8_t r_sh[];
    __shared__ uint64_t c_sh[64];
    const int i = blockIdx.x, k = threadIdx.x;
    for (int t = k; t < num_instances * 64; t += 64) r_sh[t] = r_all[t];
    gl::Acc plus = gl::acc_zero(), minus = gl::acc_zero();
    if (base) gl::acc_add(plus, agl::canon(base[i * 64 + k]));
    for (int m = 0; m < num_instances; m++) {
        __syncthreads();
        c_sh[k] = agl::canon(c_all[((size_t)m * 42 + i) * 64 + k]);
        __syncthreads();
        const int8_t* r = r_sh + m * 64;
        for (int l = 0; l < 64; l++) {
            const int rv = r[l];
            if (rv == 0) continue;
            const bool positive = (l <= k) == (rv > 0);
            const uint64_t mag = (uint64_t)(rv < 0 ? -rv : rv);
            gl::acc_mul(positive ? plus : minus, c_sh[(k - l) & 63], mag);
        }
    }
    out[i * 64 + k] = agl::canon(agl::sub(agl::acc_reduce(plus), agl::acc_reduce(minus)));
}

}  // namespace aj
}  // namespace mb
