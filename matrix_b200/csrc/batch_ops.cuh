// Element-wise batch operations over a prime field and its quadratic extension,
// shared by the Goldilocks and the almost-Goldilocks libraries
// (goldilocks-cuda-rs/cuda/wrapper.cu:100-575,1807-1860 and the agl_/aext2_
// twins in almost-goldilocks-cuda-rs/cuda/wrapper.cu). One grid-stride kernel
// per operation, 128-bit accesses for extension elements, canonical outputs.
// Like the reference's, the calls return after the launch (asynchronous on the
// caller's stream).
#pragma once
#include "common.cuh"

namespace mb {
namespace bo {

// F wraps a field namespace (gl or agl): add, sub, mul, inv, pw, canon and the
// extension type E2 with e2_add, e2_sub, e2_mul, e2_inv, e2_load, e2_store, e2_canon.
#define MB_FIELD_ADAPTER(Name, ns)                                                                              \
    struct Name {                                                                                               \
        using E2 = ns::E2;                                                                                      \
        static __device__ __forceinline__ uint64_t add(uint64_t a, uint64_t b) { return ns::add(a, b); }        \
        static __device__ __forceinline__ uint64_t sub(uint64_t a, uint64_t b) { return ns::sub(a, b); }        \
        static __device__ __forceinline__ uint64_t mul(uint64_t a, uint64_t b) { return ns::mul(a, b); }        \
        static __device__ __forceinline__ uint64_t inv(uint64_t a) { return ns::inv(a); }                       \
        static __device__ __forceinline__ uint64_t pw(uint64_t a, uint64_t e) { return ns::pw(a, e); }          \
        static __device__ __forceinline__ uint64_t canon(uint64_t a) { return ns::canon(a); }                   \
        static __device__ __forceinline__ E2 e2_add(E2 a, E2 b) { return ns::e2_add(a, b); }                    \
        static __device__ __forceinline__ E2 e2_sub(E2 a, E2 b) { return ns::e2_sub(a, b); }                    \
        static __device__ __forceinline__ E2 e2_mul(E2 a, E2 b) { return ns::e2_mul(a, b); }                    \
        static __device__ __forceinline__ E2 e2_inv(E2 a) { return ns::e2_inv(a); }                             \
        static __device__ __forceinline__ E2 e2_load(const uint64_t* p) { return ns::e2_load(p); }              \
        static __device__ __forceinline__ void e2_store(uint64_t* p, E2 v) { ns::e2_store(p, ns::e2_canon(v)); } \
    }

enum Op { ADD, SUB, MUL, DIV, NEG, SQUARE, DOUBLE, INV, MUL_SCALAR, EXP, CONJ, SCALE_ACC };

template <class F, int OP>
__global__ void __launch_bounds__(256)
base_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b, uint64_t* __restrict__ r, size_t n, uint64_t s) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        uint64_t x = a[i], y;
        if (OP == ADD) y = F::add(x, b[i]);
        else if (OP == SUB) y = F::sub(x, b[i]);
        else if (OP == MUL) y = F::mul(x, b[i]);
        else if (OP == DIV) y = F::mul(x, F::inv(b[i]));
        else if (OP == NEG) y = F::sub(0, x);
        else if (OP == SQUARE) y = F::mul(x, x);
        else if (OP == DOUBLE) y = F::add(x, x);
        else if (OP == INV) y = F::inv(x);
        else if (OP == MUL_SCALAR) y = F::mul(s, x);
        else y = F::pw(x, s);
        r[i] = F::canon(y);
    }
}

template <class F, int OP>
__global__ void __launch_bounds__(256)
ext_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b, uint64_t* r, size_t n, uint64_t s0, uint64_t s1) {
    using E2 = typename F::E2;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        E2 x = F::e2_load(a + 2 * i), y;
        if (OP == ADD) y = F::e2_add(x, F::e2_load(b + 2 * i));
        else if (OP == SUB) y = F::e2_sub(x, F::e2_load(b + 2 * i));
        else if (OP == MUL) y = F::e2_mul(x, F::e2_load(b + 2 * i));
        else if (OP == NEG) y = E2{F::sub(0, x.c0), F::sub(0, x.c1)};
        else if (OP == SQUARE) y = F::e2_mul(x, x);
        else if (OP == INV) y = F::e2_inv(x);
        else if (OP == CONJ) y = E2{x.c0, F::sub(0, x.c1)};  // also the Frobenius map: X^p = -X
        else if (OP == MUL_SCALAR) y = E2{F::mul(s0, x.c0), F::mul(s0, x.c1)};
        else if (OP == SCALE_ACC) y = F::e2_add(F::e2_load(r + 2 * i), F::e2_mul(E2{s0, s1}, x));
        else {  // EXP: square and multiply, low bit first
            y = E2{1, 0};
            E2 p = x;
            for (uint64_t e = s0; e; e >>= 1) {
                if (e & 1) y = F::e2_mul(y, p);
                p = F::e2_mul(p, p);
            }
        }
        F::e2_store(r + 2 * i, y);
    }
}

template <class F>
__global__ void lift_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        *reinterpret_cast<ulonglong2*>(out + 2 * i) = make_ulonglong2(F::canon(in[i]), 0);
}
template <class F>
__global__ void project_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) out[i] = F::canon(in[2 * i]);
}

// out[new] = in[old], bit `b` of new taken to bit inv_perm[b] of old (gather:
// coalesced writes). At most 31 index bits, like the reference's int indices.
static __global__ void bit_permute_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out,
                                          const int* __restrict__ inv_perm, int n_bits, size_t total) {
    __shared__ int perm[32];
    if (threadIdx.x < 32) perm[threadIdx.x] = threadIdx.x < n_bits ? inv_perm[threadIdx.x] : 0;
    __syncthreads();
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        size_t old = 0;
        for (int b = 0; b < n_bits; b++)
            if ((i >> b) & 1) old |= (size_t)1 << perm[b];
        out[i] = in[old];
    }
}

template <class F, int OP>
inline int run_base(const char* name, const uint64_t* a, const uint64_t* b, uint64_t* r, int n, uint64_t s = 0) {
    constexpr bool binary = OP == ADD || OP == SUB || OP == MUL || OP == DIV;
    if (n < 0 || !a || !r || (binary && !b)) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL(name);
    base_kernel<F, OP><<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(a, b, r, (size_t)n, s);
    return finish_async();
}
template <class F, int OP>
inline int run_ext(const char* name, const uint64_t* a, const uint64_t* b, uint64_t* r, int n, uint64_t s0 = 0, uint64_t s1 = 0) {
    constexpr bool binary = OP == ADD || OP == SUB || OP == MUL;
    if (n < 0 || !a || !r || (binary && !b)) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL(name);
    ext_kernel<F, OP><<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(a, b, r, (size_t)n, s0, s1);
    return finish_async();
}
template <class F>
inline int run_lift(const uint64_t* in, uint64_t* out, int n) {
    if (n < 0 || !in || !out) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("lift_to_ext2");
    lift_kernel<F><<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(in, out, (size_t)n);
    return finish_async();
}
template <class F>
inline int run_project(const uint64_t* in, uint64_t* out, int n) {
    if (n < 0 || !in || !out) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("ext2_to_base");
    project_kernel<F><<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(in, out, (size_t)n);
    return finish_async();
}
inline int run_bit_permute(const uint64_t* in, uint64_t* out, const int* d_inv_perm, int n_bits, int total) {
    if (!in || !out || !d_inv_perm || n_bits < 0 || n_bits > 31 || total < 0 || (size_t)total > ((size_t)1 << n_bits))
        return MB_ERR_ARG;
    if (total == 0) return MB_OK;
    MB_KERNEL("bit_permute");
    bit_permute_kernel<<<grid_for((size_t)total, 256, 8), 256, 0, MB_STREAM>>>(in, out, d_inv_perm, n_bits, (size_t)total);
    return finish_async();
}
inline int run_zero(uint64_t* buf, size_t n) {
    if (!buf && n) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    return cudaMemsetAsync(buf, 0, n * sizeof(uint64_t), MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}

}  // namespace bo
}  // namespace mb
