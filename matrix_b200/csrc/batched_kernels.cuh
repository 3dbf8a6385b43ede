// Batched degree-3 sumcheck with a shared eq table:
//   claim   S = sum_k alpha^k sum_x eq(t, x) a_k(x) b_k(x),   k < K instances
//   message m(c) = sum_y eq(c, y) sum_k alpha^k a_k(c, y) b_k(c, y),   c = 0..3
// (the composition of the reference's same-point batched sumcheck,
// zk-torch-4/src/fold/same_point_sumcheck.rs:58-157, with the three-table
// linear prover zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100; low variable
// first). One thread handles one output pair y for all instances, so the eq
// pair is loaded once and only four accumulators are live. Round 0 runs on the
// base-field tables; its fold lifts them to the extension and multiplies a_k by
// alpha^k once, so every later round needs one extension product per instance
// and evaluation point. The fold is fused with the next message: each round
// streams the 2K + 1 tables through HBM once.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace bt {

constexpr int MAX_K = 64;
constexpr int NC = 4;  // evaluation points c = 0..3

// Block partial rows of 8 words, last block sums them (same pattern as the linear prover).
template <class FE>
__device__ __forceinline__ void finish_message(typename FE::T (&m)[NC], uint64_t* partial, unsigned int* counter,
                                               uint64_t* final_out) {
    uint64_t v[2 * NC];
#pragma unroll
    for (int c = 0; c < NC; c++) FE::to_words(m[c], v + 2 * c);
    sc::block_sum_store<2 * NC>(v, partial + 2 * NC * (size_t)blockIdx.x, typename FE::WordAdd(), typename FE::WordCanon());
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll
    for (int k = 0; k < 2 * NC; k++) v[k] = 0;
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x)
#pragma unroll
        for (int k = 0; k < 2 * NC; k++) v[k] = typename FE::WordAdd()(v[k], __ldcg(partial + 2 * NC * (size_t)b + k));
    sc::block_sum_store<2 * NC>(v, final_out, typename FE::WordAdd(), typename FE::WordCanon());
    if (threadIdx.x == 0) *counter = 0;
}

// Round 0 message from the caller's base-field tables a0, b0: [K][stride] each;
// eq: extension; alpha_pows: K extension elements in global memory.
template <class FB, class FE>
__global__ void __launch_bounds__(256)
round0_message_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ a0p, const uint64_t* __restrict__ b0p,
                      const uint64_t* __restrict__ alpha_pows, int K, size_t stride, size_t half, uint64_t* partial,
                      unsigned int* counter, uint64_t* final_out) {
    using TE = typename FE::T;
    TE m[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) m[c] = FE::zero();
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
        TE inner[NC];
#pragma unroll
        for (int c = 0; c < NC; c++) inner[c] = FE::zero();
        for (int k = 0; k < K; k++) {
            uint64_t a0, a1, b0, b1;
            FB::load2(a0p + (size_t)k * stride, 2 * y, a0, a1);
            FB::load2(b0p + (size_t)k * stride, 2 * y, b0, b1);
            const TE w = FE::load(alpha_pows, k);
            uint64_t da = FB::sub(a1, a0), db = FB::sub(b1, b0), va = a0, vb = b0;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                uint64_t pr = FB::mul(va, vb);
                inner[c] = FE::add(inner[c], TE{FB::mul(w.c0, pr), FB::mul(w.c1, pr)});
                va = FB::add(va, da);
                vb = FB::add(vb, db);
            }
        }
        TE e0, e1;
        FE::load2(eq, 2 * y, e0, e1);
        TE de = FE::sub(e1, e0), ve = e0;
#pragma unroll
        for (int c = 0; c < NC; c++) {
            m[c] = FE::add(m[c], FE::mul(ve, inner[c]));
            ve = FE::add(ve, de);
        }
    }
    finish_message<FE>(m, partial, counter, final_out);
}

// Per-instance claims s_k = sum_x eq(x) a_k(x) b_k(x) from the base-field tables:
// partial[(block * K + k) * 2 ...]; summed by reduce_partials_kernel.
template <class FB, class FE>
__global__ void __launch_bounds__(256)
claims_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ a0p, const uint64_t* __restrict__ b0p, int K,
              size_t stride, size_t n,
              uint64_t* __restrict__ partial) {
    using TE = typename FE::T;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (int k = 0; k < K; k++) {
        TE acc = FE::zero();
        for (size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x; x < n; x += step) {
            uint64_t pr = FB::mul(a0p[(size_t)k * stride + x], b0p[(size_t)k * stride + x]);
            TE e = FE::load(eq, x);
            acc = FE::add(acc, TE{FB::mul(e.c0, pr), FB::mul(e.c1, pr)});
        }
        uint64_t v[2] = {acc.c0, acc.c1};
        sc::block_sum_store<2>(v, partial + ((size_t)blockIdx.x * K + k) * 2, typename FE::WordAdd(), typename FE::WordCanon());
        __syncthreads();
    }
}

// Fold every table on r and accumulate the next message. FIRST: inputs a, b are
// base field and the folded a_k is multiplied by alpha^k; otherwise all tables
// are extension tables (a_k already scaled). quarter = live length / 4. With
// FIRST, ab_in / b_first are the caller's [K][stride] base tables a and b;
// otherwise ab_in is [K][2][stride] extension tables and b_first is unused.
template <class FB, class FE, bool FIRST>
__global__ void __launch_bounds__(256)
fold_message_kernel(const uint64_t* __restrict__ eq_in, uint64_t* __restrict__ eq_out, const uint64_t* __restrict__ ab_in,
                    const uint64_t* __restrict__ b_first, uint64_t* __restrict__ ab_out, const uint64_t* __restrict__ alpha_pows, typename FE::T r, int K,
                    size_t stride_in, size_t stride_out, size_t quarter, uint64_t* partial, unsigned int* counter,
                    uint64_t* final_out) {
    using TE = typename FE::T;
    TE m[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) m[c] = FE::zero();
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < quarter; y += step) {
        TE inner[NC];
#pragma unroll
        for (int c = 0; c < NC; c++) inner[c] = FE::zero();
        for (int k = 0; k < K; k++) {
            TE fa0, fa1, fb0, fb1;
            if (FIRST) {
                uint64_t x0, x1, x2, x3;
                const uint64_t* pa = ab_in + (size_t)k * stride_in;
                FB::load2(pa, 4 * y, x0, x1);
                FB::load2(pa, 4 * y + 2, x2, x3);
                const TE w = FE::load(alpha_pows, k);
                fa0 = FE::mul(w, sc::FoldOp<FB, FE>::apply(x0, x1, r));
                fa1 = FE::mul(w, sc::FoldOp<FB, FE>::apply(x2, x3, r));
                const uint64_t* pb = b_first + (size_t)k * stride_in;
                FB::load2(pb, 4 * y, x0, x1);
                FB::load2(pb, 4 * y + 2, x2, x3);
                fb0 = sc::FoldOp<FB, FE>::apply(x0, x1, r);
                fb1 = sc::FoldOp<FB, FE>::apply(x2, x3, r);
            } else {
                TE x0, x1, x2, x3;
                const uint64_t* pa = ab_in + (size_t)(2 * k) * stride_in * 2;
                FE::load2(pa, 4 * y, x0, x1);
                FE::load2(pa, 4 * y + 2, x2, x3);
                fa0 = sc::FoldOp<FE, FE>::apply(x0, x1, r);
                fa1 = sc::FoldOp<FE, FE>::apply(x2, x3, r);
                const uint64_t* pb = ab_in + (size_t)(2 * k + 1) * stride_in * 2;
                FE::load2(pb, 4 * y, x0, x1);
                FE::load2(pb, 4 * y + 2, x2, x3);
                fb0 = sc::FoldOp<FE, FE>::apply(x0, x1, r);
                fb1 = sc::FoldOp<FE, FE>::apply(x2, x3, r);
            }
            FE::store2(ab_out + (size_t)(2 * k) * stride_out * 2, 2 * y, fa0, fa1);
            FE::store2(ab_out + (size_t)(2 * k + 1) * stride_out * 2, 2 * y, fb0, fb1);
            TE da = FE::sub(fa1, fa0), db = FE::sub(fb1, fb0), va = fa0, vb = fb0;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                inner[c] = FE::add(inner[c], FE::mul(va, vb));
                va = FE::add(va, da);
                vb = FE::add(vb, db);
            }
        }
        TE e0, e1, e2, e3;
        FE::load2(eq_in, 4 * y, e0, e1);
        FE::load2(eq_in, 4 * y + 2, e2, e3);
        TE q0 = sc::FoldOp<FE, FE>::apply(e0, e1, r), q1 = sc::FoldOp<FE, FE>::apply(e2, e3, r);
        FE::store2(eq_out, 2 * y, q0, q1);
        TE de = FE::sub(q1, q0), ve = q0;
#pragma unroll
        for (int c = 0; c < NC; c++) {
            m[c] = FE::add(m[c], FE::mul(ve, inner[c]));
            ve = FE::add(ve, de);
        }
    }
    finish_message<FE>(m, partial, counter, final_out);
}

// Last fold (two live elements per table): no message.
template <class FB, class FE, bool FIRST>
__global__ void final_fold_kernel(const uint64_t* __restrict__ eq_in, uint64_t* __restrict__ eq_out,
                                  const uint64_t* __restrict__ ab_in, const uint64_t* __restrict__ b_first,
                                  uint64_t* __restrict__ ab_out,
                                  const uint64_t* __restrict__ alpha_pows, typename FE::T r, int K, size_t stride_in,
                                  size_t stride_out) {
    using TE = typename FE::T;
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t == 2 * K) {
        TE e0, e1;
        FE::load2(eq_in, 0, e0, e1);
        FE::store(eq_out, 0, sc::FoldOp<FE, FE>::apply(e0, e1, r));
        return;
    }
    if (t > 2 * K) return;
    TE f;
    if (FIRST) {
        uint64_t x0, x1;
        FB::load2(((t & 1) ? b_first : ab_in) + (size_t)(t >> 1) * stride_in, 0, x0, x1);
        f = sc::FoldOp<FB, FE>::apply(x0, x1, r);
        if ((t & 1) == 0) f = FE::mul(FE::load(alpha_pows, t >> 1), f);
    } else {
        TE x0, x1;
        FE::load2(ab_in + (size_t)t * stride_in * 2, 0, x0, x1);
        f = sc::FoldOp<FE, FE>::apply(x0, x1, r);
    }
    FE::store(ab_out + (size_t)t * stride_out * 2, 0, f);
}

}  // namespace bt
}  // namespace mb
