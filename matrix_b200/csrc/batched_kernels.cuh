// Batched degree-3 sumcheck with a shared eq table over Goldilocks:
//   claim   S = sum_k alpha^k sum_x eq(t, x) a_k(x) b_k(x),   k < K instances
//   message m(c) = sum_y eq(c, y) sum_k alpha^k a_k(c, y) b_k(c, y),   c = 0..3
// (the composition of the reference's same-point batched sumcheck,
// zk-torch-4/src/fold/same_point_sumcheck.rs:58-157, with the three-table
// linear prover zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100; low variable
// first).
//
// Round 0 works on the caller's base-field tables and is independent of alpha:
// one pass produces, per instance, m_k(0..3) = sum_y eq(c, y) a_k(c, y) b_k(c, y);
// the claims are s_k = m_k(0) + m_k(1) and the round-0 message is
// sum_k alpha^k m_k(c), combined on the host. The first fold lifts the tables to
// the extension and multiplies a_k by alpha^k once; every later pass folds the
// 2K + 1 tables and accumulates the next message in the same sweep.
//
// Arithmetic: all multiplications feed exact 160-bit sums that are reduced once
// (gl::Acc). Per instance and output pair the inner polynomial
// Q(c) = sum_k a_k(c) b_k(c) is quadratic, so three lazily accumulated
// extension products (at c = 0, c = 1 and the leading coefficient) replace four
// reduced ones; Q(2), Q(3) follow by additions and eq(c) Q(c) is formed once
// per pair, not once per instance.
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

// ---- round 0: per-instance messages from the base-field tables ----------------------
// Lane l of a warp owns instance k = kbase + (l & (Kp - 1)) for the whole
// launch, so its eight exact sums (4 points x 2 components) are reduced only
// once at the end; the 32 / Kp lane groups of a warp take consecutive pairs of
// output pairs y, and the eq values eq(c, y), c = 0..3, of the warp's current
// pairs are computed once by the warp and shared through shared memory.
// eq: canonical extension table; a0p, b0p: [K][stride] (any representatives);
// half = number of pairs; partial: [gridDim.x][K][8] canonical words. Dynamic
// shared memory: warps * (64 / Kp) * 8 words.
static __global__ void __launch_bounds__(256)
instance_messages_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ a0p,
                         const uint64_t* __restrict__ b0p, int K, int Kp, size_t stride, size_t half,
                         uint64_t* __restrict__ partial) {
    extern __shared__ uint64_t dyn[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int G = 32 / Kp, g = lane / Kp;
    const int k = blockIdx.y * 32 + (lane & (Kp - 1));
    const bool live_k = k < K;
    const int ys_per_iter = 2 * G;
    uint64_t* ev = dyn + (size_t)warp * ys_per_iter * 8;  // [y][c][component]
    const uint64_t* pa = a0p + (size_t)(live_k ? k : 0) * stride;
    const uint64_t* pb = b0p + (size_t)(live_k ? k : 0) * stride;
    gl::Acc A[NC][2];
#pragma unroll
    for (int c = 0; c < NC; c++) A[c][0] = A[c][1] = gl::acc_zero();
    const size_t warps_total = (size_t)gridDim.x * nwarp, wg = (size_t)blockIdx.x * nwarp + warp;
    for (size_t ybase = wg * ys_per_iter; ybase < half; ybase += warps_total * ys_per_iter) {
        // eq(c, y) = e0 + c (e1 - e0) for the warp's pairs, one value per lane and step
        for (int j = lane; j < ys_per_iter * 8; j += 32) {
            const size_t y = ybase + (j >> 3);
            const int c = (j >> 1) & 3, comp = j & 1;
            uint64_t v = 0;
            if (y < half) {
                const uint64_t e0 = eq[4 * y + comp], e1 = eq[4 * y + 2 + comp];
                gl::Acc s = gl::Acc{e0, 0, 0};
                gl::acc_mul(s, (uint64_t)c, gl::sub_canon(e1, e0));
                v = gl::acc_reduce(s);
            }
            ev[j] = v;
        }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t y = ybase + 2 * g + h;
            if (y < half && live_k) {
                const ulonglong2 av2 = *reinterpret_cast<const ulonglong2*>(pa + 2 * y);
                const ulonglong2 bv2 = *reinterpret_cast<const ulonglong2*>(pb + 2 * y);
                const uint64_t a0 = gl::canon(av2.x), a1 = gl::canon(av2.y), b0 = gl::canon(bv2.x), b1 = gl::canon(bv2.y);
                const uint64_t da = gl::sub_canon(a1, a0), db = gl::sub_canon(b1, b0);
                uint64_t va = a0, vb = b0;
                const uint64_t* e = ev + (2 * g + h) * 8;
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    const uint64_t pr = gl::mul(va, vb);
                    gl::acc_mul(A[c][0], e[2 * c], pr);
                    gl::acc_mul(A[c][1], e[2 * c + 1], pr);
                    va = c == 0 ? a1 : gl::add_c(va, da);
                    vb = c == 0 ? b1 : gl::add_c(vb, db);
                }
            }
        }
        __syncwarp();
    }
    // lanes of one instance inside the warp, then the warps of the block
    uint64_t v[2 * NC];
#pragma unroll
    for (int c = 0; c < NC; c++) {
        v[2 * c] = gl::acc_reduce_wide(A[c][0]);
        v[2 * c + 1] = gl::acc_reduce_wide(A[c][1]);
    }
    for (int off = Kp; off < 32; off <<= 1)
#pragma unroll
        for (int j = 0; j < 2 * NC; j++) v[j] = gl::add(v[j], __shfl_xor_sync(0xffffffffu, v[j], off));
    __shared__ uint64_t across[8][32][2 * NC];
    if (lane < Kp)
#pragma unroll
        for (int j = 0; j < 2 * NC; j++) across[warp][lane][j] = v[j];
    __syncthreads();
    for (int t = threadIdx.x; t < Kp * 2 * NC; t += blockDim.x) {
        const int kk = t / (2 * NC), j = t % (2 * NC), kg = blockIdx.y * 32 + kk;
        if (kg >= K) continue;
        uint64_t s = 0;
        for (int w = 0; w < nwarp; w++) s = gl::add(s, across[w][kk][j]);
        partial[((size_t)blockIdx.x * K + kg) * 2 * NC + j] = gl::canon(s);
    }
}

// ---- fold every table on r and accumulate the next message -----------------------------
// FIRST: inputs are the caller's base-field tables a, b ([K][stride_in] each) and
// the folded a_k is multiplied by alpha^k; otherwise ab_in holds [2K][stride_in]
// canonical extension tables (a_k already scaled). quarter = live length / 4.
// wtab (FIRST only): per instance alpha^k and alpha^k r, four canonical words.
template <bool FIRST>
__global__ void __launch_bounds__(256)
fold_message_kernel(const uint64_t* __restrict__ eq_in, uint64_t* __restrict__ eq_out, const uint64_t* __restrict__ ab_in,
                    const uint64_t* __restrict__ b_first, uint64_t* __restrict__ ab_out,
                    const uint64_t* __restrict__ wtab, gl::E2 r, int K, size_t stride_in, size_t stride_out,
                    size_t quarter, uint64_t* partial, unsigned int* counter, uint64_t* final_out) {
    using FE = sc::GlExt2;
    using E2 = gl::E2;
    __shared__ uint64_t sw[FIRST ? 4 * MAX_K : 1];
    if (FIRST) {
        for (int t = threadIdx.x; t < 4 * K; t += blockDim.x) sw[t] = wtab[t];
        __syncthreads();
    }
    const gl::E2Pre rp = gl::e2_pre(r);
    E2 m[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) m[c] = E2{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < quarter; y += step) {
        gl::E2Acc q0 = gl::e2acc_zero(), q1 = gl::e2acc_zero(), q2 = gl::e2acc_zero();
        for (int k = 0; k < K; k++) {
            E2 fa0, fa1, fb0, fb1;
            if (FIRST) {
                const ulonglong2* pa = reinterpret_cast<const ulonglong2*>(ab_in + (size_t)k * stride_in + 4 * y);
                const ulonglong2* pb = reinterpret_cast<const ulonglong2*>(b_first + (size_t)k * stride_in + 4 * y);
                const ulonglong2 a01 = pa[0], a23 = pa[1], b01 = pb[0], b23 = pb[1];
                const uint64_t w0 = sw[4 * k], w1 = sw[4 * k + 1], wr0 = sw[4 * k + 2], wr1 = sw[4 * k + 3];
                // alpha^k (x0 + r d) = alpha^k x0 + (alpha^k r) d with base-field x0, d
                {
                    const uint64_t x0 = gl::canon(a01.x), d = gl::sub_canon(gl::canon(a01.y), x0);
                    gl::Acc s0 = gl::acc_zero(), s1 = gl::acc_zero();
                    gl::acc_mul(s0, w0, x0); gl::acc_mul(s0, wr0, d);
                    gl::acc_mul(s1, w1, x0); gl::acc_mul(s1, wr1, d);
                    fa0 = E2{gl::acc_reduce(s0), gl::acc_reduce(s1)};
                }
                {
                    const uint64_t x0 = gl::canon(a23.x), d = gl::sub_canon(gl::canon(a23.y), x0);
                    gl::Acc s0 = gl::acc_zero(), s1 = gl::acc_zero();
                    gl::acc_mul(s0, w0, x0); gl::acc_mul(s0, wr0, d);
                    gl::acc_mul(s1, w1, x0); gl::acc_mul(s1, wr1, d);
                    fa1 = E2{gl::acc_reduce(s0), gl::acc_reduce(s1)};
                }
                {
                    const uint64_t x0 = gl::canon(b01.x), d = gl::sub_canon(gl::canon(b01.y), x0);
                    fb0 = gl::e2_fma_pre_base(rp, d, x0);
                }
                {
                    const uint64_t x0 = gl::canon(b23.x), d = gl::sub_canon(gl::canon(b23.y), x0);
                    fb1 = gl::e2_fma_pre_base(rp, d, x0);
                }
            } else {
                const ulonglong2* pa = reinterpret_cast<const ulonglong2*>(ab_in + (size_t)(2 * k) * stride_in * 2 + 8 * y);
                const ulonglong2* pb = reinterpret_cast<const ulonglong2*>(ab_in + (size_t)(2 * k + 1) * stride_in * 2 + 8 * y);
                const ulonglong2 a0 = pa[0], a1 = pa[1], a2 = pa[2], a3 = pa[3];
                const ulonglong2 b0 = pb[0], b1 = pb[1], b2 = pb[2], b3 = pb[3];
                fa0 = gl::e2_fma_pre(rp, E2{gl::sub_canon(a1.x, a0.x), gl::sub_canon(a1.y, a0.y)}, E2{a0.x, a0.y});
                fa1 = gl::e2_fma_pre(rp, E2{gl::sub_canon(a3.x, a2.x), gl::sub_canon(a3.y, a2.y)}, E2{a2.x, a2.y});
                fb0 = gl::e2_fma_pre(rp, E2{gl::sub_canon(b1.x, b0.x), gl::sub_canon(b1.y, b0.y)}, E2{b0.x, b0.y});
                fb1 = gl::e2_fma_pre(rp, E2{gl::sub_canon(b3.x, b2.x), gl::sub_canon(b3.y, b2.y)}, E2{b2.x, b2.y});
            }
            fa0 = gl::e2_canon(fa0); fa1 = gl::e2_canon(fa1); fb0 = gl::e2_canon(fb0); fb1 = gl::e2_canon(fb1);
            ulonglong2* oa = reinterpret_cast<ulonglong2*>(ab_out + (size_t)(2 * k) * stride_out * 2 + 4 * y);
            ulonglong2* ob = reinterpret_cast<ulonglong2*>(ab_out + (size_t)(2 * k + 1) * stride_out * 2 + 4 * y);
            oa[0] = make_ulonglong2(fa0.c0, fa0.c1); oa[1] = make_ulonglong2(fa1.c0, fa1.c1);
            ob[0] = make_ulonglong2(fb0.c0, fb0.c1); ob[1] = make_ulonglong2(fb1.c0, fb1.c1);
            gl::e2acc_mul(q0, fa0, fb0);
            gl::e2acc_mul(q1, fa1, fb1);
            gl::e2acc_mul(q2, E2{gl::sub_canon(fa1.c0, fa0.c0), gl::sub_canon(fa1.c1, fa0.c1)},
                          E2{gl::sub_canon(fb1.c0, fb0.c0), gl::sub_canon(fb1.c1, fb0.c1)});
        }
        // Q(c) = Q(0) + c L + c^2 Q2 with L = Q(1) - Q(0) - Q2
        const E2 Q0 = gl::e2acc_reduce(q0), Q1 = gl::e2acc_reduce(q1), Q2 = gl::e2acc_reduce(q2);
        const E2 t = gl::e2_add(Q1, Q2);                        // Q1 + Q2
        const E2 u = gl::e2_add(t, Q2);                         // Q1 + 2 Q2
        const E2 Qc2 = gl::e2_sub(gl::e2_add(t, t), Q0);        // 2 Q1 + 2 Q2 - Q0
        const E2 Qc3 = gl::e2_sub(gl::e2_sub(gl::e2_add(gl::e2_add(u, u), u), Q0), Q0);  // 3 Q1 + 6 Q2 - 2 Q0
        const ulonglong2* pe = reinterpret_cast<const ulonglong2*>(eq_in + 8 * y);
        const ulonglong2 e0 = pe[0], e1 = pe[1], e2v = pe[2], e3 = pe[3];
        const E2 g0 = gl::e2_canon(gl::e2_fma_pre(rp, E2{gl::sub_canon(e1.x, e0.x), gl::sub_canon(e1.y, e0.y)}, E2{e0.x, e0.y}));
        const E2 g1 = gl::e2_canon(gl::e2_fma_pre(rp, E2{gl::sub_canon(e3.x, e2v.x), gl::sub_canon(e3.y, e2v.y)}, E2{e2v.x, e2v.y}));
        ulonglong2* oe = reinterpret_cast<ulonglong2*>(eq_out + 4 * y);
        oe[0] = make_ulonglong2(g0.c0, g0.c1);
        oe[1] = make_ulonglong2(g1.c0, g1.c1);
        const E2 de = E2{gl::sub_canon(g1.c0, g0.c0), gl::sub_canon(g1.c1, g0.c1)};
        const E2 ve2 = gl::e2_add(g1, de), ve3 = gl::e2_add(ve2, de);
        m[0] = gl::e2_add(m[0], gl::e2_mul_lazy(g0, Q0));
        m[1] = gl::e2_add(m[1], gl::e2_mul_lazy(g1, Q1));
        m[2] = gl::e2_add(m[2], gl::e2_mul_lazy(ve2, Qc2));
        m[3] = gl::e2_add(m[3], gl::e2_mul_lazy(ve3, Qc3));
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
