// Batched degree-3 sumcheck with a shared eq table over Goldilocks:
//   claim   S = sum_k alpha^k sum_x eq(t, x) a_k(x) b_k(x),   k < K instances
//   message m(c) = sum_y eq(c, y) sum_k alpha^k a_k(c, y) b_k(c, y),   c = 0..3
// (the composition of the reference's same-point batched sumcheck,
// zk-torch-4/src/fold/same_point_sumcheck.rs:58-157, with the three-table
// linear prover zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100; low variable
// first).
//
// Every round polynomial factors: the eq table of a round is
// C eq(t_i, x_i) eq(t_rest, y), so with E(y) = eq[2y] + eq[2y + 1] = C eq(t_rest, y)
//   m(c) = lambda(c) T(c),  lambda(c) = (1 - t_i) + c (2 t_i - 1),
//   T(c) = sum_y E(y) Q_y(c),  Q_y(c) = sum_k alpha^k a_k(c, y) b_k(c, y),
// and T is quadratic: the kernels return T(0), T(1) and its leading coefficient
// T2 (three extension elements); the host forms T(2) = 2 T(1) + 2 T2 - T(0),
// T(3) = 3 T(1) + 6 T2 - 2 T(0) and multiplies by lambda. The results are the same
// field elements as the direct sums over eq(c, y) a(c, y) b(c, y).
//
// Round 0 works on the caller's base-field tables and is independent of alpha:
// one pass produces T_k(0), T_k(1), T2_k per instance; the claims are
// s_k = m_k(0) + m_k(1) and the round-0 message is sum_k alpha^k m_k(c), combined
// on the host. The first fold lifts the tables to the extension and multiplies
// a_k by alpha^k once; every later pass folds the 2K + 1 tables and accumulates
// the next message in the same sweep.
//
// Arithmetic: all multiplications feed exact 160-bit sums that are reduced once
// (gl::Acc); Q_y(0), Q_y(1) and the leading coefficient of Q_y are three lazily
// accumulated extension products per instance, and E Q is formed once per pair,
// not once per instance.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace bt {

constexpr int MAX_K = 64;
constexpr int NC = 3;  // T(0), T(1) and the leading coefficient of T

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

// ---- round 0: per-instance T_k(0), T_k(1), T2_k from the base-field tables ---------------
// Lane l of a warp owns instance k = kbase + (l & (Kp - 1)) for the whole
// launch, so its six exact sums are reduced only once at the end; the 32 / Kp
// lane groups of a warp take consecutive pairs of output pairs y, and the
// weights E(y) of the warp's current pairs are shared through shared memory.
// The loads of step i + 1 are issued before the arithmetic of step i.
// eq: canonical extension table; a0p, b0p: [K][stride] (any representatives);
// half = number of pairs; partial: [gridDim.x][K][6] canonical words. Dynamic
// shared memory: warps * 2 * (64 / Kp) * 2 words.
static __global__ void __launch_bounds__(256)
instance_messages_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ a0p,
                         const uint64_t* __restrict__ b0p, int K, int Kp, size_t stride, size_t half,
                         uint64_t* __restrict__ partial) {
    extern __shared__ __align__(16) uint64_t dyn[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int G = 32 / Kp, g = lane / Kp;
    const int k = blockIdx.y * 32 + (lane & (Kp - 1));
    const bool live_k = k < K;
    const int ys_per_iter = 2 * G;
    const int nev = ys_per_iter * 2;  // weight words per step; one per lane when Kp >= 4
    uint64_t* ev = dyn + (size_t)warp * nev * 2;  // two buffers of [y][component]
    const uint64_t* pa = a0p + (size_t)(live_k ? k : 0) * stride;
    const uint64_t* pb = b0p + (size_t)(live_k ? k : 0) * stride;
    gl::Acc A[NC][2];
#pragma unroll
    for (int c = 0; c < NC; c++) A[c][0] = A[c][1] = gl::acc_zero();
    const size_t warps_total = (size_t)gridDim.x * nwarp, wg = (size_t)blockIdx.x * nwarp + warp;
    const size_t ystep = warps_total * ys_per_iter;

    auto weight_fill = [&](size_t ybase, uint64_t* dst) {  // unpipelined form, any Kp
        for (int j = lane; j < nev; j += 32) {
            const size_t y = ybase + (j >> 1);
            dst[j] = y < half ? gl::add_c(eq[4 * y + (j & 1)], eq[4 * y + 2 + (j & 1)]) : 0;
        }
    };
    const bool one_per_lane = nev <= 32;
    ulonglong2 ca[2], cb[2], na[2], nb[2];
    uint64_t ne0 = 0, ne1 = 0;
    auto load_pairs = [&](size_t ybase, ulonglong2 (&ta)[2], ulonglong2 (&tb)[2]) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t y = ybase + 2 * g + h;
            ta[h] = tb[h] = make_ulonglong2(0, 0);
            if (y < half && live_k) {
                ta[h] = *reinterpret_cast<const ulonglong2*>(pa + 2 * y);
                tb[h] = *reinterpret_cast<const ulonglong2*>(pb + 2 * y);
            }
        }
    };
    size_t ybase = wg * ys_per_iter;
    int buf = 0;
    if (ybase < half) {
        weight_fill(ybase, ev);
        load_pairs(ybase, ca, cb);
    }
    __syncwarp();
    for (; ybase < half; ybase += ystep, buf ^= 1) {
        const size_t ynext = ybase + ystep;
        const bool more = ynext < half;
        if (more) {
            load_pairs(ynext, na, nb);
            if (one_per_lane && lane < nev) {
                const size_t y = ynext + (lane >> 1);
                if (y < half) {
                    ne0 = eq[4 * y + (lane & 1)];
                    ne1 = eq[4 * y + 2 + (lane & 1)];
                }
            }
        }
        const uint64_t* evc = ev + buf * nev;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t y = ybase + 2 * g + h;
            if (y < half && live_k) {
                const uint64_t a0 = gl::canon(ca[h].x), a1 = gl::canon(ca[h].y), b0 = gl::canon(cb[h].x), b1 = gl::canon(cb[h].y);
                const ulonglong2 E = *reinterpret_cast<const ulonglong2*>(evc + (2 * g + h) * 2);
                const uint64_t p0 = gl::mul(a0, b0), p1 = gl::mul(a1, b1);
                const uint64_t p2 = gl::mul(gl::sub_canon(a1, a0), gl::sub_canon(b1, b0));
                gl::acc_mul(A[0][0], E.x, p0); gl::acc_mul(A[0][1], E.y, p0);
                gl::acc_mul(A[1][0], E.x, p1); gl::acc_mul(A[1][1], E.y, p1);
                gl::acc_mul(A[2][0], E.x, p2); gl::acc_mul(A[2][1], E.y, p2);
            }
        }
        if (more) {
            uint64_t* evn = ev + (buf ^ 1) * nev;
            if (one_per_lane) {
                if (lane < nev) evn[lane] = (ynext + (lane >> 1)) < half ? gl::add_c(ne0, ne1) : 0;
            } else {
                weight_fill(ynext, evn);
            }
#pragma unroll
            for (int h = 0; h < 2; h++) { ca[h] = na[h]; cb[h] = nb[h]; }
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
        const E2 Q0 = gl::e2acc_reduce(q0), Q1 = gl::e2acc_reduce(q1), Q2 = gl::e2acc_reduce(q2);
        const ulonglong2* pe = reinterpret_cast<const ulonglong2*>(eq_in + 8 * y);
        const ulonglong2 e0 = pe[0], e1 = pe[1], e2v = pe[2], e3 = pe[3];
        const E2 g0 = gl::e2_canon(gl::e2_fma_pre(rp, E2{gl::sub_canon(e1.x, e0.x), gl::sub_canon(e1.y, e0.y)}, E2{e0.x, e0.y}));
        const E2 g1 = gl::e2_canon(gl::e2_fma_pre(rp, E2{gl::sub_canon(e3.x, e2v.x), gl::sub_canon(e3.y, e2v.y)}, E2{e2v.x, e2v.y}));
        ulonglong2* oe = reinterpret_cast<ulonglong2*>(eq_out + 4 * y);
        oe[0] = make_ulonglong2(g0.c0, g0.c1);
        oe[1] = make_ulonglong2(g1.c0, g1.c1);
        const E2 Ew = E2{gl::add_c(g0.c0, g1.c0), gl::add_c(g0.c1, g1.c1)};
        m[0] = gl::e2_add(m[0], gl::e2_mul_lazy(Ew, Q0));
        m[1] = gl::e2_add(m[1], gl::e2_mul_lazy(Ew, Q1));
        m[2] = gl::e2_add(m[2], gl::e2_mul_lazy(Ew, Q2));
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
