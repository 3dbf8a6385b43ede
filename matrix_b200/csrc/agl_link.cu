// C-ABI: the packed link sumcheck over the almost-Goldilocks extension (reference declarations
// almost-goldilocks-cuda-rs/src/ffi.rs:511-593, definitions almost-goldilocks-cuda-rs/cuda/wrapper.cu:1213-1440,
// kernels cuda_almost_goldilocks/link_sumcheck.cuh:59-787; CPU definition zk-torch-4/src/pcs/link.rs:284-357).
//
// Per round, with R(u) = u^3 - u and the HIGH index bit bound first (pairs (idx, half + idx)):
//     S(k) = sum_e tag_e sum_idx eq[idx] R(w_e(k)[idx])       k = 0..3
//     E(k) = sum_e       sum_idx omega_e(k)[idx] w_e(k)[idx]   k = 0..2
// out = [S(0..3), E(0..2)]: seven extension elements, canonical. In the first round S(0), S(1) are zero
// by definition (committed coefficients lie in {-1, 0, 1}).
//
// One kernel template covers every form: witness from a table or from packed bits, index set dense or a
// support list, weights from a table or evaluated on demand for the interleaved layout.
//
// Bit-packed witnesses need no multiplication at all: with (lo, hi) in {0, 1}^2 the interpolants are small
// integers, R(w(2)) = 6 and R(w(3)) = 24 on (0, 1), R(w(3)) = -6 on (1, 0), zero otherwise, and the weight
// products are signed selections, so the round is additions of eq and omega values and is bound by the
// reads of omega; the small factors are applied once per block.
#include "agl_field.cuh"
#include "common.cuh"
#include "prof.cuh"

using namespace mb;

namespace {

using agl::E2;
constexpr int SLOTS = 7, NORM = 4, BLOCK = 256;

__device__ __forceinline__ E2 ld(const uint64_t* p, uint64_t i) { return agl::e2_load(p + 2 * i); }
__device__ __forceinline__ void st(uint64_t* p, uint64_t i, E2 v) { agl::e2_store(p + 2 * i, agl::e2_canon(v)); }
__device__ __forceinline__ E2 zero() { return E2{0, 0}; }
__device__ __forceinline__ bool is_zero(E2 v) { return (agl::canon(v.c0) | agl::canon(v.c1)) == 0; }
__device__ __forceinline__ unsigned bit_at(const uint64_t* bits, uint64_t i) { return (unsigned)((bits[i >> 6] >> (i & 63)) & 1ULL); }
__device__ __forceinline__ E2 range_poly(E2 u) { return agl::e2_sub(agl::e2_mul_lazy(agl::e2_mul_lazy(u, u), u), u); }
__device__ __forceinline__ E2 fold2(E2 lo, E2 hi, agl::E2Pre r) { return agl::e2_fma_pre(r, agl::e2_sub(hi, lo), lo); }
__device__ __forceinline__ E2 mul_small(E2 a, uint32_t k) { return E2{agl::mul_small(a.c0, k), agl::mul_small(a.c1, k)}; }

// eq(l, pt[0..m)) with pt most significant variable first.
__device__ __forceinline__ E2 eq_pointwise(const uint64_t* pt, uint64_t l, int m) {
    E2 acc{1, 0};
    for (int k = 0; k < m; k++) {
        const E2 r = ld(pt, k);
        acc = agl::e2_mul_lazy(acc, ((l >> (m - 1 - k)) & 1ULL) ? r : agl::e2_sub(E2{1, 0}, r));
    }
    return acc;
}

// Block sum of the seven slots (shuffles inside a warp, one shared-memory step across the eight warps), tag on the
// norm half, one partial per block.
__device__ __forceinline__ void block_sum_store(const E2 acc[SLOTS], const uint64_t* tags, uint64_t* partial, uint64_t e, uint64_t chunk,
                                                uint64_t nchunk) {
    const int tid = threadIdx.x;
    __shared__ uint64_t sh[BLOCK / 32][SLOTS][2];
#pragma unroll
    for (int k = 0; k < SLOTS; k++) {
        E2 v = acc[k];
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const E2 o{__shfl_down_sync(0xffffffffu, v.c0, off), __shfl_down_sync(0xffffffffu, v.c1, off)};
            v = agl::e2_add(v, o);
        }
        if ((tid & 31) == 0) {
            sh[tid >> 5][k][0] = v.c0;
            sh[tid >> 5][k][1] = v.c1;
        }
    }
    __syncthreads();
    if (tid < SLOTS) {
        E2 v = zero();
        for (int wp = 0; wp < BLOCK / 32; wp++) v = agl::e2_add(v, E2{sh[wp][tid][0], sh[wp][tid][1]});
        if (tid < NORM) v = agl::e2_mul_lazy(ld(tags, e), v);
        st(partial, (e * nchunk + chunk) * SLOTS + tid, v);
    }
}

// The bit-packed terms of one pair: s01 / s10 collect eq over (0,1) / (1,0) pairs, acc[4..6] the weight sums.
__device__ __forceinline__ void bit_pair_terms(E2& s01, E2& s10, E2 acc[SLOTS], unsigned blo, unsigned bhi, E2 o_lo, E2 o_hi, E2 eqs) {
    if (blo && !bhi) s10 = agl::e2_add(s10, eqs);
    if (bhi && !blo) s01 = agl::e2_add(s01, eqs);
    if (blo) acc[4] = agl::e2_add(acc[4], o_lo);
    if (bhi) acc[5] = agl::e2_add(acc[5], o_hi);
    const E2 o2 = agl::e2_sub(agl::e2_add(o_hi, o_hi), o_lo);   // omega(2); w(2) = 2 hi - lo in {-1, 1, 2}
    if (blo && !bhi) acc[6] = agl::e2_sub(acc[6], o2);
    else if (!blo) acc[6] = agl::e2_add(acc[6], agl::e2_add(o2, o2));
    else acc[6] = agl::e2_add(acc[6], o2);
}

// Position of the n-th (1-based) set bit of a 64-bit word.
__device__ __forceinline__ unsigned nth_set_bit(uint64_t m, unsigned n) {
    const unsigned lo = (unsigned)m, c = __popc(lo);
    return n <= c ? __fns(lo, 0, (int)n) : 32u + __fns((unsigned)(m >> 32), 0, (int)(n - c));
}

// Exact 96-bit sums of 64-bit words (no reduction per addition): up to 2^32 terms.
struct Raw {
    uint64_t lo;
    uint32_t hi;
};
struct RawE2 {
    Raw c0, c1;
};
__device__ __forceinline__ void raw_add(Raw& a, uint64_t x) {
    asm("add.cc.u64 %0, %0, %2;\n\taddc.u32 %1, %1, 0;" : "+l"(a.lo), "+r"(a.hi) : "l"(x));
}
__device__ __forceinline__ void raw_add(RawE2& a, E2 x) {
    raw_add(a.c0, x.c0);
    raw_add(a.c1, x.c1);
}
__device__ __forceinline__ E2 raw_reduce(const RawE2& a) {
    return E2{agl::reduce128(a.c0.lo, (uint64_t)a.c0.hi), agl::reduce128(a.c1.lo, (uint64_t)a.c1.hi)};
}

struct RoundArgs {
    const uint64_t* bits;      // witness bits, rows of bits_stride_words (BITS)
    const uint64_t* w;         // witness table, rows of w_stride (!BITS)
    const uint64_t* omega;     // weight table, rows of omega_stride (!ONDEMAND)
    const uint64_t* pts;       // [n_commit][blocks][leaf_arity] (ONDEMAND)
    const uint64_t* scale;     // [n_commit][blocks] (ONDEMAND)
    const uint64_t* eq;        // by idx (dense) or by list position (LISTED)
    const uint64_t* tags;
    const uint32_t* list;
    const uint64_t* list_off;
    const uint64_t* list_len;
    uint64_t w_stride, bits_stride_words, omega_stride, half;
    uint32_t block_mask;
    int block_bits, leaf_arity, round, first_round;
    uint64_t* partial;         // [n_commit][chunks][7]
};

// grid (chunks, n_commit), 256 threads.
template <bool BITS, bool LISTED, bool ONDEMAND>
__global__ void __launch_bounds__(BLOCK) link_round_kernel(RoundArgs a) {
    const uint64_t e = blockIdx.y, chunk = blockIdx.x, nchunk = gridDim.x;
    const int tid = threadIdx.x;
    const uint64_t* be = BITS ? a.bits + e * a.bits_stride_words : nullptr;
    const uint64_t* we = BITS ? nullptr : a.w + 2 * e * a.w_stride;
    const uint64_t* oe = ONDEMAND ? nullptr : a.omega + 2 * e * a.omega_stride;
    const uint64_t loff = LISTED ? a.list_off[e] : 0;
    const uint64_t n = LISTED ? a.list_len[e] : a.half;
    const uint64_t blocks = (uint64_t)a.block_mask + 1;
    const int m = a.leaf_arity - a.round;

    // BITS: acc[0] = sum of eq over (0,1) pairs, acc[1] = over (1,0) pairs, acc[4..6] as defined.
    E2 acc[SLOTS];
#pragma unroll
    for (int k = 0; k < SLOTS; k++) acc[k] = zero();

    for (uint64_t t = chunk * BLOCK + tid; t < n; t += nchunk * BLOCK) {
        const uint64_t idx = LISTED ? (uint64_t)a.list[loff + t] : t;
        unsigned blo = 0, bhi = 0;
        E2 w_lo = zero(), w_hi = zero();
        if (BITS) {
            blo = bit_at(be, idx);
            bhi = bit_at(be, a.half + idx);
            if (!(blo | bhi)) continue;
        } else {
            w_lo = ld(we, idx);
            w_hi = ld(we, a.half + idx);
            if (!LISTED && is_zero(w_lo) && is_zero(w_hi)) continue;
        }
        E2 o_lo, o_hi;
        if (ONDEMAND) {
            const uint64_t b = idx & a.block_mask;
            const uint64_t* ptb = a.pts + 2 * ((e * blocks + b) * (uint64_t)a.leaf_arity + (uint64_t)a.round);
            const E2 sc = ld(a.scale, e * blocks + b);
            o_lo = agl::e2_mul_lazy(sc, eq_pointwise(ptb, idx >> a.block_bits, m));
            o_hi = agl::e2_mul_lazy(sc, eq_pointwise(ptb, (a.half + idx) >> a.block_bits, m));
        } else {
            o_lo = ld(oe, idx);
            o_hi = ld(oe, a.half + idx);
        }
        const E2 eqs = ld(a.eq, LISTED ? loff + t : idx);
        if (BITS) {
            bit_pair_terms(acc[0], acc[1], acc, blo, bhi, o_lo, o_hi, eqs);
        } else {
            const E2 w_d = agl::e2_sub(w_hi, w_lo), o_d = agl::e2_sub(o_hi, o_lo);
            const E2 w1 = agl::e2_add(w_lo, w_d), w2 = agl::e2_add(w1, w_d), w3 = agl::e2_add(w2, w_d);
            if (!a.first_round) {
                acc[0] = agl::e2_add(acc[0], agl::e2_mul_lazy(eqs, range_poly(w_lo)));
                acc[1] = agl::e2_add(acc[1], agl::e2_mul_lazy(eqs, range_poly(w1)));
            }
            acc[2] = agl::e2_add(acc[2], agl::e2_mul_lazy(eqs, range_poly(w2)));
            acc[3] = agl::e2_add(acc[3], agl::e2_mul_lazy(eqs, range_poly(w3)));
            const E2 o1 = agl::e2_add(o_lo, o_d), o2 = agl::e2_add(o1, o_d);
            acc[4] = agl::e2_add(acc[4], agl::e2_mul_lazy(o_lo, w_lo));
            acc[5] = agl::e2_add(acc[5], agl::e2_mul_lazy(o1, w1));
            acc[6] = agl::e2_add(acc[6], agl::e2_mul_lazy(o2, w2));
        }
    }
    if (BITS) {
        const E2 s01 = acc[0], s10 = acc[1];
        acc[0] = zero();
        acc[1] = zero();
        acc[2] = mul_small(s01, 6);
        acc[3] = agl::e2_sub(mul_small(s01, 24), mul_small(s10, 6));
    }

    block_sum_store(acc, a.tags, a.partial, e, chunk, nchunk);
}

// Round 0 off bits, dense index set, half a multiple of 64. A warp takes 32 word pairs (2048 index pairs) at a
// time, counts the live pairs (lo | hi), and hands them out one per lane in compact order, so the work and the
// weight reads follow the number of live pairs at any density, with 32 independent pairs in flight per warp;
// batches that are mostly live are swept a word at a time instead (one lane per bit position).
__global__ void __launch_bounds__(BLOCK) link_round0_words_kernel(RoundArgs a) {
    const uint64_t e = blockIdx.y, chunk = blockIdx.x, nchunk = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31;
    const uint64_t* be = a.bits + e * a.bits_stride_words;
    const uint64_t* oe = a.omega + 2 * e * a.omega_stride;
    const uint64_t words = a.half >> 6;
    const uint64_t warp = chunk * (BLOCK / 32) + (tid >> 5), nwarps = nchunk * (BLOCK / 32);
    // raw sums by pair type (lo, hi) = (1,0), (0,1), (1,1): weights at idx (L) and at half + idx (H), eq for the mixed types
    RawE2 L10{}, L01{}, L11{}, H10{}, H01{}, H11{}, S10{}, S01{};
    for (uint64_t wb = warp * 32; wb < words; wb += nwarps * 32) {
        const uint64_t wi = wb + lane;
        const uint64_t lo = wi < words ? be[wi] : 0, hi = wi < words ? be[words + wi] : 0;
        const uint64_t act = lo | hi;
        const unsigned cnt = __popcll(act);
        unsigned inc = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned u = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += u;
        }
        const unsigned pre = inc - cnt, total = __shfl_sync(0xffffffffu, inc, 31);
        auto consume = [&](uint64_t idx, unsigned blo, unsigned bhi) {
            const E2 o_lo = ld(oe, idx), o_hi = ld(oe, a.half + idx);
            if (blo & bhi) {
                raw_add(L11, o_lo);
                raw_add(H11, o_hi);
            } else {
                const E2 eqs = ld(a.eq, idx);
                if (blo) {
                    raw_add(L10, o_lo);
                    raw_add(H10, o_hi);
                    raw_add(S10, eqs);
                } else {
                    raw_add(L01, o_lo);
                    raw_add(H01, o_hi);
                    raw_add(S01, eqs);
                }
            }
        };
        if (total >= 768) {
            // mostly live: a lane per bit position, 32 consecutive pairs per step (coalesced weight reads)
            for (int j = 0; j < 32; j++) {
                const uint64_t wlo = __shfl_sync(0xffffffffu, lo, j), whi = __shfl_sync(0xffffffffu, hi, j);
                if (!(wlo | whi)) continue;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const unsigned bit = lane + 32 * h;
                    const unsigned blo = (unsigned)(wlo >> bit) & 1u, bhi = (unsigned)(whi >> bit) & 1u;
                    if (blo | bhi) consume(((wb + j) << 6) + bit, blo, bhi);
                }
            }
            continue;
        }
        for (unsigned k0 = 0; k0 < total; k0 += 32) {
            const bool live = k0 + lane < total;
            const unsigned r = live ? k0 + lane : total - 1;
            int j = 0;   // the lane whose word holds live pair r: last j with pre_j <= r
#pragma unroll
            for (int step = 16; step; step >>= 1) {
                const unsigned pc = __shfl_sync(0xffffffffu, pre, (j + step) & 31);
                if (j + step < 32 && pc <= r) j += step;
            }
            const uint64_t wlo = __shfl_sync(0xffffffffu, lo, j), whi = __shfl_sync(0xffffffffu, hi, j);
            const unsigned pj = __shfl_sync(0xffffffffu, pre, j);
            if (live) {
                const unsigned bit = nth_set_bit(wlo | whi, r - pj + 1);
                consume(((wb + j) << 6) + bit, (unsigned)(wlo >> bit) & 1u, (unsigned)(whi >> bit) & 1u);
            }
        }
    }
    // E(0) = sum lo omega_lo, E(1) = sum hi omega_hi, E(2) = sum (2 hi - lo)(2 omega_hi - omega_lo); S(2) = 6 s01, S(3) = 24 s01 - 6 s10
    const E2 l10 = raw_reduce(L10), l01 = raw_reduce(L01), l11 = raw_reduce(L11);
    const E2 h10 = raw_reduce(H10), h01 = raw_reduce(H01), h11 = raw_reduce(H11);
    const E2 s10 = raw_reduce(S10), s01 = raw_reduce(S01);
    E2 acc[SLOTS];
    acc[0] = zero();
    acc[1] = zero();
    acc[2] = mul_small(s01, 6);
    acc[3] = agl::e2_sub(mul_small(s01, 24), mul_small(s10, 6));
    acc[4] = agl::e2_add(l10, l11);
    acc[5] = agl::e2_add(h01, h11);
    const E2 t11 = agl::e2_sub(agl::e2_add(h11, h11), l11), t01 = agl::e2_sub(agl::e2_add(h01, h01), l01),
             t10 = agl::e2_sub(agl::e2_add(h10, h10), l10);
    acc[6] = agl::e2_sub(agl::e2_add(t11, agl::e2_add(t01, t01)), t10);
    block_sum_store(acc, a.tags, a.partial, e, chunk, nchunk);
}

// Table witness, dense index set: a warp sweeps 32 pairs at a time (coalesced reads of both halves), queues the
// indices of the live ones in shared memory and runs the arithmetic only on full groups of 32 live pairs, so a
// sparse table costs its live pairs plus one pass over the witness, whatever the spacing of the live entries
// (skipping inside the sweep alone would be bounded by the warp width). half <= 2^32.
__global__ void __launch_bounds__(BLOCK) link_round_dense_kernel(RoundArgs a) {
    __shared__ uint32_t queue[BLOCK / 32][64];
    const uint64_t e = blockIdx.y, chunk = blockIdx.x, nchunk = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const uint64_t* we = a.w + 2 * e * a.w_stride;
    const uint64_t* oe = a.omega + 2 * e * a.omega_stride;
    E2 acc[SLOTS];
#pragma unroll
    for (int k = 0; k < SLOTS; k++) acc[k] = zero();
    auto process = [&](uint64_t idx) {
        const E2 w_lo = ld(we, idx), w_hi = ld(we, a.half + idx);
        const E2 o_lo = ld(oe, idx), o_hi = ld(oe, a.half + idx), eqs = ld(a.eq, idx);
        const E2 w_d = agl::e2_sub(w_hi, w_lo), o_d = agl::e2_sub(o_hi, o_lo);
        const E2 w1 = agl::e2_add(w_lo, w_d), w2 = agl::e2_add(w1, w_d), w3 = agl::e2_add(w2, w_d);
        if (!a.first_round) {
            acc[0] = agl::e2_add(acc[0], agl::e2_mul_lazy(eqs, range_poly(w_lo)));
            acc[1] = agl::e2_add(acc[1], agl::e2_mul_lazy(eqs, range_poly(w1)));
        }
        acc[2] = agl::e2_add(acc[2], agl::e2_mul_lazy(eqs, range_poly(w2)));
        acc[3] = agl::e2_add(acc[3], agl::e2_mul_lazy(eqs, range_poly(w3)));
        const E2 o1 = agl::e2_add(o_lo, o_d), o2 = agl::e2_add(o1, o_d);
        acc[4] = agl::e2_add(acc[4], agl::e2_mul_lazy(o_lo, w_lo));
        acc[5] = agl::e2_add(acc[5], agl::e2_mul_lazy(o1, w1));
        acc[6] = agl::e2_add(acc[6], agl::e2_mul_lazy(o2, w2));
    };
    unsigned qn = 0;   // queued indices of this warp, the same value in every lane
    const uint64_t warp = chunk * (BLOCK / 32) + wp, nwarps = nchunk * (BLOCK / 32);
    uint64_t base = warp * 32;
    for (;;) {
        while (qn < 32 && base < a.half) {   // sweep until a full group is queued or the range ends
            const uint64_t idx = base + lane;
            bool live = false;
            if (idx < a.half) live = !(is_zero(ld(we, idx)) && is_zero(ld(we, a.half + idx)));
            const unsigned mask = __ballot_sync(0xffffffffu, live);
            if (live) queue[wp][qn + __popc(mask & ((1u << lane) - 1u))] = (uint32_t)idx;
            qn += __popc(mask);
            base += nwarps * 32;
        }
        if (qn == 0) break;
        __syncwarp();
        const unsigned take = qn < 32 ? qn : 32;
        qn -= take;
        const uint32_t mine = queue[wp][qn + (lane < take ? lane : 0)];
        __syncwarp();
        if (lane < take) process(mine);
    }
    block_sum_store(acc, a.tags, a.partial, e, chunk, nchunk);
}

// out[k] = sum of partial[b][k]; one block per slot.
__global__ void __launch_bounds__(BLOCK) link_reduce_kernel(const uint64_t* __restrict__ partial, uint64_t n_blocks, uint64_t* __restrict__ out) {
    const int k = blockIdx.x, tid = threadIdx.x;
    E2 v = zero();
    for (uint64_t b = tid; b < n_blocks; b += BLOCK) v = agl::e2_add(v, ld(partial, b * SLOTS + k));
    __shared__ uint64_t sh[BLOCK / 32][2];
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        const E2 o{__shfl_down_sync(0xffffffffu, v.c0, off), __shfl_down_sync(0xffffffffu, v.c1, off)};
        v = agl::e2_add(v, o);
    }
    if ((tid & 31) == 0) {
        sh[tid >> 5][0] = v.c0;
        sh[tid >> 5][1] = v.c1;
    }
    __syncthreads();
    if (tid == 0) {
        E2 s = zero();
        for (int wp = 0; wp < BLOCK / 32; wp++) s = agl::e2_add(s, E2{sh[wp][0], sh[wp][1]});
        st(out, k, s);
    }
}

// In-place fold of rows of two tables: t[i] = lo + r (hi - lo). `tb` may be null.
__global__ void link_fold_kernel(uint64_t* __restrict__ ta, uint64_t* __restrict__ tb, uint64_t stride_a, uint64_t stride_b, uint64_t half,
                                 uint64_t n_commit, E2 r) {
    const agl::E2Pre rp = agl::e2_pre(r);
    const uint64_t total = half * n_commit;
    for (uint64_t t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t e = t / half, i = t - e * half;
        uint64_t* pa = ta + 2 * e * stride_a;
        st(pa, i, fold2(ld(pa, i), ld(pa, half + i), rp));
        if (tb) {
            uint64_t* pb = tb + 2 * e * stride_b;
            st(pb, i, fold2(ld(pb, i), ld(pb, half + i), rp));
        }
    }
}

// Same over support lists; grid (x, n_commit).
__global__ void link_fold_sparse_kernel(uint64_t* __restrict__ w, uint64_t* __restrict__ omega, const uint32_t* __restrict__ list,
                                        const uint64_t* __restrict__ list_off, const uint64_t* __restrict__ list_len, uint64_t stride,
                                        uint64_t half, E2 r) {
    const agl::E2Pre rp = agl::e2_pre(r);
    const uint64_t e = blockIdx.y, n = list_len[e];
    const uint32_t* le = list + list_off[e];
    uint64_t *pw = w + 2 * e * stride, *po = omega + 2 * e * stride;
    for (uint64_t t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; t < n; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t i = le[t];
        st(pw, i, fold2(ld(pw, i), ld(pw, half + i), rp));
        st(po, i, fold2(ld(po, i), ld(po, half + i), rp));
    }
}

// Witness fold out of place, from bits (a selection among 0, 1, r, 1 - r) or from a table; omega, when given, in place.
template <bool BITS>
__global__ void link_fold_w_kernel(const uint64_t* __restrict__ bits, const uint64_t* __restrict__ w_in, uint64_t* __restrict__ w_out,
                                   uint64_t* __restrict__ omega, uint64_t in_stride, uint64_t bits_stride_words, uint64_t out_stride,
                                   uint64_t omega_stride, uint64_t half, uint64_t n_commit, E2 r) {
    const agl::E2Pre rp = agl::e2_pre(r);
    const E2 rc = agl::e2_canon(r), omr = agl::e2_canon(agl::e2_sub(E2{1, 0}, r));
    const uint64_t total = half * n_commit;
    for (uint64_t t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t e = t / half, i = t - e * half;
        E2 v;
        if (BITS) {
            const uint64_t* be = bits + e * bits_stride_words;
            const unsigned lo = bit_at(be, i), hi = bit_at(be, half + i);
            v = lo ? (hi ? E2{1, 0} : omr) : (hi ? rc : zero());
        } else {
            const uint64_t* pi = w_in + 2 * e * in_stride;
            v = fold2(ld(pi, i), ld(pi, half + i), rp);
        }
        st(w_out + 2 * e * out_stride, i, v);
        if (omega) {
            uint64_t* po = omega + 2 * e * omega_stride;
            st(po, i, fold2(ld(po, i), ld(po, half + i), rp));
        }
    }
}

// table[i], table[span + i] = v (1 - r), v r for i < span; grid.y selects (base, r) pairs when given.
__global__ void link_expand_kernel(uint64_t* __restrict__ table, const uint64_t* __restrict__ bases, const uint64_t* __restrict__ rs,
                                   uint64_t span, E2 r_one) {
    const uint64_t q = blockIdx.y;
    uint64_t* tb = bases ? table + 2 * bases[q] : table;
    const E2 r = rs ? ld(rs, q) : r_one;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < span; i += (uint64_t)gridDim.x * blockDim.x) {
        const E2 v = ld(tb, i), vr = agl::e2_mul_lazy(v, r);
        st(tb, i, agl::e2_sub(v, vr));
        st(tb, span + i, vr);
    }
}

// One thread per output pair of elements: 64 elements per input word.
__global__ void link_expand_bits_kernel(const uint64_t* __restrict__ bits, uint64_t* __restrict__ out, uint64_t n_elems) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n_elems; i += (uint64_t)gridDim.x * blockDim.x)
        agl::e2_store(out + 2 * i, E2{(uint64_t)bit_at(bits, i), 0});
}

__global__ void link_eq_gather_kernel(const uint64_t* __restrict__ alpha, uint64_t n_vars, const uint32_t* __restrict__ list,
                                      uint64_t* __restrict__ out, uint64_t total) {
    for (uint64_t t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x)
        st(out, t, eq_pointwise(alpha, list[t], (int)n_vars));
}

template <bool BITS, bool LISTED, bool ONDEMAND>
int run_round(const RoundArgs& a, uint64_t n_commit, uint64_t chunks, uint64_t* d_out) {
    if (!a.eq || !a.tags || !a.partial || !d_out || chunks == 0 || chunks > 0x7fffffffULL || n_commit > 65535) return MB_ERR_ARG;
    if (n_commit == 0) {
        MB_CUDA(cudaMemsetAsync(d_out, 0, SLOTS * 16, MB_STREAM));
        return finish_sync();
    }
    {
        MB_KERNEL("link_round");
        dim3 grid((unsigned)chunks, (unsigned)n_commit);
        link_round_kernel<BITS, LISTED, ONDEMAND><<<grid, BLOCK, 0, MB_STREAM>>>(a);
    }
    {
        MB_KERNEL("link_reduce");
        link_reduce_kernel<<<SLOTS, BLOCK, 0, MB_STREAM>>>(a.partial, n_commit * chunks, d_out);
    }
    return finish_sync();
}

RoundArgs base_args(const uint64_t* eq, const uint64_t* tags, uint64_t half, int first_round, uint64_t* partial) {
    RoundArgs a{};
    a.eq = eq;
    a.tags = tags;
    a.half = half;
    a.first_round = first_round;
    a.partial = partial;
    return a;
}

}  // namespace

extern "C" {

int link_round_message_ffi(const uint64_t* d_w, const uint64_t* d_omega, const uint64_t* d_eq_suffix, const uint64_t* d_tags, uint64_t stride,
                           uint64_t omega_stride, uint64_t half, uint64_t n_commit, int first_round, uint64_t* d_partial, uint64_t chunks,
                           uint64_t* d_out) {
    if (!d_w || !d_omega) return MB_ERR_ARG;
    RoundArgs a = base_args(d_eq_suffix, d_tags, half, first_round, d_partial);
    a.w = d_w;
    a.omega = d_omega;
    a.w_stride = stride;
    a.omega_stride = omega_stride;
    if (half > 0xffffffffULL || n_commit == 0) return run_round<false, false, false>(a, n_commit, chunks, d_out);
    if (!a.eq || !a.tags || !a.partial || !d_out || chunks == 0 || chunks > 0x7fffffffULL || n_commit > 65535) return MB_ERR_ARG;
    {
        MB_KERNEL("link_round_dense");
        link_round_dense_kernel<<<dim3((unsigned)chunks, (unsigned)n_commit), BLOCK, 0, MB_STREAM>>>(a);
    }
    {
        MB_KERNEL("link_reduce");
        link_reduce_kernel<<<SLOTS, BLOCK, 0, MB_STREAM>>>(a.partial, n_commit * chunks, d_out);
    }
    return finish_sync();
}

int link_round_message_sparse_ffi(const uint64_t* d_w, const uint64_t* d_omega, const uint64_t* d_eq_suffix, const uint64_t* d_tags,
                                  const uint32_t* d_list, const uint64_t* d_list_off, const uint64_t* d_list_len, uint64_t stride,
                                  uint64_t omega_stride, uint64_t half, uint64_t n_commit, int first_round, uint64_t* d_partial,
                                  uint64_t chunks, uint64_t* d_out) {
    if (!d_w || !d_omega || !d_list || !d_list_off || !d_list_len) return MB_ERR_ARG;
    RoundArgs a = base_args(d_eq_suffix, d_tags, half, first_round, d_partial);
    a.w = d_w;
    a.omega = d_omega;
    a.w_stride = stride;
    a.omega_stride = omega_stride;
    a.list = d_list;
    a.list_off = d_list_off;
    a.list_len = d_list_len;
    return run_round<false, true, false>(a, n_commit, chunks, d_out);
}

int link_round0_bits_ffi(const uint64_t* d_bits, const uint64_t* d_omega, const uint64_t* d_eq, const uint64_t* d_tags, uint64_t stride,
                         uint64_t half, uint64_t n_commit, uint64_t* d_partial, uint64_t chunks, uint64_t* d_out) {
    if (!d_bits || !d_omega || (stride & 63)) return MB_ERR_ARG;
    RoundArgs a = base_args(d_eq, d_tags, half, 1, d_partial);
    a.bits = d_bits;
    a.omega = d_omega;
    a.bits_stride_words = stride >> 6;
    a.omega_stride = stride;
    if ((half & 63) || n_commit == 0) return run_round<true, false, false>(a, n_commit, chunks, d_out);
    if (!a.eq || !a.tags || !a.partial || !d_out || chunks == 0 || chunks > 0x7fffffffULL || n_commit > 65535) return MB_ERR_ARG;
    {
        MB_KERNEL("link_round0_words");
        link_round0_words_kernel<<<dim3((unsigned)chunks, (unsigned)n_commit), BLOCK, 0, MB_STREAM>>>(a);
    }
    {
        MB_KERNEL("link_reduce");
        link_reduce_kernel<<<SLOTS, BLOCK, 0, MB_STREAM>>>(a.partial, n_commit * chunks, d_out);
    }
    return finish_sync();
}

int link_round0_bits_sparse_ffi(const uint64_t* d_bits, const uint64_t* d_omega, const uint64_t* d_eq, const uint64_t* d_tags,
                                const uint32_t* d_list, const uint64_t* d_list_off, const uint64_t* d_list_len, uint64_t stride,
                                uint64_t half, uint64_t n_commit, uint64_t* d_partial, uint64_t chunks, uint64_t* d_out) {
    if (!d_bits || !d_omega || !d_list || !d_list_off || !d_list_len || (stride & 63)) return MB_ERR_ARG;
    RoundArgs a = base_args(d_eq, d_tags, half, 1, d_partial);
    a.bits = d_bits;
    a.omega = d_omega;
    a.bits_stride_words = stride >> 6;
    a.omega_stride = stride;
    a.list = d_list;
    a.list_off = d_list_off;
    a.list_len = d_list_len;
    return run_round<true, true, false>(a, n_commit, chunks, d_out);
}

// Interleaved layout (block index in the low bits): weights scale[e][b] * eq(leaf index, pts[e][b][round..]).
int link_round_interleaved_ffi(const uint64_t* d_bits, const uint64_t* d_w, const uint64_t* d_pts, const uint64_t* d_scale,
                               const uint64_t* d_eq, const uint64_t* d_tags, const uint32_t* d_list, const uint64_t* d_list_off,
                               const uint64_t* d_list_len, uint64_t w_stride, uint64_t bits_stride_words, uint64_t half, uint64_t n_commit,
                               uint32_t block_mask, int block_bits, int leaf_arity, int round, int first_round, uint64_t* d_partial,
                               uint64_t chunks, uint64_t* d_out) {
    if (!d_pts || !d_scale || !d_list || !d_list_off || !d_list_len || round < 0 || round > leaf_arity || block_bits < 0 || block_bits > 31 ||
        (first_round ? !d_bits : !d_w))
        return MB_ERR_ARG;
    RoundArgs a = base_args(d_eq, d_tags, half, first_round, d_partial);
    a.bits = d_bits;
    a.w = d_w;
    a.pts = d_pts;
    a.scale = d_scale;
    a.w_stride = w_stride;
    a.bits_stride_words = bits_stride_words;
    a.list = d_list;
    a.list_off = d_list_off;
    a.list_len = d_list_len;
    a.block_mask = block_mask;
    a.block_bits = block_bits;
    a.leaf_arity = leaf_arity;
    a.round = round;
    return first_round ? run_round<true, true, true>(a, n_commit, chunks, d_out) : run_round<false, true, true>(a, n_commit, chunks, d_out);
}

int link_fold_ffi(uint64_t* d_w, uint64_t* d_omega, uint64_t stride, uint64_t omega_stride, uint64_t half, uint64_t n_commit, uint64_t r_c0,
                  uint64_t r_c1) {
    if (!d_w || !d_omega) return MB_ERR_ARG;
    if (half * n_commit == 0) return MB_OK;
    MB_KERNEL("link_fold");
    link_fold_kernel<<<grid_for(half * n_commit, BLOCK, 8), BLOCK, 0, MB_STREAM>>>(d_w, d_omega, stride, omega_stride, half, n_commit,
                                                                                  E2{r_c0, r_c1});
    return finish_sync();
}

int link_fold_sparse_ffi(uint64_t* d_w, uint64_t* d_omega, const uint32_t* d_list, const uint64_t* d_list_off, const uint64_t* d_list_len,
                         uint64_t stride, uint64_t half, uint64_t n_commit, uint64_t r_c0, uint64_t r_c1) {
    if (!d_w || !d_omega || !d_list || !d_list_off || !d_list_len || n_commit > 65535) return MB_ERR_ARG;
    if (n_commit == 0) return MB_OK;
    MB_KERNEL("link_fold_sparse");
    dim3 grid((unsigned)(sm_count() * 8 / (n_commit < 8 ? n_commit : 8) + 1), (unsigned)n_commit);
    link_fold_sparse_kernel<<<grid, BLOCK, 0, MB_STREAM>>>(d_w, d_omega, d_list, d_list_off, d_list_len, stride, half, E2{r_c0, r_c1});
    return finish_sync();
}

// Round-0 fold: bits in, half-size table out (rows of `half`), omega folded in place (rows of `stride`).
int link_fold0_bits_ffi(const uint64_t* d_bits, uint64_t* d_w_out, uint64_t* d_omega, uint64_t stride, uint64_t half, uint64_t n_commit,
                        uint64_t r_c0, uint64_t r_c1) {
    if (!d_bits || !d_w_out || !d_omega || (stride & 63)) return MB_ERR_ARG;
    if (half * n_commit == 0) return MB_OK;
    MB_KERNEL("link_fold0_bits");
    link_fold_w_kernel<true><<<grid_for(half * n_commit, BLOCK, 8), BLOCK, 0, MB_STREAM>>>(d_bits, nullptr, d_w_out, d_omega, 0, stride >> 6, half,
                                                                                          stride, half, n_commit, E2{r_c0, r_c1});
    return finish_sync();
}

// Witness-only fold of the interleaved layout.
int link_fold_w_ffi(const uint64_t* d_bits, const uint64_t* d_w_in, uint64_t* d_w_out, uint64_t in_stride, uint64_t bits_stride_words,
                    uint64_t out_stride, uint64_t half, uint64_t n_commit, int first_round, uint64_t r_c0, uint64_t r_c1) {
    if (!d_w_out || (first_round ? !d_bits : !d_w_in)) return MB_ERR_ARG;
    if (half * n_commit == 0) return MB_OK;
    MB_KERNEL("link_fold_w");
    const int grid = grid_for(half * n_commit, BLOCK, 8);
    if (first_round)
        link_fold_w_kernel<true><<<grid, BLOCK, 0, MB_STREAM>>>(d_bits, nullptr, d_w_out, nullptr, 0, bits_stride_words, out_stride, 0, half,
                                                                n_commit, E2{r_c0, r_c1});
    else
        link_fold_w_kernel<false><<<grid, BLOCK, 0, MB_STREAM>>>(nullptr, d_w_in, d_w_out, nullptr, in_stride, 0, out_stride, 0, half, n_commit,
                                                                 E2{r_c0, r_c1});
    return finish_sync();
}

// One variable of an eq table built most-significant variable first: the live span doubles.
int link_eq_expand_ffi(uint64_t* d_table, uint64_t span, uint64_t r_c0, uint64_t r_c1) {
    if (!d_table) return MB_ERR_ARG;
    if (span == 0) return MB_OK;
    MB_KERNEL("link_eq_expand");
    link_expand_kernel<<<dim3((unsigned)grid_for(span, BLOCK, 8), 1), BLOCK, 0, MB_STREAM>>>(d_table, nullptr, nullptr, span, E2{r_c0, r_c1});
    return finish_sync();
}

// The same step for n_active weight slices at once: slice q starts at element d_bases[q], challenge d_rs[q].
int link_omega_expand_ffi(uint64_t* d_omega, const uint64_t* d_bases, const uint64_t* d_rs, uint64_t span, uint64_t n_active) {
    if (!d_omega || !d_bases || !d_rs || n_active > 65535) return MB_ERR_ARG;
    if (span == 0 || n_active == 0) return MB_OK;
    MB_KERNEL("link_omega_expand");
    unsigned gx = (unsigned)((span + BLOCK - 1) / BLOCK);
    const unsigned cap = (unsigned)(sm_count() * 8 / (n_active < 8 ? n_active : 8) + 1);
    if (gx > cap) gx = cap;
    link_expand_kernel<<<dim3(gx, (unsigned)n_active), BLOCK, 0, MB_STREAM>>>(d_omega, d_bases, d_rs, span, E2{0, 0});
    return finish_sync();
}

// d_out[n_words * 64] extension elements (bit, 0).
int link_expand_bits_ffi(const uint64_t* d_bits, uint64_t* d_out, uint64_t n_words) {
    if (!d_bits || !d_out) return MB_ERR_ARG;
    if (n_words == 0) return MB_OK;
    MB_KERNEL("link_expand_bits");
    link_expand_bits_kernel<<<grid_for(n_words * 64, BLOCK, 8), BLOCK, 0, MB_STREAM>>>(d_bits, d_out, n_words * 64);
    return finish_sync();
}

// d_out[t] = eq(d_list[t], alpha), alpha = n_vars extension elements, most significant variable first.
int link_eq_gather_ffi(const uint64_t* d_alpha, uint64_t n_vars, const uint32_t* d_list, uint64_t* d_out, uint64_t total) {
    if (!d_alpha || !d_list || !d_out || n_vars > 32) return MB_ERR_ARG;
    if (total == 0) return MB_OK;
    MB_KERNEL("link_eq_gather");
    link_eq_gather_kernel<<<grid_for(total, BLOCK, 8), BLOCK, 0, MB_STREAM>>>(d_alpha, n_vars, d_list, d_out, total);
    return finish_sync();
}

}  // extern "C"
