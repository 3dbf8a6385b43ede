// C-ABI: the batched same-point sumcheck family over almost-Goldilocks Ext2
// (reference: almost-goldilocks-cuda-rs/src/ffi.rs:177-195,265-423; kernels
// cuda_almost_goldilocks/almost_sumcheck_prover.cuh:233-1007; Rust drivers
// almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:468-1674).
//
// Every instance ("leaf") proves sum_x eq(x) f(x): degree 2, messages at
// c = 0, 1, 2. Three layouts of the same computation:
//   interleaved  d_polys[leaf] = eq table, then f table (2 N words each);
//   shared eq    eq tables of the distinct points in d_eq, f tables in d_f,
//                a leaf -> point map; eq is folded once per distinct point;
//   factored     eq is never folded: its suffix tables eqsuf_t are built once
//                and a round returns A = sum eqsuf[y] F[2y], B = sum eqsuf[y] F[2y+1].
// Message kernels write per-block partial sums in the reference's layout
// (the caller picks the number of blocks and adds the rows). Folds bind the
// low variable. All calls are asynchronous on the caller's stream, like the
// reference's.
#include "agl_traits.cuh"
#include "eq_kernels.cuh"

using namespace mb;
using namespace mb::sc;

namespace {

using E2 = agl::E2;
constexpr int BLK = 256;

__device__ __forceinline__ E2 ld(const uint64_t* p) { return agl::e2_load(p); }
__device__ __forceinline__ void st(uint64_t* p, E2 v) { agl::e2_store(p, agl::e2_canon(v)); }
__device__ __forceinline__ E2 fold2(E2 a, E2 b, E2 r) { return agl::e2_fma_pre(agl::e2_pre(r), agl::e2_sub(b, a), a); }
__device__ __forceinline__ uint64_t bit_at(const uint64_t* packed, size_t i) { return (packed[i >> 6] >> (i & 63)) & 1ULL; }

// partial[(blockIdx.x * gridDim.y + blockIdx.y) * 2 NV ...] = this block's sums
template <int NV>
__device__ __forceinline__ void store_block_sums(E2 (&acc)[NV], uint64_t* partial) {
    uint64_t v[2 * NV];
#pragma unroll
    for (int c = 0; c < NV; c++) { v[2 * c] = acc[c].c0; v[2 * c + 1] = acc[c].c1; }
    block_sum_store<2 * NV>(v, partial + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * 2 * NV, AglAdd(), AglCanon());
}

// Exact sum of extension products: c0 = s00 + 3 s11, c1 = s01 (X^2 = 3), every s an unreduced 160-bit sum of
// 64 x 64 products of canonical words (room for 2^32 of them); one reduction per thread at the end.
struct ProdSum {
    gl::Acc s00, s11, s01;
};
__device__ __forceinline__ ProdSum prod_zero() { return ProdSum{gl::acc_zero(), gl::acc_zero(), gl::acc_zero()}; }
__device__ __forceinline__ void prod_add(ProdSum& s, E2 a, E2 b) {
    gl::acc_mul(s.s00, a.c0, b.c0);
    gl::acc_mul(s.s11, a.c1, b.c1);
    gl::acc_mul(s.s01, a.c0, b.c1);
    gl::acc_mul(s.s01, a.c1, b.c0);
}
__device__ __forceinline__ E2 prod_reduce(const ProdSum& s) {
    // acc_reduce_wide: a thread may add thousands of products, the top limb is not small
    return E2{agl::add(agl::acc_reduce_wide(s.s00), agl::mul_small(agl::acc_reduce_wide(s.s11), 3)), agl::acc_reduce_wide(s.s01)};
}
// Exact sum of extension elements (128-bit integer sums of canonical words).
struct ElemSum {
    gl::Acc c0, c1;
};
__device__ __forceinline__ void elem_add(ElemSum& s, E2 a) {
    gl::acc_add(s.c0, a.c0);
    gl::acc_add(s.c1, a.c1);
}
__device__ __forceinline__ E2 elem_reduce(const ElemSum& s) { return E2{agl::acc_reduce_wide(s.c0), agl::acc_reduce_wide(s.c1)}; }

// m(0), m(1), m(2) of sum_y eq f over pairs (2y, 2y + 1). F_MODE 0: f is an Ext2 table; 1: packed bits.
// With d_e = e1 - e0, d_f = f1 - f0: m(2) = 2 m(1) - m(0) + 2 sum d_e d_f, so a pair costs three products that
// are accumulated without reduction (twelve 64 x 64 multiply-accumulates and two extension subtractions; the
// term-by-term form reduced every product and every partial sum). With a binary f the sums are selections:
// m(0) = sum of e0 over f0 = 1, m(1) = sum of e1 over f1 = 1, sum d_e d_f = sum of d_e over f1 > f0 minus the
// sum over f1 < f0, all exact integer sums.
template <int F_MODE>
__global__ void __launch_bounds__(BLK)
eqf_message_kernel(const uint64_t* __restrict__ eq_base, size_t eq_stride, const int* __restrict__ eq_map,
                   const uint64_t* __restrict__ f_base, size_t f_stride, size_t half, uint64_t* __restrict__ partial) {
    const int leaf = blockIdx.y;
    const uint64_t* eq = eq_base + (size_t)(eq_map ? eq_map[leaf] : leaf) * eq_stride;
    const uint64_t* f = f_base + (size_t)leaf * f_stride;
    E2 acc[3];
    const size_t step = (size_t)gridDim.x * blockDim.x;
    if (F_MODE == 0) {
        ProdSum p0 = prod_zero(), p1 = prod_zero(), pd = prod_zero();
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
            // any representative below 2^64 will do: the products are exact integers
            const E2 e0 = ld(eq + 4 * y), e1 = ld(eq + 4 * y + 2), f0 = ld(f + 4 * y), f1 = ld(f + 4 * y + 2);
            prod_add(p0, e0, f0);
            prod_add(p1, e1, f1);
            prod_add(pd, agl::e2_sub(e1, e0), agl::e2_sub(f1, f0));
        }
        acc[0] = prod_reduce(p0);
        acc[1] = prod_reduce(p1);
        const E2 d = prod_reduce(pd);
        acc[2] = agl::e2_add(agl::e2_sub(agl::e2_add(acc[1], acc[1]), acc[0]), agl::e2_add(d, d));
    } else {
        ElemSum s0{gl::acc_zero(), gl::acc_zero()}, s1 = s0, up = s0, down = s0;
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
            const uint64_t word = f[(2 * y) >> 6];
            const int f0 = (int)((word >> ((2 * y) & 63)) & 1), f1 = (int)((word >> ((2 * y + 1) & 63)) & 1);
            if (!(f0 | f1)) continue;
            const E2 e0 = ld(eq + 4 * y), e1 = ld(eq + 4 * y + 2);
            if (f0) elem_add(s0, e0);
            if (f1) elem_add(s1, e1);
            if (f0 != f1) {
                const E2 de = agl::e2_sub(e1, e0);
                if (f1) elem_add(up, de);
                else elem_add(down, de);
            }
        }
        acc[0] = elem_reduce(s0);
        acc[1] = elem_reduce(s1);
        const E2 d = agl::e2_sub(elem_reduce(up), elem_reduce(down));
        acc[2] = agl::e2_add(agl::e2_sub(agl::e2_add(acc[1], acc[1]), acc[0]), agl::e2_add(d, d));
    }
    store_block_sums<3>(acc, partial);
}

// Fold on r and the next round's message in one pass over the tables (an addition: the reference folds, then reads
// the folded tables again for the message). Thread per pair y of the FOLDED tables: it reads elements 4y .. 4y + 3 of
// eq and f (f from packed bits when F_MODE is 1: f' in {0, 1 - r, r, 1}), writes elements 2y, 2y + 1 of the folded
// tables and adds the pair to the exact sums of the message of the next round.
template <int F_MODE>
__global__ void __launch_bounds__(BLK)
eqf_fold_message_kernel(const uint64_t* __restrict__ in, const uint64_t* __restrict__ packed, size_t packed_words,
                        uint64_t* __restrict__ out, E2 r, size_t n, size_t quarter, uint64_t* __restrict__ partial) {
    const int leaf = blockIdx.y;
    const uint64_t* eq = in + (size_t)leaf * 4 * n;
    const uint64_t* f = eq + 2 * n;
    const uint64_t* bits = packed + (size_t)leaf * packed_words;
    uint64_t* oe = out + (size_t)leaf * 4 * n;
    uint64_t* of = oe + 2 * n;
    const agl::E2Pre pr = agl::e2_pre(r);
    const E2 one{1, 0}, rc = agl::e2_canon(r), omr = agl::e2_canon(agl::e2_sub(one, r));
    ProdSum p0 = prod_zero(), p1 = prod_zero(), pd = prod_zero();
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < quarter; y += step) {
        const E2 a0 = ld(eq + 8 * y), a1 = ld(eq + 8 * y + 2), a2 = ld(eq + 8 * y + 4), a3 = ld(eq + 8 * y + 6);
        const E2 e0 = agl::e2_canon(agl::e2_fma_pre(pr, agl::e2_sub(a1, a0), a0));
        const E2 e1 = agl::e2_canon(agl::e2_fma_pre(pr, agl::e2_sub(a3, a2), a2));
        E2 f0, f1;
        if (F_MODE == 0) {
            const E2 b0 = ld(f + 8 * y), b1 = ld(f + 8 * y + 2), b2 = ld(f + 8 * y + 4), b3 = ld(f + 8 * y + 6);
            f0 = agl::e2_canon(agl::e2_fma_pre(pr, agl::e2_sub(b1, b0), b0));
            f1 = agl::e2_canon(agl::e2_fma_pre(pr, agl::e2_sub(b3, b2), b2));
        } else {
            const unsigned nib = (unsigned)((bits[(4 * y) >> 6] >> ((4 * y) & 63)) & 15);   // four bits of one word
            const unsigned lo = nib & 3, hi = nib >> 2;
            f0 = lo == 3 ? one : lo == 2 ? rc : lo == 1 ? omr : E2{0, 0};
            f1 = hi == 3 ? one : hi == 2 ? rc : hi == 1 ? omr : E2{0, 0};
        }
        agl::e2_store(oe + 4 * y, e0);
        agl::e2_store(oe + 4 * y + 2, e1);
        agl::e2_store(of + 4 * y, f0);
        agl::e2_store(of + 4 * y + 2, f1);
        prod_add(p0, e0, f0);
        prod_add(p1, e1, f1);
        prod_add(pd, agl::e2_sub(e1, e0), agl::e2_sub(f1, f0));
    }
    E2 acc[3];
    acc[0] = prod_reduce(p0);
    acc[1] = prod_reduce(p1);
    const E2 d = prod_reduce(pd);
    acc[2] = agl::e2_add(agl::e2_sub(agl::e2_add(acc[1], acc[1]), acc[0]), agl::e2_add(d, d));
    store_block_sums<3>(acc, partial);
}

// A = sum_y eqsuf[y] F[2y], B = sum_y eqsuf[y] F[2y + 1]
__global__ void __launch_bounds__(BLK)
factored_message_kernel(const uint64_t* __restrict__ eqsuf, size_t eqsuf_stride, size_t eqsuf_off_words,
                        const uint64_t* __restrict__ fu, size_t poly_stride, size_t half, uint64_t* __restrict__ partial) {
    const int u = blockIdx.y;
    const uint64_t* e = eqsuf + (size_t)u * eqsuf_stride + eqsuf_off_words;
    const uint64_t* f = fu + (size_t)u * poly_stride;
    E2 acc[2] = {{0, 0}, {0, 0}};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
        const E2 w = ld(e + 2 * y);
        acc[0] = agl::e2_add(acc[0], agl::e2_mul_lazy(w, ld(f + 4 * y)));
        acc[1] = agl::e2_add(acc[1], agl::e2_mul_lazy(w, ld(f + 4 * y + 2)));
    }
    store_block_sums<2>(acc, partial);
}

// sum of eq[i] over the set bits of each plane
__global__ void __launch_bounds__(BLK)
selective_add_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ planes, size_t packed_words, size_t total,
                     uint64_t* __restrict__ partial) {
    const uint64_t* p = planes + (size_t)blockIdx.y * packed_words;
    E2 acc[1] = {{0, 0}};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
        if (bit_at(p, i)) acc[0] = agl::e2_add(acc[0], ld(eq + 2 * i));
    store_block_sums<1>(acc, partial);
}

// `tables` Ext2 tables per y-slice (blockIdx.y), out[y] = in[2y] + r (in[2y+1] - in[2y]); strides in words.
__global__ void __launch_bounds__(BLK)
fold_tables_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, E2 r, size_t slice_stride, size_t table_stride,
                   int tables, size_t half) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (int t = 0; t < tables; t++) {
        const uint64_t* pi = in + (size_t)blockIdx.y * slice_stride + (size_t)t * table_stride;
        uint64_t* po = out + (size_t)blockIdx.y * slice_stride + (size_t)t * table_stride;
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step)
            st(po + 2 * y, fold2(ld(pi + 4 * y), ld(pi + 4 * y + 2), r));
    }
}

// Round 0 with binary f: eq folded as usual, f' = f0 + r (f1 - f0) in {0, 1, r, 1 - r}.
__global__ void __launch_bounds__(BLK)
binary_fold_kernel(const uint64_t* __restrict__ polys, const uint64_t* __restrict__ packed, uint64_t* __restrict__ out, E2 r,
                   size_t n, size_t half, size_t packed_words) {
    const uint64_t* eq = polys + (size_t)blockIdx.y * 4 * n;
    const uint64_t* bits = packed + (size_t)blockIdx.y * packed_words;
    uint64_t* o = out + (size_t)blockIdx.y * 4 * n;
    const E2 one{1, 0}, omr = agl::e2_sub(one, r);
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
        st(o + 2 * y, fold2(ld(eq + 4 * y), ld(eq + 4 * y + 2), r));
        const uint64_t f0 = bit_at(bits, 2 * y), f1 = bit_at(bits, 2 * y + 1);
        E2 rf{0, 0};
        if (f0 && f1) rf = one;
        else if (f1) rf = r;
        else if (f0) rf = omr;
        st(o + 2 * n + 2 * y, rf);
    }
}

// Lifts of packed planes to Ext2 tables (second word zero). MODE 0: bits; 1: pos - neg.
template <int MODE>
__global__ void __launch_bounds__(BLK)
lift_kernel(const uint64_t* __restrict__ pos, const uint64_t* __restrict__ neg, uint64_t* __restrict__ out, size_t out_stride,
            size_t out_offset, size_t n, size_t packed_words) {
    const uint64_t* pp = pos + (size_t)blockIdx.y * packed_words;
    const uint64_t* pn = MODE ? neg + (size_t)blockIdx.y * packed_words : nullptr;
    uint64_t* o = out + (size_t)blockIdx.y * out_stride + out_offset;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        uint64_t c0 = bit_at(pp, i);
        if (MODE) c0 = agl::canon(c0 + bit_at(pn, i) * (agl::P - 1));
        *reinterpret_cast<ulonglong2*>(o + 2 * i) = make_ulonglong2(c0, 0);
    }
}

// F_u[x] = sum over the leaves of point u of alpha_leaf * f_leaf[x]; f binary (MODE 0) or pos - neg (MODE 1).
template <int MODE>
__global__ void __launch_bounds__(BLK)
build_fu_kernel(const uint64_t* __restrict__ pos, const uint64_t* __restrict__ neg, const uint64_t* __restrict__ alphas,
                const int* __restrict__ leaf_sorted, const int* __restrict__ offsets, uint64_t* __restrict__ fu, size_t n,
                size_t packed_words) {
    const int u = blockIdx.y, lo = offsets[u], hi = offsets[u + 1];
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x; x < n; x += step) {
        E2 acc{0, 0};
        for (int s = lo; s < hi; s++) {
            const int leaf = leaf_sorted[s];
            const bool pb = bit_at(pos + (size_t)leaf * packed_words, x);
            const bool nb = MODE ? bit_at(neg + (size_t)leaf * packed_words, x) : false;
            if (pb | nb) {
                const E2 a = ld(alphas + 2 * (size_t)leaf);
                if (pb) acc = agl::e2_add(acc, a);
                if (nb) acc = agl::e2_sub(acc, a);
            }
        }
        st(fu + (size_t)u * 2 * n + 2 * x, acc);
    }
}

// eqsuf_t[x_t + 2 y] = eq1(R_t, x_t) eqsuf_{t+1}[y]: one layer, the new variable is the low index bit.
__global__ void __launch_bounds__(BLK)
eq_suffix_layer_kernel(const uint64_t* __restrict__ r_all, uint64_t* __restrict__ eqsuf, int t, int log_n, size_t in_off,
                       size_t out_off, size_t in_size, size_t stride) {
    const int u = blockIdx.y;
    const E2 r = ld(r_all + ((size_t)u * log_n + t) * 2);
    uint64_t* base = eqsuf + (size_t)u * stride;
    const uint64_t* in = base + in_off * 2;
    uint64_t* out = base + out_off * 2;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < in_size; i += step) {
        const E2 a = ld(in + 2 * i), ar = agl::e2_mul(a, r);
        st(out + 4 * i, agl::e2_sub(a, ar));
        st(out + 4 * i + 2, ar);
    }
}
__global__ void eq_suffix_init_kernel(uint64_t* eqsuf, size_t stride) {
    eqsuf[(size_t)blockIdx.x * stride] = 1;
    eqsuf[(size_t)blockIdx.x * stride + 1] = 0;
}

inline int gx(size_t items, int requested = 0) {
    if (requested > 0) return requested;
    return grid_for(items, BLK, 8);
}

}  // namespace

extern "C" {

// d_partial[block][leaf][c][2], c = 0, 1, 2; d_polys[leaf] = eq table then f table, original_size elements each.
int aext2_sumcheck_batched_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, size_t original_size, size_t half,
                                             int num_leaves, int num_blocks_x) {
    if (!d_polys || !d_partial || num_leaves < 1 || num_blocks_x < 1 || half < 1 || half > original_size / 2) return MB_ERR_ARG;
    MB_KERNEL("aext2_batched_message");
    dim3 grid(num_blocks_x, num_leaves);
    eqf_message_kernel<0><<<grid, BLK, 0, MB_STREAM>>>(d_polys, 4 * original_size, nullptr, d_polys + 2 * original_size,
                                                        4 * original_size, half, d_partial);
    return finish_async();
}

int aext2_sumcheck_batched_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0, uint64_t challenge_c1,
                                    size_t original_size, size_t half, int num_leaves) {
    if (!d_input || !d_output || num_leaves < 1 || half < 1 || half > original_size / 2) return MB_ERR_ARG;
    MB_KERNEL("aext2_batched_fold");
    dim3 grid(gx(half), num_leaves);
    fold_tables_kernel<<<grid, BLK, 0, MB_STREAM>>>(d_input, d_output, E2{challenge_c0, challenge_c1}, 4 * original_size,
                                                    2 * original_size, 2, half);
    return finish_async();
}

int aext2_sumcheck_batched_round0_binary_msg_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_partial,
                                                 size_t original_size, size_t half, int num_leaves, int num_blocks_x,
                                                 size_t packed_size_u64) {
    if (!d_polys || !d_packed || !d_partial || num_leaves < 1 || num_blocks_x < 1 || half < 1 || half > original_size / 2)
        return MB_ERR_ARG;
    MB_KERNEL("aext2_batched_binary_message");
    dim3 grid(num_blocks_x, num_leaves);
    eqf_message_kernel<1><<<grid, BLK, 0, MB_STREAM>>>(d_polys, 4 * original_size, nullptr, d_packed, packed_size_u64, half, d_partial);
    return finish_async();
}

int aext2_sumcheck_batched_round0_binary_fold_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_output,
                                                  uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size, size_t half,
                                                  int num_leaves, size_t packed_size_u64) {
    if (!d_polys || !d_packed || !d_output || num_leaves < 1 || half < 1 || half > original_size / 2) return MB_ERR_ARG;
    MB_KERNEL("aext2_batched_binary_fold");
    dim3 grid(gx(half), num_leaves);
    binary_fold_kernel<<<grid, BLK, 0, MB_STREAM>>>(d_polys, d_packed, d_output, E2{challenge_c0, challenge_c1}, original_size, half,
                                                    packed_size_u64);
    return finish_async();
}

// Additions: the fold on the challenge and the message of the next round in one pass. `half` is the half of the
// INPUT tables (as for the fold); it must be even. d_partial[block][leaf][c][2] of the round after the fold.
int aext2_sumcheck_batched_fold_message_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0, uint64_t challenge_c1,
                                            size_t original_size, size_t half, int num_leaves, int num_blocks_x, uint64_t* d_partial) {
    if (!d_input || !d_output || !d_partial || num_leaves < 1 || num_blocks_x < 1 || half < 2 || (half & 1) || half > original_size / 2)
        return MB_ERR_ARG;
    MB_KERNEL("aext2_batched_fold_message");
    dim3 grid(num_blocks_x, num_leaves);
    eqf_fold_message_kernel<0><<<grid, BLK, 0, MB_STREAM>>>(d_input, d_input, 0, d_output, E2{challenge_c0, challenge_c1}, original_size,
                                                              half / 2, d_partial);
    return finish_async();
}
int aext2_sumcheck_batched_round0_binary_fold_message_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_output,
                                                          uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size, size_t half,
                                                          int num_leaves, int num_blocks_x, size_t packed_size_u64, uint64_t* d_partial) {
    if (!d_polys || !d_packed || !d_output || !d_partial || num_leaves < 1 || num_blocks_x < 1 || half < 2 || (half & 1) ||
        half > original_size / 2)
        return MB_ERR_ARG;
    MB_KERNEL("aext2_batched_binary_fold_message");
    dim3 grid(num_blocks_x, num_leaves);
    eqf_fold_message_kernel<1><<<grid, BLK, 0, MB_STREAM>>>(d_polys, d_packed, packed_size_u64, d_output, E2{challenge_c0, challenge_c1},
                                                              original_size, half / 2, d_partial);
    return finish_async();
}

int aext2_sharedeq_msg_ffi(const uint64_t* d_eq, const uint64_t* d_f, const int* d_leaf_to_unique, uint64_t* d_partial,
                           size_t original_size, size_t half, int num_leaves, int num_blocks_x) {
    if (!d_eq || !d_f || !d_leaf_to_unique || !d_partial || num_leaves < 1 || num_blocks_x < 1 || half < 1 ||
        half > original_size / 2)
        return MB_ERR_ARG;
    MB_KERNEL("aext2_sharedeq_message");
    dim3 grid(num_blocks_x, num_leaves);
    eqf_message_kernel<0><<<grid, BLK, 0, MB_STREAM>>>(d_eq, 2 * original_size, d_leaf_to_unique, d_f, 2 * original_size, half, d_partial);
    return finish_async();
}

// d_partial[block][unique][A, B][2]
int aext2_sharedeq_factored_msg_ffi(const uint64_t* d_eqsuf, const uint64_t* d_fu, uint64_t* d_partial, size_t eqsuf_off_elems,
                                    size_t eqsuf_stride_u64, size_t poly_stride_u64, size_t half, int num_unique, int num_blocks_x) {
    if (!d_eqsuf || !d_fu || !d_partial || num_unique < 1 || num_blocks_x < 1 || half < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_sharedeq_factored_message");
    dim3 grid(num_blocks_x, num_unique);
    factored_message_kernel<<<grid, BLK, 0, MB_STREAM>>>(d_eqsuf, eqsuf_stride_u64, 2 * eqsuf_off_elems, d_fu, poly_stride_u64, half, d_partial);
    return finish_async();
}

// `count` independent tables of original_size elements, each folded by the challenge.
int aext2_fold_single_ffi(const uint64_t* d_in, uint64_t* d_out, uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size,
                          size_t half, int count) {
    if (!d_in || !d_out || count < 1 || half < 1 || half > original_size / 2) return MB_ERR_ARG;
    MB_KERNEL("aext2_fold_single");
    dim3 grid(gx(half), count);
    fold_tables_kernel<<<grid, BLK, 0, MB_STREAM>>>(d_in, d_out, E2{challenge_c0, challenge_c1}, 2 * original_size, 0, 1, half);
    return finish_async();
}

// All suffix stages eqsuf_n .. eqsuf_1 of num_unique points: eqsuf_t at element offset 2^(log_n - t) - 1.
int aext2_eq_suffix_dp_ffi(const uint64_t* d_r_all, uint64_t* d_eqsuf, int log_n, int num_unique, size_t eqsuf_stride_u64) {
    if (!d_r_all || !d_eqsuf || log_n < 1 || log_n > 40 || num_unique < 1) return MB_ERR_ARG;
    {
        MB_KERNEL("aext2_eq_suffix_init");
        eq_suffix_init_kernel<<<num_unique, 1, 0, MB_STREAM>>>(d_eqsuf, eqsuf_stride_u64);
    }
    for (int t = log_n - 1; t >= 1; t--) {
        const size_t in_size = (size_t)1 << (log_n - t - 1), in_off = in_size - 1, out_off = ((size_t)1 << (log_n - t)) - 1;
        MB_KERNEL("aext2_eq_suffix_layer");
        dim3 grid(gx(in_size), num_unique);
        eq_suffix_layer_kernel<<<grid, BLK, 0, MB_STREAM>>>(d_r_all, d_eqsuf, t, log_n, in_off, out_off, in_size, eqsuf_stride_u64);
    }
    return finish_async();
}

int aext2_batched_lift_binary_ffi(const uint64_t* d_packed, uint64_t* d_polys, size_t original_size, int num_leaves,
                                  size_t packed_size_u64) {
    if (!d_packed || !d_polys || num_leaves < 1 || original_size < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_lift");
    dim3 grid(gx(original_size), num_leaves);
    lift_kernel<0><<<grid, BLK, 0, MB_STREAM>>>(d_packed, nullptr, d_polys, 4 * original_size, 2 * original_size, original_size, packed_size_u64);
    return finish_async();
}
int aext2_lift_binary_contig_ffi(const uint64_t* d_packed, uint64_t* d_f, size_t original_size, int num_leaves, size_t packed_size_u64) {
    if (!d_packed || !d_f || num_leaves < 1 || original_size < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_lift");
    dim3 grid(gx(original_size), num_leaves);
    lift_kernel<0><<<grid, BLK, 0, MB_STREAM>>>(d_packed, nullptr, d_f, 2 * original_size, 0, original_size, packed_size_u64);
    return finish_async();
}
int aext2_batched_lift_ternary_single_ffi(const uint64_t* d_pos, const uint64_t* d_neg, uint64_t* d_polys, size_t original_size,
                                          int num_leaves, size_t packed_size_u64) {
    if (!d_pos || !d_neg || !d_polys || num_leaves < 1 || original_size < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_lift");
    dim3 grid(gx(original_size), num_leaves);
    lift_kernel<1><<<grid, BLK, 0, MB_STREAM>>>(d_pos, d_neg, d_polys, 4 * original_size, 2 * original_size, original_size, packed_size_u64);
    return finish_async();
}

// d_partial[block][plane][2] = this block's share of sum_{i in plane} eq[i]
int aext2_selective_add_batched_planes_ffi(const uint64_t* d_eq, const uint64_t* d_packed_planes, uint64_t* d_partial, size_t total,
                                           int n_planes, size_t packed_size_u64, int num_blocks_x) {
    if (!d_eq || !d_packed_planes || !d_partial || n_planes < 1 || num_blocks_x < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_selective_add");
    dim3 grid(num_blocks_x, n_planes);
    selective_add_kernel<<<grid, BLK, 0, MB_STREAM>>>(d_eq, d_packed_planes, packed_size_u64, total, d_partial);
    return finish_async();
}

int aext2_build_fu_ffi(const uint64_t* d_packed, const uint64_t* d_alphas, const int* d_leaf_idx_sorted, const int* d_unique_offsets,
                       uint64_t* d_Fu, size_t original_size, int num_unique, size_t packed_size_u64) {
    if (!d_packed || !d_alphas || !d_leaf_idx_sorted || !d_unique_offsets || !d_Fu || num_unique < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_build_fu");
    dim3 grid(gx(original_size), num_unique);
    build_fu_kernel<0><<<grid, BLK, 0, MB_STREAM>>>(d_packed, nullptr, d_alphas, d_leaf_idx_sorted, d_unique_offsets, d_Fu, original_size,
                                                    packed_size_u64);
    return finish_async();
}
int aext2_build_fu_ternary_ffi(const uint64_t* d_pos, const uint64_t* d_neg, const uint64_t* d_alphas, const int* d_leaf_idx_sorted,
                               const int* d_unique_offsets, uint64_t* d_Fu, size_t original_size, int num_unique, size_t packed_size_u64) {
    if (!d_pos || !d_neg || !d_alphas || !d_leaf_idx_sorted || !d_unique_offsets || !d_Fu || num_unique < 1) return MB_ERR_ARG;
    MB_KERNEL("aext2_build_fu");
    dim3 grid(gx(original_size), num_unique);
    build_fu_kernel<1><<<grid, BLK, 0, MB_STREAM>>>(d_pos, d_neg, d_alphas, d_leaf_idx_sorted, d_unique_offsets, d_Fu, original_size,
                                                    packed_size_u64);
    return finish_async();
}

// eq tables on a caller stream (ffi.rs:177-195). The table is returned in d_buf_a; d_buf_b is scratch.
int aext2_eq_dp_all_stream_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result, void* stream) {
    if (!d_result) return MB_ERR_ARG;
    int rc = eq::build<AglExt2>(d_r, d_buf_a, d_buf_b, log_n, stream ? (cudaStream_t)stream : MB_STREAM);
    if (rc == MB_OK) *d_result = d_buf_a;
    return rc;
}
// num_leaves tables: point l at d_r_all + l * log_n elements, buffers l at leaf_stride elements apart.
int aext2_eq_dp_all_batched_ffi(const uint64_t* d_r_all, uint64_t* d_buf_a_all, uint64_t* d_buf_b_all, int log_n, int num_leaves,
                                size_t leaf_stride, uint64_t** d_result, void* stream) {
    if (!d_result || num_leaves < 0) return MB_ERR_ARG;
    cudaStream_t s = stream ? (cudaStream_t)stream : MB_STREAM;
    for (int l = 0; l < num_leaves; l++) {
        int rc = eq::build<AglExt2>(d_r_all + (size_t)l * log_n * 2, d_buf_a_all + (size_t)l * leaf_stride * 2,
                                    d_buf_b_all + (size_t)l * leaf_stride * 2, log_n, s);
        if (rc != MB_OK) return rc;
    }
    *d_result = d_buf_a_all;
    return MB_OK;
}

}  // extern "C"
