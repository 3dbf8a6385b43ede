// Multilinear sumcheck kernels, generic over the field (a traits class).
//
// Work per round of the linear sumcheck (reference kernels
// cuda/sumcheck_prover.cuh:37-151,171-292 and the almost-Goldilocks twins
// cuda_almost_goldilocks/almost_sumcheck_prover.cuh:24-218):
//   message  P(c) = sum_y prod_i (a_i + c (b_i - a_i)),  c = 0..D,
//            a_i = T_i[2y], b_i = T_i[2y+1]
//   fold     T_i'[y] = a_i + r (b_i - a_i)
// The reference launches these as two kernels per round, so every table is read
// twice. Here the fold on challenge r_k is fused with the message of round k+1:
// one pass reads four consecutive elements per table, writes the two folded
// ones and accumulates the next message from them, so each round streams the
// tables through HBM once (read S, write S/2).
//
// Tables are poly-major with a fixed stride (the original table length), the
// layout of GpuSumcheckState (goldilocks-cuda-rs/src/sumcheck_prover.rs:20-28).
// Everything written to global memory is canonical.
#pragma once
#include "common.cuh"
#include "gl_field.cuh"

namespace mb {
namespace sc {

constexpr int BLOCK = 256;
constexpr int MAX_D = 8;  // cuda/sumcheck_prover.cuh:18-19

// ---- field traits ---------------------------------------------------------
// WordAdd / WordCanon act on single u64 residues of the base field; block
// reductions use them on the flattened words of an element.
struct GlAdd {
    __device__ __forceinline__ uint64_t operator()(uint64_t a, uint64_t b) const { return gl::add(a, b); }
};
struct GlCanon {
    __host__ __device__ __forceinline__ uint64_t operator()(uint64_t a) const { return gl::canon(a); }
};

struct GlBase {
    using T = uint64_t;
    using WordAdd = GlAdd;
    using WordCanon = GlCanon;
    static constexpr int NW = 1;
    static __device__ __forceinline__ T load(const uint64_t* p, size_t i) { return p[i]; }
    static __device__ __forceinline__ void load2(const uint64_t* p, size_t i, T& a, T& b) {
        ulonglong2 v = *reinterpret_cast<const ulonglong2*>(p + i);
        a = v.x; b = v.y;
    }
    static __device__ __forceinline__ void store(uint64_t* p, size_t i, T v) { p[i] = gl::canon(v); }
    static __device__ __forceinline__ void store2(uint64_t* p, size_t i, T a, T b) {
        *reinterpret_cast<ulonglong2*>(p + i) = make_ulonglong2(gl::canon(a), gl::canon(b));
    }
    static __device__ __forceinline__ T add(T a, T b) { return gl::add(a, b); }
    static __device__ __forceinline__ T sub(T a, T b) { return gl::sub(a, b); }
    static __device__ __forceinline__ T mul(T a, T b) { return gl::mul(a, b); }
    static __device__ __forceinline__ T zero() { return 0; }
    static __device__ __forceinline__ void to_words(T v, uint64_t* w) { w[0] = v; }
    static __device__ __forceinline__ T from_words(const uint64_t* w) { return w[0]; }
    // a factor used many times (nothing to prepare in the base field)
    using Pre = uint64_t;
    static __device__ __forceinline__ Pre pre(T x) { return x; }
    static __device__ __forceinline__ T mul_pre(Pre p, T x) { return gl::mul(p, x); }
};

struct GlExt2 {
    using T = gl::E2;
    using WordAdd = GlAdd;
    using WordCanon = GlCanon;
    static constexpr int NW = 2;
    static __device__ __forceinline__ T load(const uint64_t* p, size_t i) { return gl::e2_load(p + 2 * i); }
    static __device__ __forceinline__ void load2(const uint64_t* p, size_t i, T& a, T& b) {
        a = gl::e2_load(p + 2 * i);
        b = gl::e2_load(p + 2 * i + 2);
    }
    static __device__ __forceinline__ void store(uint64_t* p, size_t i, T v) {
        gl::e2_store(p + 2 * i, gl::e2_canon(v));
    }
    static __device__ __forceinline__ void store2(uint64_t* p, size_t i, T a, T b) {
        store(p, i, a);
        store(p, i + 1, b);
    }
    static __device__ __forceinline__ T add(T a, T b) { return gl::e2_add(a, b); }
    static __device__ __forceinline__ T sub(T a, T b) { return gl::e2_sub(a, b); }
    static __device__ __forceinline__ T mul(T a, T b) { return gl::e2_mul_lazy(a, b); }
    static __device__ __forceinline__ T zero() { return gl::E2{0, 0}; }
    static __device__ __forceinline__ void to_words(T v, uint64_t* w) { w[0] = v.c0; w[1] = v.c1; }
    static __device__ __forceinline__ T from_words(const uint64_t* w) { return T{w[0], w[1]}; }
    // a factor used many times, with its c1 times the non-residue prepared: four products, two reductions
    using Pre = gl::E2Pre;
    static __device__ __forceinline__ Pre pre(T x) { return gl::e2_pre(x); }
    static __device__ __forceinline__ T mul_pre(Pre p, T x) { return gl::e2_mul_pre(p, x); }
    // an exact sum of at most 64 products of 64-bit words, reduced to a loose residue
    static __device__ __forceinline__ uint64_t reduce_acc(const gl::Acc& s) { return gl::acc_reduce(s); }
};

// Exact sums of products for a field: A holds sum x_k y_k without any reduction; at most LAZY_MAX products
// may be added before reduce(). Specialised per field (almost-Goldilocks in agl_traits.cuh).
template <class F>
struct Lazy;
constexpr int LAZY_MAX = 64;
template <>
struct Lazy<GlBase> {
    using A = gl::Acc;
    static __device__ __forceinline__ A zero() { return gl::acc_zero(); }
    static __device__ __forceinline__ void mul(A& s, uint64_t x, uint64_t y) { gl::acc_mul(s, x, y); }
    static __device__ __forceinline__ uint64_t reduce(const A& s) { return gl::acc_reduce(s); }
};
template <>
struct Lazy<GlExt2> {
    using A = gl::E2Acc;
    static __device__ __forceinline__ A zero() { return gl::e2acc_zero(); }
    static __device__ __forceinline__ void mul(A& s, gl::E2 x, gl::E2 y) { gl::e2acc_mul(s, x, y); }
    static __device__ __forceinline__ gl::E2 reduce(const A& s) { return gl::e2acc_reduce(s); }
};

// Round polynomial of a product of two tables from three exact sums. With a = value at 0, b = value at 1 and
// d = b - a per table, P(c) = S0 + c S1 + c^2 S2 where S0 = sum a0 a1 = P(0), S2 = sum d0 d1 and
// P(1) = sum b0 b1, hence P(2) = 2 P(1) - S0 + 2 S2. The three sums take one multiply-accumulate chain each per
// pair and are reduced once per LAZY_MAX pairs, instead of three reduced products, three modular additions and
// two rounds of value updates per pair.
template <class F>
struct PairSums {
    using T = typename F::T;
    typename Lazy<F>::A s0, s1, s2;
    T t0, t1, t2;
    int pending;
    __device__ __forceinline__ void init() {
        s0 = Lazy<F>::zero(); s1 = Lazy<F>::zero(); s2 = Lazy<F>::zero();
        t0 = F::zero(); t1 = F::zero(); t2 = F::zero();
        pending = 0;
    }
    __device__ __forceinline__ void flush() {
        t0 = F::add(t0, Lazy<F>::reduce(s0));
        t1 = F::add(t1, Lazy<F>::reduce(s1));
        t2 = F::add(t2, Lazy<F>::reduce(s2));
        s0 = Lazy<F>::zero(); s1 = Lazy<F>::zero(); s2 = Lazy<F>::zero();
        pending = 0;
    }
    // a_i, b_i: the two tables' values at 0 and 1
    __device__ __forceinline__ void add_pair(T a0, T b0, T a1, T b1) {
        Lazy<F>::mul(s0, a0, a1);
        Lazy<F>::mul(s1, b0, b1);
        Lazy<F>::mul(s2, F::sub(b0, a0), F::sub(b1, a1));
        if (++pending == LAZY_MAX) flush();
    }
    // acc[0..2] = this thread's share of P(0), P(1), P(2)
    __device__ __forceinline__ void finish(T (&acc)[3]) {
        flush();
        acc[0] = t0;
        acc[1] = t1;
        T twice = F::add(F::add(t1, t1), F::add(t2, t2));
        acc[2] = F::sub(twice, t0);
    }
};

// ---- block-wide sum of NV residues per thread -------------------------------
// Warp shuffles, then one shared-memory hop across warps. Thread 0 writes the
// canonical totals to out[0..NV). blockDim.x must be a multiple of 32.
template <int NV, class AddFn, class CanonFn>
__device__ __forceinline__ void block_sum_store(uint64_t (&v)[NV], uint64_t* out, AddFn addf, CanonFn canonf) {
    __shared__ uint64_t sm[32][NV];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int k = 0; k < NV; k++) v[k] = addf(v[k], __shfl_down_sync(0xffffffffu, v[k], off));
    }
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < NV; k++) sm[warp][k] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
#pragma unroll
        for (int k = 0; k < NV; k++) v[k] = lane < nw ? sm[lane][k] : 0;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int k = 0; k < NV; k++) v[k] = addf(v[k], __shfl_down_sync(0xffffffffu, v[k], off));
        }
        if (lane == 0) {
#pragma unroll
            for (int k = 0; k < NV; k++) out[k] = canonf(v[k]);
        }
    }
}

// acc[c] += prod_i (val_i + c * diff_i) for c = 0..D; consumes val.
template <class F, int D>
__device__ __forceinline__ void accumulate_pair(typename F::T (&val)[D], const typename F::T (&diff)[D],
                                                typename F::T (&acc)[D + 1]) {
#pragma unroll
    for (int c = 0; c <= D; c++) {
        typename F::T prod = val[0];
#pragma unroll
        for (int i = 1; i < D; i++) prod = F::mul(prod, val[i]);
        acc[c] = F::add(acc[c], prod);
        if (c < D) {
#pragma unroll
            for (int i = 0; i < D; i++) val[i] = F::add(val[i], diff[i]);
        }
    }
}

// Block partial -> global row; optionally the last block to finish adds all rows
// up ("last block done" pattern: a fence, one atomic ticket per block) and
// writes the (D+1)*NW canonical totals to final_out, so no second launch and no
// host-side summation is needed. `counter` must be zero on entry and is reset
// to zero by the last block. Rows written by other blocks are read with
// cache-global loads, which never hit a stale L1 line.
template <class F, int D>
__device__ __forceinline__ void store_partials(typename F::T (&acc)[D + 1], uint64_t* partial,
                                                unsigned int* counter, uint64_t* final_out) {
    constexpr int NV = (D + 1) * F::NW;
    uint64_t v[NV];
#pragma unroll
    for (int c = 0; c <= D; c++) F::to_words(acc[c], v + c * F::NW);
    block_sum_store<NV>(v, partial + (size_t)blockIdx.x * NV, typename F::WordAdd(), typename F::WordCanon());
    if (final_out == nullptr) return;
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        __threadfence();
        unsigned int ticket = atomicAdd(counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll
    for (int k = 0; k < NV; k++) v[k] = 0;
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
#pragma unroll
        for (int k = 0; k < NV; k++) v[k] = typename F::WordAdd()(v[k], __ldcg(partial + (size_t)b * NV + k));
    }
    block_sum_store<NV>(v, final_out, typename F::WordAdd(), typename F::WordCanon());
    if (threadIdx.x == 0) *counter = 0;
}

// ---- round message ----------------------------------------------------------
// partial[(blockIdx.x * (D+1) + c) * NW ...] = this block's share of P(c).
template <class F, int D>
__global__ void __launch_bounds__(D == 2 ? 512 : D == 3 ? 1024 : 256)   // D = 2 keeps exact sums in registers
round_message_kernel(const uint64_t* __restrict__ polys, size_t stride, size_t half, uint64_t* __restrict__ partial,
                     unsigned int* counter, uint64_t* final_out) {
    using T = typename F::T;
    T acc[D + 1];
    const size_t step = (size_t)gridDim.x * blockDim.x;
    if constexpr (D == 2) {
        PairSums<F> ps;
        ps.init();
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
            T a0, b0, a1, b1;
            F::load2(polys, 2 * y, a0, b0);
            F::load2(polys + stride * F::NW, 2 * y, a1, b1);
            ps.add_pair(a0, b0, a1, b1);
        }
        ps.finish(acc);
    } else {
#pragma unroll
        for (int c = 0; c <= D; c++) acc[c] = F::zero();
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
            T val[D], diff[D];
#pragma unroll
            for (int i = 0; i < D; i++) {
                T a, b;
                F::load2(polys + (size_t)i * stride * F::NW, 2 * y, a, b);
                val[i] = a;
                diff[i] = F::sub(b, a);
            }
            accumulate_pair<F, D>(val, diff, acc);
        }
    }
    store_partials<F, D>(acc, partial, counter, final_out);
}

// ---- plain fold (out of place) ------------------------------------------------
// out[i*stride + y] = a + r (b - a); blockIdx.y selects the table.
template <class F>
__global__ void fold_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, typename F::T r,
                            size_t stride, size_t half) {
    using T = typename F::T;
    const uint64_t* pin = in + (size_t)blockIdx.y * stride * F::NW;
    uint64_t* pout = out + (size_t)blockIdx.y * stride * F::NW;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
        T a, b;
        F::load2(pin, 2 * y, a, b);
        F::store(pout, y, F::add(a, F::mul(r, F::sub(b, a))));
    }
}

// ---- fused fold + next message ---------------------------------------------------
// Input tables hold 4*quarter live elements each; the fold on r writes
// 2*quarter elements per table and the message of the following round is
// accumulated from them. FIn is the input field; the output and the message are
// always in FOut (a base-field input is lifted by the extension challenge).
template <class FIn, class FOut>
struct FoldOp;

template <class F>
struct FoldOp<F, F> {
    static __device__ __forceinline__ typename F::T apply(typename F::T a, typename F::T b, typename F::T r) {
        return F::add(a, F::mul(r, F::sub(b, a)));
    }
};
// Goldilocks: a + r (b - a) as two exact sums of products (the factor r with
// 7 r.c1 precomputed is loop invariant), one reduction per component.
template <>
struct FoldOp<GlBase, GlExt2> {
    static __device__ __forceinline__ gl::E2 apply(uint64_t a, uint64_t b, gl::E2 r) {
        return gl::e2_fma_pre_base(gl::e2_pre(r), gl::sub(b, a), a);
    }
};
template <>
struct FoldOp<GlExt2, GlExt2> {
    static __device__ __forceinline__ gl::E2 apply(gl::E2 a, gl::E2 b, gl::E2 r) {
        return gl::e2_fma_pre(gl::e2_pre(r), gl::e2_sub(b, a), a);
    }
};

template <class FIn, class FOut, int D>
__global__ void __launch_bounds__(BLOCK)
fold_message_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, typename FOut::T r_val,
                    const uint64_t* __restrict__ r_ptr, size_t stride_in, size_t stride_out, size_t quarter,
                    uint64_t* __restrict__ partial, unsigned int* counter, uint64_t* final_out) {
    using TI = typename FIn::T;
    using TO = typename FOut::T;
    TO r = r_val;
    if (r_ptr != nullptr) r = FOut::load(r_ptr, 0);
    TO acc[D + 1];
    const size_t step = (size_t)gridDim.x * blockDim.x;
    if constexpr (D == 2) {
        PairSums<FOut> ps;
        ps.init();
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < quarter; y += step) {
            TO f[2][2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                TI e0, e1, e2, e3;
                const uint64_t* pin = in + (size_t)i * stride_in * FIn::NW;
                FIn::load2(pin, 4 * y, e0, e1);
                FIn::load2(pin, 4 * y + 2, e2, e3);
                f[i][0] = FoldOp<FIn, FOut>::apply(e0, e1, r);
                f[i][1] = FoldOp<FIn, FOut>::apply(e2, e3, r);
                FOut::store2(out + (size_t)i * stride_out * FOut::NW, 2 * y, f[i][0], f[i][1]);
            }
            ps.add_pair(f[0][0], f[0][1], f[1][0], f[1][1]);
        }
        ps.finish(acc);
    } else {
#pragma unroll
        for (int c = 0; c <= D; c++) acc[c] = FOut::zero();
        for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < quarter; y += step) {
            TO val[D], diff[D];
#pragma unroll
            for (int i = 0; i < D; i++) {
                TI e0, e1, e2, e3;
                const uint64_t* pin = in + (size_t)i * stride_in * FIn::NW;
                FIn::load2(pin, 4 * y, e0, e1);
                FIn::load2(pin, 4 * y + 2, e2, e3);
                TO f0 = FoldOp<FIn, FOut>::apply(e0, e1, r);
                TO f1 = FoldOp<FIn, FOut>::apply(e2, e3, r);
                FOut::store2(out + (size_t)i * stride_out * FOut::NW, 2 * y, f0, f1);
                val[i] = f0;
                diff[i] = FOut::sub(f1, f0);
            }
            accumulate_pair<FOut, D>(val, diff, acc);
        }
    }
    store_partials<FOut, D>(acc, partial, counter, final_out);
}

// Last fold of a base-field table pair by an extension challenge (no message).
template <class FIn, class FOut>
__global__ void fold_lift_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, typename FOut::T r_val,
                                 const uint64_t* __restrict__ r_ptr, size_t stride_in, size_t stride_out, size_t half) {
    typename FOut::T r = r_val;
    if (r_ptr != nullptr) r = FOut::load(r_ptr, 0);
    const uint64_t* pin = in + (size_t)blockIdx.y * stride_in * FIn::NW;
    uint64_t* pout = out + (size_t)blockIdx.y * stride_out * FOut::NW;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < half; y += step) {
        typename FIn::T a, b;
        FIn::load2(pin, 2 * y, a, b);
        FOut::store(pout, y, FoldOp<FIn, FOut>::apply(a, b, r));
    }
}

// Sum `nblocks` block partials of NV words each into out[0..NV): one block.
template <int BLOCKDIM, class AddFn, class CanonFn>
__global__ void reduce_partials_kernel(const uint64_t* __restrict__ partial, int nblocks, int nv,
                                       uint64_t* __restrict__ out) {
    __shared__ uint64_t sm[BLOCKDIM];
    for (int k = 0; k < nv; k++) {
        uint64_t s = 0;
        for (int b = threadIdx.x; b < nblocks; b += BLOCKDIM) s = AddFn()(s, partial[(size_t)b * nv + k]);
        sm[threadIdx.x] = s;
        __syncthreads();
        for (int off = BLOCKDIM / 2; off > 0; off >>= 1) {
            if (threadIdx.x < off) sm[threadIdx.x] = AddFn()(sm[threadIdx.x], sm[threadIdx.x + off]);
            __syncthreads();
        }
        if (threadIdx.x == 0) out[k] = CanonFn()(sm[0]);
        __syncthreads();
    }
}

}  // namespace sc
}  // namespace mb
