// Partial evaluation of a multilinear table: fix its m low variables at r[0..m),
// out[j] = sum_b in[j 2^m + b] eq(r, b), by repeated folding
// T'[y] = T[2y] + r_i (T[2y+1] - T[2y])
// (reference: cuda/partial_eval.cuh:31-219, almost twin
// cuda_almost_goldilocks/almost_partial_eval.cuh:22-180, one launch and one full
// pass per variable). Here m variables take ceil(m / 4) passes and the traffic is
// about N (1 + 2^-4) instead of about 3 N.
//  * The first pass over a base-field table (the large one) is an inner product:
//    out[j] = sum_b in[16 j + b] w_b with the 16 weights eq(r[0..4), b) held in
//    registers, accumulated as exact 160-bit sums and reduced once per output
//    (two multiply-accumulate chains per element instead of a reduced fold per
//    level). A block stages 4096 consecutive elements in shared memory with
//    coalesced 16-byte loads; each thread then reads its run of 16 from a padded
//    layout without bank conflicts.
//  * Other passes (extension tables, at most 1/16 of the data) fold a run of 2^K
//    consecutive elements through K variables in registers.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace pe {

constexpr int K_MAX = 4;

// Folds variables [lvl, lvl + K): reads 2^K elements of FIn per output, the
// first level lifts FIn to FOut through FoldOp, the others stay in FOut.
// r holds FOut elements.
template <class FIn, class FOut, int K>
__global__ void __launch_bounds__(256)
fold_levels_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, const uint64_t* __restrict__ r, int lvl,
                   size_t n_out) {
    using TI = typename FIn::T;
    using TO = typename FOut::T;
    TO rr[K];
#pragma unroll
    for (int k = 0; k < K; k++) rr[k] = FOut::load(r, lvl + k);
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_out; j += step) {
        TO v[1 << (K - 1)];
#pragma unroll
        for (int p = 0; p < (1 << (K - 1)); p++) {
            TI a, b;
            FIn::load2(in, (j << K) + 2 * p, a, b);
            v[p] = sc::FoldOp<FIn, FOut>::apply(a, b, rr[0]);
        }
#pragma unroll
        for (int k = 1; k < K; k++) {
#pragma unroll
            for (int p = 0; p < (1 << (K - 1 - k)); p++)
                v[p] = sc::FoldOp<FOut, FOut>::apply(v[2 * p], v[2 * p + 1], rr[k]);
        }
        FOut::store(out, j, v[0]);
    }
}

// First pass over a base-field table: K variables at once as an inner product with
// eq weights. One tile = 256 outputs = 256 * 2^K inputs; n_out is a multiple of 256.
template <class FIn, class FOut, int K>
__global__ void __launch_bounds__(256, 4)
dot_levels_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, const uint64_t* __restrict__ r, int lvl,
                  size_t n_out) {
    using TO = typename FOut::T;
    constexpr int R = 1 << K;           // inputs per output
    constexpr int ROW = R + 1;          // padded run in shared memory
    __shared__ uint64_t tile[256 * ROW];
    __shared__ uint64_t wsm[2 * R];     // the weights stay in shared memory: registers are what bounds residency here
    if (threadIdx.x == 0) {
        // w_b = prod_k (b_k ? r_k : 1 - r_k), bit k of b with r[lvl + k]
        TO w[R];
        w[0] = TO{1, 0};
#pragma unroll
        for (int k = 0; k < K; k++) {
            const TO rk = FOut::load(r, lvl + k);
#pragma unroll
            for (int b = 0; b < (1 << k); b++) {
                TO hi = FOut::mul(w[b], rk);
                w[b + (1 << k)] = hi;
                w[b] = FOut::sub(w[b], hi);
            }
        }
#pragma unroll
        for (int b = 0; b < R; b++) FOut::to_words(w[b], wsm + 2 * b);
    }
    __syncthreads();
    const size_t tiles = n_out >> 8;
    for (size_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const uint64_t* src = in + t * (256 * R);
#pragma unroll
        for (int i = 0; i < R / 2; i++) {
            const int e = 2 * (i * 256 + (int)threadIdx.x);   // element index inside the tile, even
            ulonglong2 v = *reinterpret_cast<const ulonglong2*>(src + e);
            const int row = e >> K, col = e & (R - 1);
            tile[row * ROW + col] = v.x;
            tile[row * ROW + col + 1] = v.y;
        }
        __syncthreads();
        gl::Acc s0 = gl::acc_zero(), s1 = gl::acc_zero();
#pragma unroll
        for (int b = 0; b < R; b++) {
            const uint64_t v = tile[threadIdx.x * ROW + b];
            gl::acc_mul(s0, v, wsm[2 * b]);
            gl::acc_mul(s1, v, wsm[2 * b + 1]);
        }
        FOut::store(out, t * 256 + threadIdx.x, TO{FOut::reduce_acc(s0), FOut::reduce_acc(s1)});
        __syncthreads();
    }
}

template <class FIn, class FOut>
inline void launch_dot(const uint64_t* in, uint64_t* out, const uint64_t* r, int lvl, int k, size_t n_out, cudaStream_t st) {
    int grid = grid_for(n_out, 256, 4);
    MB_KERNEL_ON("partial_eval_dot", st);
    switch (k) {
        case 1: dot_levels_kernel<FIn, FOut, 1><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
        case 2: dot_levels_kernel<FIn, FOut, 2><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
        case 3: dot_levels_kernel<FIn, FOut, 3><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
        default: dot_levels_kernel<FIn, FOut, 4><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
    }
}

template <class FIn, class FOut>
inline void launch_levels(const uint64_t* in, uint64_t* out, const uint64_t* r, int lvl, int k, size_t n_out,
                          cudaStream_t st) {
    int grid = grid_for(n_out, 256, 8);
    MB_KERNEL_ON("partial_eval_levels", st);
    switch (k) {
        case 1: fold_levels_kernel<FIn, FOut, 1><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
        case 2: fold_levels_kernel<FIn, FOut, 2><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
        case 3: fold_levels_kernel<FIn, FOut, 3><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
        default: fold_levels_kernel<FIn, FOut, 4><<<grid, 256, 0, st>>>(in, out, r, lvl, n_out); break;
    }
}

// d_in: 2^log_n elements of FIn; result: 2^(log_n - m) elements of FOut in
// d_out. d_tmp: scratch of at least 2^(log_n - min(m, K_MAX)) FOut elements
// (unused when m <= K_MAX). d_in is not modified unless it aliases d_out/d_tmp.
template <class FIn, class FOut>
inline int partial_eval(const uint64_t* d_in, uint64_t* d_out, uint64_t* d_tmp, const uint64_t* d_r, int log_n, int m,
                        cudaStream_t st) {
    if (log_n < 0 || log_n > 40 || m < 0 || m > log_n || !d_in || !d_out || (m > 0 && !d_r)) return MB_ERR_ARG;
    if (m == 0) return MB_OK;
    int passes = (m + K_MAX - 1) / K_MAX;
    if (passes > 1 && !d_tmp) return MB_ERR_ARG;
    // ping-pong so that the last pass lands in d_out
    uint64_t* bufs[2] = {d_out, d_tmp};
    int which = (passes % 2 == 1) ? 0 : 1;
    const uint64_t* src = d_in;
    int lvl = 0, left = m, cur_log = log_n;
    bool first = true;
    while (left > 0) {
        int k = left < K_MAX ? left : K_MAX;
        size_t n_out = (size_t)1 << (cur_log - k);
        uint64_t* dst = bufs[which];
        bool done = false;
        if constexpr (FIn::NW == 1 && FOut::NW == 2) {
            if (first && n_out >= 256) {
                launch_dot<FIn, FOut>(src, dst, d_r, lvl, k, n_out, st);
                done = true;
            }
        }
        if (done) {
        } else if (first) {
            launch_levels<FIn, FOut>(src, dst, d_r, lvl, k, n_out, st);
        } else {
            launch_levels<FOut, FOut>(src, dst, d_r, lvl, k, n_out, st);
        }
        first = false;
        src = dst;
        which ^= 1;
        lvl += k;
        left -= k;
        cur_log -= k;
    }
    return finish_async();
}

}  // namespace pe
}  // namespace mb
