// eq(r, x) tables for all x in {0,1}^n, bit i of x <-> r[i]
// (reference: cuda/eq_lagrange.cuh:22-158, convention pinned by the CPU loop in
// cuda/eq_lagrange_kernels.cu:31-53).
//
// The reference doubles the table n times with one launch per variable. The
// table is a tensor product, so here two small tables (low and high variables)
// are built by one launch of two blocks and a single write-only pass forms
// out[x] = lo[x & mask] * hi[x >> n_lo]: one multiplication per element and no
// re-reading of partial tables. Products of the same factors give the same
// residue in any order, so the result is bit-identical.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace eq {

// Block b builds the table over variables [lo_b, lo_b + nbits_b) into out_b,
// doubling in place: out[j + half] = a r, out[j] = a - a r.
// `init` (may be null) points at one element that replaces the initial 1 of block 0's
// table, which scales the whole eq table by it.
template <class F>
__global__ void small_tables_kernel(const uint64_t* __restrict__ r, int nbits0, uint64_t* out0, int nbits1,
                                    uint64_t* out1, const uint64_t* __restrict__ init = nullptr) {
    using T = typename F::T;
    const int var_lo = blockIdx.x == 0 ? 0 : nbits0;
    const int nbits = blockIdx.x == 0 ? nbits0 : nbits1;
    uint64_t* out = blockIdx.x == 0 ? out0 : out1;
    if (threadIdx.x == 0) {
        uint64_t one[2] = {1, 0};
        for (int w = 0; w < F::NW; w++) out[w] = (init != nullptr && blockIdx.x == 0) ? init[w] : one[w];
    }
    __syncthreads();
    for (int i = 0; i < nbits; i++) {
        T ri = F::load(r, var_lo + i);
        const size_t half = (size_t)1 << i;
        for (size_t j = threadIdx.x; j < half; j += blockDim.x) {
            T a = F::load(out, j);
            T ar = F::mul(a, ri);
            F::store(out, j, F::sub(a, ar));
            F::store(out, j + half, ar);
        }
        __syncthreads();
    }
}

// out[row 2^n_lo + j] = lo[j] * hi[row]: a block keeps one hi entry (prepared once) per row of 2^n_lo outputs.
template <class F>
__global__ void __launch_bounds__(256)
outer_product_kernel(const uint64_t* __restrict__ lo, const uint64_t* __restrict__ hi, int n_lo,
                     uint64_t* __restrict__ out, size_t n) {
    const size_t lo_size = (size_t)1 << n_lo, rows = n >> n_lo;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const typename F::Pre h = F::pre(F::load(hi, row));
        for (size_t j = threadIdx.x; j < lo_size; j += blockDim.x)
            F::store(out, row * lo_size + j, F::mul_pre(h, F::load(lo, j)));
    }
}

// Builds the table in d_out (2^log_n elements). d_scratch needs room for
// 2^(log_n/2) + 2^(log_n - log_n/2) elements when log_n > 12 (unused otherwise).
template <class F>
inline int build(const uint64_t* d_r, uint64_t* d_out, uint64_t* d_scratch, int log_n, cudaStream_t st,
                 const uint64_t* d_init = nullptr) {
    if (log_n < 0 || log_n > 40 || !d_out || (log_n > 0 && !d_r)) return MB_ERR_ARG;
    if (log_n <= 12) {
        {
            MB_KERNEL_ON("small_tables", st);
            small_tables_kernel<F><<<1, 256, 0, st>>>(d_r, log_n, d_out, 0, d_out, d_init);
        }
        return finish_async();
    }
    if (!d_scratch) return MB_ERR_ARG;
    int n_lo = log_n / 2, n_hi = log_n - n_lo;
    uint64_t* lo = d_scratch;
    uint64_t* hi = d_scratch + ((size_t)F::NW << n_lo);
    {
        MB_KERNEL_ON("small_tables", st);
        small_tables_kernel<F><<<2, 1024, 0, st>>>(d_r, n_lo, lo, n_hi, hi, d_init);
    }
    size_t n = (size_t)1 << log_n;
    {
        MB_KERNEL_ON("outer_product", st);
        outer_product_kernel<F><<<grid_for((n >> n_lo) * 256, 256, 8), 256, 0, st>>>(lo, hi, n_lo, d_out, n);
    }
    return finish_async();
}

// `count` tables of 2^log_n elements at once: table t from the point at d_r + t * r_stride words into
// d_out + t * out_stride words. d_scratch needs count * (2^(log_n/2) + 2^(log_n - log_n/2)) elements when
// log_n > 12. Two launches for all tables instead of two per table (a small-tables launch keeps two blocks busy).
template <class F>
__global__ void small_tables_batched_kernel(const uint64_t* __restrict__ r_all, size_t r_stride, int nbits0, int nbits1,
                                            uint64_t* scratch_all, size_t scratch_stride) {
    using T = typename F::T;
    const size_t t = blockIdx.x >> 1;
    const int which = blockIdx.x & 1;
    const uint64_t* r = r_all + t * r_stride;
    const int var_lo = which == 0 ? 0 : nbits0;
    const int nbits = which == 0 ? nbits0 : nbits1;
    uint64_t* out = scratch_all + t * scratch_stride + (which == 0 ? 0 : ((size_t)F::NW << nbits0));
    if (threadIdx.x == 0) {
        const uint64_t one[2] = {1, 0};
        for (int w = 0; w < F::NW; w++) out[w] = one[w];
    }
    __syncthreads();
    for (int i = 0; i < nbits; i++) {
        T ri = F::load(r, var_lo + i);
        const size_t half = (size_t)1 << i;
        for (size_t j = threadIdx.x; j < half; j += blockDim.x) {
            T a = F::load(out, j);
            T ar = F::mul(a, ri);
            F::store(out, j, F::sub(a, ar));
            F::store(out, j + half, ar);
        }
        __syncthreads();
    }
}
template <class F>
__global__ void __launch_bounds__(256)
outer_product_batched_kernel(const uint64_t* __restrict__ scratch_all, size_t scratch_stride, int n_lo, uint64_t* __restrict__ out_all,
                             size_t out_stride, size_t n) {
    const uint64_t* lo = scratch_all + (size_t)blockIdx.y * scratch_stride;
    const uint64_t* hi = lo + ((size_t)F::NW << n_lo);
    uint64_t* out = out_all + (size_t)blockIdx.y * out_stride;
    const size_t lo_size = (size_t)1 << n_lo, rows = n >> n_lo;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const typename F::Pre h = F::pre(F::load(hi, row));
        for (size_t j = threadIdx.x; j < lo_size; j += blockDim.x)
            F::store(out, row * lo_size + j, F::mul_pre(h, F::load(lo, j)));
    }
}
template <class F>
inline int build_batched(const uint64_t* d_r, size_t r_stride, uint64_t* d_out, size_t out_stride, uint64_t* d_scratch, int log_n,
                         int count, cudaStream_t st) {
    if (count < 1 || count > 65535) return MB_ERR_ARG;
    if (log_n <= 12) {
        for (int t = 0; t < count; t++) {
            int rc = build<F>(d_r + (size_t)t * r_stride, d_out + (size_t)t * out_stride, nullptr, log_n, st);
            if (rc != MB_OK) return rc;
        }
        return MB_OK;
    }
    if (!d_scratch || !d_r || !d_out) return MB_ERR_ARG;
    const int n_lo = log_n / 2, n_hi = log_n - n_lo;
    const size_t scratch_stride = ((size_t)F::NW << n_lo) + ((size_t)F::NW << n_hi);
    const size_t n = (size_t)1 << log_n;
    {
        MB_KERNEL_ON("small_tables", st);
        small_tables_batched_kernel<F><<<2 * count, 1024, 0, st>>>(d_r, r_stride, n_lo, n_hi, d_scratch, scratch_stride);
    }
    {
        MB_KERNEL_ON("outer_product", st);
        int per_leaf = grid_for((n >> n_lo) * 256, 256, 8) / count;
        if (per_leaf < 8) per_leaf = 8;
        dim3 grid(per_leaf, count);
        outer_product_batched_kernel<F><<<grid, 256, 0, st>>>(d_scratch, scratch_stride, n_lo, d_out, out_stride, n);
    }
    return finish_async();
}

}  // namespace eq
}  // namespace mb
