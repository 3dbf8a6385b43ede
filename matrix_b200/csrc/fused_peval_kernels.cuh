// Fused bit-permutation + partial evaluation:
//   out[j] = sum_{b < 2^m} evals[perm(j 2^m + b)] * eq[b],   perm(x) = lo_lut[x & (2^half - 1)] | hi_lut[x >> half]
// with base-field evaluations and an extension-field eq table (reference:
// cuda/fused_permute_peval.cuh:31-120, almost twin
// cuda_almost_goldilocks/almost_fused_permute_peval.cuh:23; LUT construction
// almost-goldilocks-cuda-rs/src/partial_eval.rs:283-321). The threads that share
// one output follow the number of terms: a block when 2^m >= 256, a group of
// 2^min(m, 5) lanes of a warp below that (one thread per output for m = 0), so
// that few fixed variables do not leave most of a block idle. The two look-up
// tables are staged in shared memory when they fit (up to 200 KB), otherwise
// read through L2. Sums are exact and canonical, so the grouping does not show
// in the result. When the number of outputs is a multiple of four, a group
// computes four consecutive outputs at once: if the permutation keeps the two
// lowest output variables as the two lowest input variables (the usual case: the
// fixed variables are moved down, the rest keeps its order), their four inputs
// are one aligned 32-byte sector, fetched with two 16-byte loads instead of four
// sectors of which one word each would be used.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace fp {

template <class FB, class FE, bool LUT_IN_SMEM>
__global__ void __launch_bounds__(256)
fused_permute_peval_kernel(const uint64_t* __restrict__ evals, uint64_t* __restrict__ out,
                           const uint64_t* __restrict__ eq_table, const uint32_t* __restrict__ lo_lut,
                           const uint32_t* __restrict__ hi_lut, int n, int m, int half, int output_size) {
    extern __shared__ uint32_t s_lut[];
    const int lo_size = 1 << half, hi_size = 1 << (n - half);
    const uint32_t* lo = lo_lut;
    const uint32_t* hi = hi_lut;
    if (LUT_IN_SMEM) {
        for (int i = threadIdx.x; i < lo_size; i += blockDim.x) s_lut[i] = lo_lut[i];
        for (int i = threadIdx.x; i < hi_size; i += blockDim.x) s_lut[lo_size + i] = hi_lut[i];
        __syncthreads();
        lo = s_lut;
        hi = s_lut + lo_size;
    }
    const uint32_t lo_mask = (uint32_t)lo_size - 1;
    const uint32_t inner = 1u << m;
    for (int j = blockIdx.x; j < output_size; j += gridDim.x) {
        typename FE::T acc = FE::zero();
        const uint32_t base = (uint32_t)j << m;
        // four gathers in flight per thread (m >= 10 gives every thread at least four terms), and the
        // products summed exactly: one reduction per thread and output instead of one per term
        gl::Acc s0 = gl::acc_zero(), s1 = gl::acc_zero();
        uint32_t b = threadIdx.x, pending = 0;
        for (; b + 3 * 256 < inner; b += 4 * 256) {
            uint64_t v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                uint32_t x = base + b + u * 256;
                v[u] = evals[lo[x & lo_mask] | hi[x >> half]];
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                typename FE::T e = FE::load(eq_table, b + u * 256);
                gl::acc_mul(s0, v[u], e.c0);
                gl::acc_mul(s1, v[u], e.c1);
            }
            pending += 4;
            if (pending >= 128) {   // the exact sums hold a bounded number of products
                acc = FE::add(acc, typename FE::T{FE::reduce_acc(s0), FE::reduce_acc(s1)});
                s0 = gl::acc_zero();
                s1 = gl::acc_zero();
                pending = 0;
            }
        }
        for (; b < inner; b += 256) {
            uint32_t x = base + b;
            uint64_t v = evals[lo[x & lo_mask] | hi[x >> half]];
            typename FE::T e = FE::load(eq_table, b);
            gl::acc_mul(s0, v, e.c0);
            gl::acc_mul(s1, v, e.c1);
        }
        acc = FE::add(acc, typename FE::T{FE::reduce_acc(s0), FE::reduce_acc(s1)});
        uint64_t w[2] = {acc.c0, acc.c1};
        sc::block_sum_store<2>(w, out + 2 * (size_t)j, typename FE::WordAdd(), typename FE::WordCanon());
        __syncthreads();
    }
}

// Few terms per output: groups of T = 2^log_t lanes (T <= 32) share one output.
template <class FB, class FE, bool LUT_IN_SMEM>
__global__ void __launch_bounds__(256)
fused_permute_peval_group_kernel(const uint64_t* __restrict__ evals, uint64_t* __restrict__ out,
                                 const uint64_t* __restrict__ eq_table, const uint32_t* __restrict__ lo_lut,
                                 const uint32_t* __restrict__ hi_lut, int n, int m, int half, int output_size, int log_t) {
    extern __shared__ uint32_t s_lut[];
    const int lo_size = 1 << half, hi_size = 1 << (n - half);
    const uint32_t* lo = lo_lut;
    const uint32_t* hi = hi_lut;
    if (LUT_IN_SMEM) {
        for (int i = threadIdx.x; i < lo_size; i += blockDim.x) s_lut[i] = lo_lut[i];
        for (int i = threadIdx.x; i < hi_size; i += blockDim.x) s_lut[lo_size + i] = hi_lut[i];
        __syncthreads();
        lo = s_lut;
        hi = s_lut + lo_size;
    }
    const uint32_t lo_mask = (uint32_t)lo_size - 1;
    const uint32_t inner = 1u << m, T = 1u << log_t;
    const uint32_t lane = threadIdx.x & 31, sub = lane & (T - 1), per_warp = 32u >> log_t;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const typename FE::WordAdd wadd;
    const typename FE::WordCanon wcanon;
    // whole warps iterate together: the shuffles below need every lane
    for (size_t jw = warp * per_warp; jw < (size_t)output_size; jw += warps * per_warp) {
        const size_t j = jw + (lane >> log_t);
        const bool live = j < (size_t)output_size;
        typename FE::T acc = FE::zero();
        if (live) {
            const uint32_t base = (uint32_t)j << m;
            for (uint32_t b = sub; b < inner; b += T) {
                uint32_t x = base + b;
                uint64_t v = evals[lo[x & lo_mask] | hi[x >> half]];
                typename FE::T e = FE::load(eq_table, b);
                acc = FE::add(acc, typename FE::T{FB::mul(e.c0, v), FB::mul(e.c1, v)});
            }
        }
        uint64_t w0 = acc.c0, w1 = acc.c1;
        for (uint32_t off = T >> 1; off; off >>= 1) {
            w0 = wadd(w0, __shfl_xor_sync(0xffffffffu, w0, off));
            w1 = wadd(w1, __shfl_xor_sync(0xffffffffu, w1, off));
        }
        if (live && sub == 0) *reinterpret_cast<ulonglong2*>(out + 2 * j) = make_ulonglong2(wcanon(w0), wcanon(w1));
    }
}

// Four consecutive outputs per group of T = 2^log_t lanes (output_size is a multiple of 4).
template <class FB, class FE, bool LUT_IN_SMEM>
__global__ void __launch_bounds__(256)
fused_permute_peval_quad_kernel(const uint64_t* __restrict__ evals, uint64_t* __restrict__ out,
                                const uint64_t* __restrict__ eq_table, const uint32_t* __restrict__ lo_lut,
                                const uint32_t* __restrict__ hi_lut, int n, int m, int half, int output_size, int log_t,
                                bool aligned) {
    extern __shared__ uint32_t s_lut[];
    const int lo_size = 1 << half, hi_size = 1 << (n - half);
    const uint32_t* lo = lo_lut;
    const uint32_t* hi = hi_lut;
    if (LUT_IN_SMEM) {
        for (int i = threadIdx.x; i < lo_size; i += blockDim.x) s_lut[i] = lo_lut[i];
        for (int i = threadIdx.x; i < hi_size; i += blockDim.x) s_lut[lo_size + i] = hi_lut[i];
        __syncthreads();
        lo = s_lut;
        hi = s_lut + lo_size;
    }
    const uint32_t lo_mask = (uint32_t)lo_size - 1;
    // the same for every thread: do output bits 0 and 1 come from input bits 0 and 1?
    const bool sector = aligned && (lo[(1u << m) & lo_mask] | hi[(1u << m) >> half]) == 1u &&
                        (lo[(2u << m) & lo_mask] | hi[(2u << m) >> half]) == 2u;
    const uint32_t inner = 1u << m, T = 1u << log_t;
    const uint32_t lane = threadIdx.x & 31, sub = lane & (T - 1), per_warp = 32u >> log_t;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t quads = (size_t)output_size >> 2;
    const typename FE::WordAdd wadd;
    const typename FE::WordCanon wcanon;
    for (size_t qw = warp * per_warp; qw < quads; qw += warps * per_warp) {
        const size_t q = qw + (lane >> log_t);
        const bool live = q < quads;
        uint64_t w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) w[k] = 0;
        if (live) {
            gl::Acc s[8];
#pragma unroll
            for (int k = 0; k < 8; k++) s[k] = gl::acc_zero();
            const uint32_t base = (uint32_t)(4 * q) << m;
            uint32_t pending = 0;
#pragma unroll 2
            for (uint32_t b = sub; b < inner; b += T) {
                uint64_t v[4];
                if (sector) {
                    const uint32_t x = base + b;
                    const uint64_t* p = evals + (lo[x & lo_mask] | hi[x >> half]);   // a multiple of four elements
                    const ulonglong2 u0 = *reinterpret_cast<const ulonglong2*>(p);
                    const ulonglong2 u1 = *reinterpret_cast<const ulonglong2*>(p + 2);
                    v[0] = u0.x; v[1] = u0.y; v[2] = u1.x; v[3] = u1.y;
                } else {
#pragma unroll
                    for (uint32_t t = 0; t < 4; t++) {
                        const uint32_t x = base + (t << m) + b;
                        v[t] = evals[lo[x & lo_mask] | hi[x >> half]];
                    }
                }
                const typename FE::T e = FE::load(eq_table, b);
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    gl::acc_mul(s[2 * t], v[t], e.c0);
                    gl::acc_mul(s[2 * t + 1], v[t], e.c1);
                }
                if (++pending == 128) {   // the exact sums hold a bounded number of products
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        w[k] = wadd(w[k], FE::reduce_acc(s[k]));
                        s[k] = gl::acc_zero();
                    }
                    pending = 0;
                }
            }
#pragma unroll
            for (int k = 0; k < 8; k++) w[k] = wadd(w[k], FE::reduce_acc(s[k]));
        }
        for (uint32_t off = T >> 1; off; off >>= 1) {
#pragma unroll
            for (int k = 0; k < 8; k++) w[k] = wadd(w[k], __shfl_xor_sync(0xffffffffu, w[k], off));
        }
        if (live && sub == 0) {
#pragma unroll
            for (int t = 0; t < 4; t++)
                *reinterpret_cast<ulonglong2*>(out + 2 * (4 * q + t)) = make_ulonglong2(wcanon(w[2 * t]), wcanon(w[2 * t + 1]));
        }
    }
}

template <class FB, class FE>
inline int launch(const uint64_t* d_evals, uint64_t* d_output, const uint64_t* d_eq_table, const uint32_t* d_lo_lut,
                  const uint32_t* d_hi_lut, int n, int m, int half, int output_size, cudaStream_t st) {
    if (!d_evals || !d_output || !d_eq_table || !d_lo_lut || !d_hi_lut) return MB_ERR_ARG;
    if (n < 1 || n > 31 || m < 0 || m > n || half < 0 || half > n || output_size < 1 || output_size > (1 << (n - m)))
        return MB_ERR_ARG;
    size_t lut_bytes = ((size_t)(1 << half) + ((size_t)1 << (n - half))) * sizeof(uint32_t);
    MB_KERNEL_ON("fused_permute_peval", st);
    const bool in_smem = lut_bytes <= 200 * 1024;
    // resident blocks per SM are bounded by the staged tables
    int per_sm = 8;
    if (in_smem && lut_bytes * 8 > 200 * 1024) per_sm = (int)((200 * 1024) / lut_bytes) > 0 ? (int)((200 * 1024) / lut_bytes) : 1;
    const size_t smem = in_smem ? lut_bytes : 0;
    const int log_t = m < 5 ? m : 5;
    if (output_size % 4 == 0 && m + 2 <= n) {
        auto k = in_smem ? fused_permute_peval_quad_kernel<FB, FE, true> : fused_permute_peval_quad_kernel<FB, FE, false>;
        if (smem > 40 * 1024 &&  // dynamic + static shared memory above the 48 KB default
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_CUDA;
        // every lane takes at least 16 terms when there are that many: the lanes of a warp then read
        // neighbouring sectors of the same term instead of one far-apart sector per term
        const int log_tq = m <= 4 ? 0 : (m - 4 < 5 ? m - 4 : 5);
        int grid = grid_for(((size_t)output_size >> 2) << log_tq, 256, per_sm < 4 ? per_sm : 4);
        // 16-byte loads of the inputs need a 16-byte aligned table
        const bool aligned = (reinterpret_cast<uintptr_t>(d_evals) & 15) == 0;
        k<<<grid, 256, smem, st>>>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut, n, m, half, output_size, log_tq,
                                   aligned);
    } else if (m >= 8) {
        auto k = in_smem ? fused_permute_peval_kernel<FB, FE, true> : fused_permute_peval_kernel<FB, FE, false>;
        if (smem > 40 * 1024 &&
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_CUDA;
        int grid = output_size < sm_count() * 8 ? output_size : sm_count() * 8;
        k<<<grid, 256, smem, st>>>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut, n, m, half, output_size);
    } else {
        auto k = in_smem ? fused_permute_peval_group_kernel<FB, FE, true> : fused_permute_peval_group_kernel<FB, FE, false>;
        if (smem > 40 * 1024 &&
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_CUDA;
        int grid = grid_for(((size_t)output_size) << log_t, 256, per_sm);
        k<<<grid, 256, smem, st>>>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut, n, m, half, output_size, log_t);
    }
    return finish_async();
}

}  // namespace fp
}  // namespace mb
