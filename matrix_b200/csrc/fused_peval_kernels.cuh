// Fused bit-permutation + partial evaluation:
//   out[j] = sum_{b < 2^m} evals[perm(j 2^m + b)] * eq[b],   perm(x) = lo_lut[x & (2^half - 1)] | hi_lut[x >> half]
// with base-field evaluations and an extension-field eq table (reference:
// cuda/fused_permute_peval.cuh:31-120, almost twin
// cuda_almost_goldilocks/almost_fused_permute_peval.cuh:23; LUT construction
// almost-goldilocks-cuda-rs/src/partial_eval.rs:283-321). One block per output,
// the two look-up tables staged in shared memory when they fit (up to 200 KB),
// otherwise read through L2.
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
        for (uint32_t b = threadIdx.x; b < inner; b += blockDim.x) {
            uint32_t x = base + b;
            uint64_t v = evals[lo[x & lo_mask] | hi[x >> half]];
            typename FE::T e = FE::load(eq_table, b);
            acc = FE::add(acc, typename FE::T{FB::mul(e.c0, v), FB::mul(e.c1, v)});
        }
        uint64_t w[2] = {acc.c0, acc.c1};
        sc::block_sum_store<2>(w, out + 2 * (size_t)j, typename FE::WordAdd(), typename FE::WordCanon());
        __syncthreads();
    }
}

template <class FB, class FE>
inline int launch(const uint64_t* d_evals, uint64_t* d_output, const uint64_t* d_eq_table, const uint32_t* d_lo_lut,
                  const uint32_t* d_hi_lut, int n, int m, int half, int output_size, cudaStream_t st) {
    if (!d_evals || !d_output || !d_eq_table || !d_lo_lut || !d_hi_lut) return MB_ERR_ARG;
    if (n < 1 || n > 31 || m < 0 || m > n || half < 0 || half > n || output_size < 1 || output_size > (1 << (n - m)))
        return MB_ERR_ARG;
    size_t lut_bytes = ((size_t)(1 << half) + ((size_t)1 << (n - half))) * sizeof(uint32_t);
    int grid = output_size < sm_count() * 8 ? output_size : sm_count() * 8;
    MB_KERNEL_ON("fused_permute_peval", st);
    if (lut_bytes <= 200 * 1024) {
        auto k = fused_permute_peval_kernel<FB, FE, true>;
        if (lut_bytes > 48 * 1024 &&
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lut_bytes) != cudaSuccess)
            return MB_ERR_CUDA;
        k<<<grid, 256, lut_bytes, st>>>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut, n, m, half, output_size);
    } else {
        fused_permute_peval_kernel<FB, FE, false><<<grid, 256, 0, st>>>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut,
                                                                         n, m, half, output_size);
    }
    return finish_async();
}

}  // namespace fp
}  // namespace mb
