// Host-side launchers for the sumcheck kernels: argument checks, dispatch on the
// number of tables, launch geometry. None of them synchronises.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace sc {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Threads per block for a caller-chosen grid of `num_blocks`: enough to cover the
// work in one sweep when possible, between one warp and 1024 threads.
inline int threads_for(size_t items, int num_blocks) {
    size_t per_block = (items + (size_t)num_blocks - 1) / (size_t)num_blocks;
    int t = 32;
    while ((size_t)t < per_block && t < 1024) t <<= 1;
    return t;
}

#define MB_DISPATCH_D(d, CALL)            \
    switch (d) {                          \
        case 1: { constexpr int D = 1; CALL; } break; \
        case 2: { constexpr int D = 2; CALL; } break; \
        case 3: { constexpr int D = 3; CALL; } break; \
        case 4: { constexpr int D = 4; CALL; } break; \
        case 5: { constexpr int D = 5; CALL; } break; \
        case 6: { constexpr int D = 6; CALL; } break; \
        case 7: { constexpr int D = 7; CALL; } break; \
        case 8: { constexpr int D = 8; CALL; } break; \
        default: return MB_ERR_ARG;       \
    }

// Writes num_blocks * (d+1) partial sums; the caller adds them up (as the
// reference's GpuSumcheckState does on the host,
// goldilocks-cuda-rs/src/sumcheck_prover.rs:109-121).
template <class F>
int launch_round_message(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t stride, size_t half,
                         int num_blocks, cudaStream_t st, unsigned int* d_counter = nullptr,
                         uint64_t* d_final = nullptr) {
    if (d < 1 || d > MAX_D || num_blocks < 1 || !d_polys || !d_partial) return MB_ERR_ARG;
    if (half < 1 || 2 * half > stride) return MB_ERR_ARG;
    if (!aligned16(d_polys) || ((stride * F::NW) & 1)) return MB_ERR_ARG;
    int threads = threads_for(half, num_blocks);
    // launch bounds of round_message_kernel: 512 threads for two tables (register budget of the exact
    // sums), 1024 for three, 256 for every other count (one table included); the kernels are
    // grid-stride loops, so a smaller block only means more sweeps
    const int bound = d == 2 ? 512 : d == 3 ? 1024 : 256;
    if (threads > bound) threads = bound;
    MB_KERNEL_ON("sumcheck_round_message", st);
    MB_DISPATCH_D(d, (round_message_kernel<F, D><<<num_blocks, threads, 0, st>>>(d_polys, stride, half, d_partial,
                                                                                     d_counter, d_final)));
    return finish_async();
}

template <class F>
int launch_fold(const uint64_t* d_in, uint64_t* d_out, typename F::T r, int d, size_t stride, size_t half,
                cudaStream_t st) {
    if (d < 1 || d > MAX_D || !d_in || !d_out) return MB_ERR_ARG;
    if (half < 1 || 2 * half > stride) return MB_ERR_ARG;
    if (!aligned16(d_in) || ((stride * F::NW) & 1)) return MB_ERR_ARG;
    dim3 grid(grid_for(half, BLOCK, 8), d);
    {
        MB_KERNEL_ON("fold", st);
        fold_kernel<F><<<grid, BLOCK, 0, st>>>(d_in, d_out, r, stride, half);
    }
    return finish_async();
}

// num_blocks is both the grid and the number of partial rows written.
template <class FIn, class FOut>
int launch_fold_message(const uint64_t* d_in, uint64_t* d_out, typename FOut::T r, const uint64_t* d_r, int d,
                        size_t stride_in, size_t stride_out, size_t quarter, uint64_t* d_partial, int num_blocks,
                        cudaStream_t st, unsigned int* d_counter = nullptr, uint64_t* d_final = nullptr) {
    if (d < 1 || d > MAX_D || num_blocks < 1 || !d_in || !d_out || !d_partial) return MB_ERR_ARG;
    if (quarter < 1 || 4 * quarter > stride_in || 2 * quarter > stride_out) return MB_ERR_ARG;
    if (!aligned16(d_in) || !aligned16(d_out) || ((stride_in * FIn::NW) & 1) || ((stride_out * FOut::NW) & 1))
        return MB_ERR_ARG;
    MB_KERNEL_ON("sumcheck_fold_message", st);
    MB_DISPATCH_D(d, (fold_message_kernel<FIn, FOut, D><<<num_blocks, BLOCK, 0, st>>>(
                         d_in, d_out, r, d_r, stride_in, stride_out, quarter, d_partial, d_counter, d_final)));
    return finish_async();
}

template <class FIn, class FOut>
int launch_fold_lift(const uint64_t* d_in, uint64_t* d_out, typename FOut::T r, const uint64_t* d_r, int d,
                     size_t stride_in, size_t stride_out, size_t half, cudaStream_t st) {
    if (d < 1 || d > MAX_D || !d_in || !d_out) return MB_ERR_ARG;
    if (half < 1 || 2 * half > stride_in || half > stride_out) return MB_ERR_ARG;
    if (!aligned16(d_in) || ((stride_in * FIn::NW) & 1)) return MB_ERR_ARG;
    dim3 grid(grid_for(half, BLOCK, 8), d);
    {
        MB_KERNEL_ON("fold_lift", st);
        fold_lift_kernel<FIn, FOut><<<grid, BLOCK, 0, st>>>(d_in, d_out, r, d_r, stride_in, stride_out, half);
    }
    return finish_async();
}

// Grid used by this library's own provers for a pass over `items` work items.
inline int prover_grid(size_t items) { return grid_for(items, BLOCK, 6); }

}  // namespace sc
}  // namespace mb
