// Shared host-side helpers for the C-ABI translation units: return codes, the
// stream every call runs on, launch geometry and a block-wide modular
// reduction.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

// Return codes of every extern "C" entry point. 0 / -1 / -3 are the reference's
// (almost-goldilocks-cuda-rs/cuda/wrapper.cu:1151-1170; goldilocks-cuda-rs
// returns -1 for any CUDA error); -2 marks an argument this library rejects
// before launching anything.
#define MB_OK 0
#define MB_ERR_CUDA (-1)
#define MB_ERR_ARG (-2)
#define MB_ERR_UNSUPPORTED (-3)

// Work is issued on the calling thread's own stream, so concurrent callers on
// different host threads do not serialise on the legacy default stream
// (the reference builds with --default-stream per-thread,
// almost-goldilocks-cuda-rs/build.rs:87-88).
#define MB_STREAM cudaStreamPerThread

#define MB_CUDA(expr)                                   \
    do {                                                \
        cudaError_t _e = (expr);                        \
        if (_e != cudaSuccess) return MB_ERR_CUDA;      \
    } while (0)

#include "prof.cuh"

namespace mb {

// Launch status, then completion of the caller's stream: the reference's entry
// points return only after their result is ready.
inline int finish_sync() {
    if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
inline int finish_async() { return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_CUDA; }

// Number of SMs of the current device (148 on B200), cached per thread.
inline int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

// Grid for a grid-stride kernel: enough blocks to cover `items`, capped at
// `per_sm` resident blocks on every SM.
inline int grid_for(size_t items, int block, int per_sm) {
    size_t need = (items + block - 1) / block;
    size_t cap = (size_t)sm_count() * per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

}  // namespace mb
