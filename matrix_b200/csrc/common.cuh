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

// Scratch and result buffers the library allocates for itself come from the
// device's stream-ordered pool on the caller's stream. The pool keeps freed
// memory (release threshold raised once per device), so repeated calls reuse
// their buffers instead of paying cudaMalloc / cudaFree every time; the role of
// the caching allocator in almost-goldilocks-cuda-rs/cuda/wrapper.cu:145-235.
inline void pool_setup_once() {
    static thread_local int ready_dev = -1;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev == ready_dev) return;
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
        unsigned long long keep = ~0ULL;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    ready_dev = dev;
}
inline cudaError_t pool_alloc(void** p, size_t bytes) {
    pool_setup_once();
    return cudaMallocAsync(p, bytes, MB_STREAM);
}
inline void pool_free(void* p) {
    if (p) cudaFreeAsync(p, MB_STREAM);
}

// Small pinned host landing zone, one per host thread, for results that are
// read back every round (round polynomials, roots).
inline uint64_t* pinned_scratch() {
    struct Holder {
        uint64_t* p = nullptr;
        ~Holder() { if (p) cudaFreeHost(p); }
    };
    static thread_local Holder h;
    if (!h.p && cudaMallocHost(&h.p, 64 * sizeof(uint64_t)) != cudaSuccess) h.p = nullptr;
    return h.p;
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
