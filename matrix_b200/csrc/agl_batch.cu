// C-ABI: element-wise batch operations over almost-Goldilocks and its quadratic
// extension that the first wrapper file does not hold (reference:
// almost-goldilocks-cuda-rs/src/ffi.rs:103-138,687; definitions in
// almost-goldilocks-cuda-rs/cuda/wrapper.cu), and the stream / copy helpers of
// ffi.rs:77-100,342-350.
#include "batch_ops.cuh"
#include "agl_field.cuh"
#include <cstring>
#include <mutex>

using namespace mb;
using namespace mb::bo;
MB_FIELD_ADAPTER(AglF, agl);

extern "C" {

int agl_batch_div_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_base<AglF, DIV>("agl_batch", a, b, r, n); }
int agl_batch_neg_ffi(const uint64_t* a, uint64_t* r, int n) { return run_base<AglF, NEG>("agl_batch", a, nullptr, r, n); }
int agl_batch_square_ffi(const uint64_t* a, uint64_t* r, int n) { return run_base<AglF, SQUARE>("agl_batch", a, nullptr, r, n); }
int agl_batch_double_ffi(const uint64_t* a, uint64_t* r, int n) { return run_base<AglF, DOUBLE>("agl_batch", a, nullptr, r, n); }
int agl_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* a, uint64_t* r, int n) {
    return run_base<AglF, MUL_SCALAR>("agl_batch", a, nullptr, r, n, scalar);
}
int agl_batch_exp_ffi(const uint64_t* a, uint64_t exp, uint64_t* r, int n) { return run_base<AglF, EXP>("agl_batch", a, nullptr, r, n, exp); }

int aext2_batch_add_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_ext<AglF, ADD>("aext2_batch", a, b, r, n); }
int aext2_batch_sub_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_ext<AglF, SUB>("aext2_batch", a, b, r, n); }
int aext2_batch_neg_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<AglF, NEG>("aext2_batch", a, nullptr, r, n); }
int aext2_batch_square_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<AglF, SQUARE>("aext2_batch", a, nullptr, r, n); }
int aext2_batch_frobenius_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<AglF, CONJ>("aext2_batch", a, nullptr, r, n); }
int aext2_batch_conjugate_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<AglF, CONJ>("aext2_batch", a, nullptr, r, n); }
int aext2_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* a, uint64_t* r, int n) {
    return run_ext<AglF, MUL_SCALAR>("aext2_batch", a, nullptr, r, n, scalar);
}
int aext2_batch_exp_ffi(const uint64_t* a, uint64_t exp, uint64_t* r, int n) { return run_ext<AglF, EXP>("aext2_batch", a, nullptr, r, n, exp); }
int aext2_scale_accumulate_ffi(uint64_t scalar_c0, uint64_t scalar_c1, const uint64_t* src, uint64_t* acc, int n) {
    return run_ext<AglF, SCALE_ACC>("aext2_batch", src, nullptr, acc, n, scalar_c0, scalar_c1);
}

int agl_to_aext2_batch_ffi(const uint64_t* input, uint64_t* output, int n) { return run_lift<AglF>(input, output, n); }
int aext2_to_agl_batch_ffi(const uint64_t* input, uint64_t* output, int n) { return run_project<AglF>(input, output, n); }
int agl_zero_buffer_ffi(uint64_t* d_buf, size_t n) { return run_zero(d_buf, n); }
int agl_bit_permute_ffi(const uint64_t* d_input, uint64_t* d_output, const int* d_perm_map, int n_bits, int total) {
    return run_bit_permute(d_input, d_output, d_perm_map, n_bits, total);
}

// ---- streams, copies between devices, pool (ffi.rs:77-100,342-350) ----
const char* agl_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }
int cuda_memset(void* dst, int value, size_t size) {
    if (!dst && size) return MB_ERR_ARG;
    if (cudaMemsetAsync(dst, value, size, MB_STREAM) != cudaSuccess) return MB_ERR_CUDA;
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
// Synchronises the caller's own (per-thread) stream only.
int cuda_sync_mine() { return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_stream_create(void** stream) {
    if (!stream) return MB_ERR_ARG;
    cudaStream_t s;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return MB_ERR_CUDA;
    *stream = s;
    return MB_OK;
}
int cuda_stream_destroy(void* stream) { return cudaStreamDestroy((cudaStream_t)stream) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_stream_synchronize(void* stream) { return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_memcpy_dtod_async(void* dst, const void* src, size_t size, void* stream) {
    return cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToDevice, (cudaStream_t)stream) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int cuda_memcpy_htod_async(void* dst, const void* src, size_t size, void* stream) {
    return cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, (cudaStream_t)stream) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
// Works with or without peer access (staged through the host when there is none).
int cuda_memcpy_peer(void* dst, int dst_dev, const void* src, int src_dev, size_t size) {
    return cudaMemcpyPeer(dst, dst_dev, src, src_dev, size) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
// From the current device to `peer`; already enabled counts as success.
int cuda_enable_peer_access(int peer) {
    cudaError_t err = cudaDeviceEnablePeerAccess(peer, 0);
    if (err == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return MB_OK; }
    if (err != cudaSuccess) { cudaGetLastError(); return MB_ERR_CUDA; }
    return MB_OK;
}
// Hands memory cached by the stream-ordered pool and by cuda_malloc's block cache back to the driver.
int mb_alloc_cache_flush();
int cuda_pool_trim(size_t min_bytes_to_keep) {
    mb_alloc_cache_flush();
    int dev = 0;
    cudaMemPool_t pool;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetDefaultMemPool(&pool, dev) != cudaSuccess) return MB_ERR_CUDA;
    return cudaMemPoolTrimTo(pool, min_bytes_to_keep) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
// Bytes the pool holds beyond what is in use (the role of the reference's allocator cache counter).
size_t agl_cached_bytes() {
    int dev = 0;
    cudaMemPool_t pool;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetDefaultMemPool(&pool, dev) != cudaSuccess) return 0;
    unsigned long long reserved = 0, used = 0;
    if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved) != cudaSuccess) return 0;
    if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &used) != cudaSuccess) return 0;
    return reserved > used ? (size_t)(reserved - used) : 0;
}

// Pageable host memory <-> device through two pinned 64 MiB buffers per device, so the
// DMA of one chunk overlaps the host copy of the next (ffi.rs:63-64). dir 0: device to host.
static int staged_copy(void* dst, const void* src, size_t bytes, int dir) {
    if (bytes == 0) return MB_OK;
    if (!dst || !src) return MB_ERR_ARG;
    constexpr size_t CH = (size_t)64 << 20;
    constexpr int MAX_DEV = 16;
    struct Lane {
        std::mutex mx;
        void* buf[2] = {nullptr, nullptr};
        cudaEvent_t ev[2];
        cudaStream_t st = nullptr;
    };
    static Lane lanes[MAX_DEV];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MB_ERR_CUDA;
    if (dev < 0 || dev >= MAX_DEV)
        return cudaMemcpy(dst, src, bytes, dir ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    Lane& L = lanes[dev];
    std::lock_guard<std::mutex> lk(L.mx);
    if (!L.st) {
        for (int k = 0; k < 2; k++) {
            if (cudaMallocHost(&L.buf[k], CH) != cudaSuccess) return MB_ERR_CUDA;
            if (cudaEventCreateWithFlags(&L.ev[k], cudaEventDisableTiming) != cudaSuccess) return MB_ERR_CUDA;
        }
        if (cudaStreamCreateWithFlags(&L.st, cudaStreamNonBlocking) != cudaSuccess) return MB_ERR_CUDA;
    }
    if (cudaStreamSynchronize(MB_STREAM) != cudaSuccess) return MB_ERR_CUDA;  // the data was produced on the caller's stream
    const size_t chunks = (bytes + CH - 1) / CH;
    auto len = [&](size_t c) { return c + 1 < chunks ? CH : bytes - c * CH; };
    if (dir == 0) {
        for (size_t c = 0; c <= chunks; c++) {
            if (c < chunks) {
                if (cudaMemcpyAsync(L.buf[c & 1], (const char*)src + c * CH, len(c), cudaMemcpyDeviceToHost, L.st) != cudaSuccess) return MB_ERR_CUDA;
                cudaEventRecord(L.ev[c & 1], L.st);
            }
            if (c > 0) {
                if (cudaEventSynchronize(L.ev[(c - 1) & 1]) != cudaSuccess) return MB_ERR_CUDA;
                std::memcpy((char*)dst + (c - 1) * CH, L.buf[(c - 1) & 1], len(c - 1));
            }
        }
    } else {
        for (size_t c = 0; c < chunks; c++) {
            if (c >= 2 && cudaEventSynchronize(L.ev[c & 1]) != cudaSuccess) return MB_ERR_CUDA;  // buffer free again
            std::memcpy(L.buf[c & 1], (const char*)src + c * CH, len(c));
            if (cudaMemcpyAsync((char*)dst + c * CH, L.buf[c & 1], len(c), cudaMemcpyHostToDevice, L.st) != cudaSuccess) return MB_ERR_CUDA;
            cudaEventRecord(L.ev[c & 1], L.st);
        }
        if (cudaStreamSynchronize(L.st) != cudaSuccess) return MB_ERR_CUDA;
    }
    return MB_OK;
}
int agl_d2h_staged(void* h_dst, const void* d_src, size_t bytes) { return staged_copy(h_dst, d_src, bytes, 0); }
int agl_h2d_staged(void* d_dst, const void* h_src, size_t bytes) { return staged_copy(d_dst, h_src, bytes, 1); }

}  // extern "C"
