// Initialisation, memory, device and timing entry points of the Goldilocks
// C-ABI (reference: goldilocks-cuda-rs/src/ffi.rs:10-27,303-308, definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:27-98).
//
// Buffers belong to the caller: it gets them from cuda_malloc and gives them
// back with cuda_free. Copies run on the calling thread's stream and return
// when done.
#include "common.cuh"
#include <cstring>

namespace {
// out[i] = splitmix64 output number i + 1 started at `seed`, reduced mod `modulus`
// (the generator of matrix_b200/inputs.py, so device-made inputs equal host-made ones).
__global__ void fill_splitmix_kernel(uint64_t* __restrict__ out, size_t n, uint64_t seed, uint64_t modulus) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        uint64_t z = seed + (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ULL;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
        z = z ^ (z >> 31);
        out[i] = z % modulus;
    }
}
}  // namespace

extern "C" {

// Synthetic inputs made on the device (benchmarks of sizes the host should not stage).
int mb_fill_splitmix(uint64_t* d_out, size_t n, uint64_t seed, uint64_t modulus) {
    if (!d_out || modulus == 0) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    fill_splitmix_kernel<<<mb::grid_for(n, 256, 8), 256, 0, MB_STREAM>>>(d_out, n, seed, modulus);
    return mb::finish_sync();
}

// The reference uploads field and hash constants here, once per device. This
// library's tables are statically initialised __constant__ data, present on
// every device as soon as the module loads, so the calls only check that a
// device exists (and, like the reference, make device 0 current).
int goldilocks_cuda_init() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return MB_ERR_CUDA;
    MB_CUDA(cudaSetDevice(0));
    return MB_OK;
}
int poseidon2_cuda_init() {
    int n = 0;
    return (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? MB_OK : MB_ERR_CUDA;
}
int monolith_cuda_init() {
    int n = 0;
    return (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? MB_OK : MB_ERR_CUDA;
}

int cuda_malloc(void** ptr, size_t size) {
    if (!ptr) return MB_ERR_ARG;
    return cudaMalloc(ptr, size) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int cuda_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }

static int copy_sync(void* dst, const void* src, size_t size, cudaMemcpyKind kind) {
    if (size == 0) return MB_OK;
    MB_CUDA(cudaMemcpyAsync(dst, src, size, kind, MB_STREAM));
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int cuda_memcpy_htod(void* dst, const void* src, size_t size) { return copy_sync(dst, src, size, cudaMemcpyHostToDevice); }
int cuda_memcpy_dtoh(void* dst, const void* src, size_t size) { return copy_sync(dst, src, size, cudaMemcpyDeviceToHost); }
int cuda_memcpy_dtod(void* dst, const void* src, size_t size) { return copy_sync(dst, src, size, cudaMemcpyDeviceToDevice); }

int cuda_device_synchronize() { return cudaDeviceSynchronize() == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_get_last_error() { return (int)cudaGetLastError(); }
int cuda_peek_at_last_error() { return (int)cudaPeekAtLastError(); }
int cuda_mem_get_info(size_t* free_b, size_t* total_b) {
    return cudaMemGetInfo(free_b, total_b) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}

int cuda_set_device(int device) { return cudaSetDevice(device) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_get_device(int* device) { return cudaGetDevice(device) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_get_device_count(int* count) { return cudaGetDeviceCount(count) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int cuda_get_device_name(int device, char* name, int max_len) {
    if (!name || max_len <= 0) return MB_ERR_ARG;
    cudaDeviceProp prop;
    MB_CUDA(cudaGetDeviceProperties(&prop, device));
    strncpy(name, prop.name, (size_t)max_len - 1);
    name[max_len - 1] = '\0';
    return MB_OK;
}

int gl_memset_zero(uint64_t* d_buf, size_t n_u64) {
    MB_CUDA(cudaMemsetAsync(d_buf, 0, n_u64 * sizeof(uint64_t), MB_STREAM));
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}

// ---- additions -------------------------------------------------------------

// Pinned host memory for callers that stage inputs and proofs.
int mb_host_alloc(void** ptr, size_t size) { return cudaMallocHost(ptr, size) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int mb_host_free(void* ptr) { return cudaFreeHost(ptr) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }

// Asynchronous copies on the calling thread's stream (complete at mb_stream_sync
// or at any synchronising entry point called later from the same thread).
int mb_memcpy_htod_async(void* dst, const void* src, size_t size) {
    return cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int mb_memcpy_dtoh_async(void* dst, const void* src, size_t size) {
    return cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToHost, MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int mb_stream_sync() { return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }

// CUDA-event stopwatch on the calling thread's stream: the stream all of this
// library's kernels launched from that thread run on.
int mb_event_create(void** ev) {
    cudaEvent_t e;
    MB_CUDA(cudaEventCreate(&e));
    *ev = (void*)e;
    return MB_OK;
}
int mb_event_record(void* ev) { return cudaEventRecord((cudaEvent_t)ev, MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int mb_event_sync(void* ev) { return cudaEventSynchronize((cudaEvent_t)ev) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }
int mb_event_elapsed_ms(void* start, void* stop, float* ms) {
    return cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int mb_event_destroy(void* ev) { return cudaEventDestroy((cudaEvent_t)ev) == cudaSuccess ? MB_OK : MB_ERR_CUDA; }

}  // extern "C"
