// Initialisation, memory, device and timing entry points of the Goldilocks
// C-ABI (reference: goldilocks-cuda-rs/src/ffi.rs:10-27,303-308, definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:27-98).
//
// Buffers belong to the caller: it gets them from cuda_malloc and gives them
// back with cuda_free. Copies run on the calling thread's stream and return
// when done.
#include "common.cuh"
#include <cstring>

#include <cstdlib>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace mb {

class AllocCache {
public:
    static constexpr int MAX_DEV = 64;
    AllocCache() {
        const char* e = std::getenv("AGL_ALLOC_CACHE");
        on_ = !(e && e[0] == '0' && e[1] == 0);
    }
    int allocate(void** out, size_t size) {
        int dev = 0;
        if (!on_ || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV)
            return cudaMalloc(out, size) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
        const size_t want = ((size ? size : 1) + 511) & ~(size_t)511;
        Block hit{};
        bool found = false;
        {
            std::lock_guard<std::mutex> lk(mu_);
            auto& fl = free_[dev];
            auto it = fl.lower_bound(want);
            if (it != fl.end() && it->first <= want + want / 4 + ((size_t)2 << 20)) {
                hit = it->second;
                fl.erase(it);
                cached_[dev] -= hit.size;
                found = true;
            }
        }
        if (found) {
            // the previous owner's work on the block must be over before anyone touches it again
            if (cudaEventQuery(hit.ev) != cudaSuccess) {
                cudaGetLastError();
                cudaEventSynchronize(hit.ev);
            }
            std::lock_guard<std::mutex> lk(mu_);
            events_[dev].push_back(hit.ev);
            live_[hit.p] = Live{dev, hit.size};
            *out = hit.p;
            return MB_OK;
        }
        void* p = nullptr;
        if (cudaMalloc(&p, want) != cudaSuccess) {
            cudaGetLastError();  // clear the error, release what the cache holds, try once more
            flush(dev);
            if (cudaMalloc(&p, want) != cudaSuccess) {
                cudaGetLastError();
                return MB_ERR_CUDA;
            }
        }
        std::lock_guard<std::mutex> lk(mu_);
        live_[p] = Live{dev, want};
        *out = p;
        return MB_OK;
    }
    int release(void* p) {
        if (!p) return MB_OK;
        Live info{};
        cudaEvent_t ev = nullptr;
        {
            std::lock_guard<std::mutex> lk(mu_);
            auto it = live_.find(p);
            if (!on_ || it == live_.end())  // not handed out by this cache
                return cudaFree(p) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
            info = it->second;
            live_.erase(it);
            auto& pool = events_[info.dev];
            if (!pool.empty()) {
                ev = pool.back();
                pool.pop_back();
            }
        }
        int cur = info.dev;
        cudaGetDevice(&cur);
        // The event has to be recorded on the block's device; a buffer dropped while another device is
        // current (or when no event can be had) goes straight back to the driver.
        if (cur != info.dev || (!ev && cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess)) {
            if (ev) {
                std::lock_guard<std::mutex> lk(mu_);
                events_[info.dev].push_back(ev);
            }
            return cudaFree(p) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
        }
        cudaEventRecord(ev, MB_STREAM);
        std::lock_guard<std::mutex> lk(mu_);
        free_[info.dev].emplace(info.size, Block{p, info.size, ev});
        cached_[info.dev] += info.size;
        return MB_OK;
    }
    int flush_current() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return MB_ERR_CUDA;
        flush(dev);
        return MB_OK;
    }
    size_t cached_bytes_current() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 0;
        std::lock_guard<std::mutex> lk(mu_);
        return cached_[dev];
    }

private:
    struct Block {
        void* p;
        size_t size;
        cudaEvent_t ev;
    };
    struct Live {
        int dev;
        size_t size;
    };
    // Called with `dev` current (allocate) or made current by the caller (flush_current).
    void flush(int dev) {
        std::vector<Block> drop;
        {
            std::lock_guard<std::mutex> lk(mu_);
            for (auto& kv : free_[dev]) drop.push_back(kv.second);
            free_[dev].clear();
            cached_[dev] = 0;
        }
        for (auto& b : drop) {
            cudaEventSynchronize(b.ev);
            cudaFree(b.p);
            std::lock_guard<std::mutex> lk(mu_);
            events_[dev].push_back(b.ev);
        }
    }
    bool on_ = true;
    std::mutex mu_;
    std::multimap<size_t, Block> free_[MAX_DEV];
    std::vector<cudaEvent_t> events_[MAX_DEV];
    size_t cached_[MAX_DEV] = {};
    std::unordered_map<void*, Live> live_;
};

// One cache per library image, never destroyed (buffers may be dropped during process exit).
inline AllocCache& alloc_cache() {
    static AllocCache* c = new AllocCache();
    return *c;
}

}  // namespace mb

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

// cuda_malloc / cuda_free keep freed blocks for reuse, the role of the caching allocator in
// almost-goldilocks-cuda-rs/cuda/wrapper.cu:118-235: the Rust callers create and drop a DeviceBuffer around
// almost every call, and cudaMalloc / cudaFree serialise on a driver lock (cudaFree also waits for the
// device). Same contract: a request takes the smallest cached block of its device that fits and is at most
// 25 % + 2 MiB larger; when the driver is out of memory the device's cache is released and the request
// retried; AGL_ALLOC_CACHE=0 restores plain cudaMalloc / cudaFree. A freed block remembers an event
// recorded on the freeing thread's stream; it is handed out again only once that event has completed
// (checked without blocking first; the wait is rare because entry points return after their work is done).
int cuda_malloc(void** ptr, size_t size) {
    if (!ptr) return MB_ERR_ARG;
    return mb::alloc_cache().allocate(ptr, size);
}
int cuda_free(void* ptr) { return mb::alloc_cache().release(ptr); }
// Gives the current device's cached blocks back to the driver (cuda_pool_trim does this too).
int mb_alloc_cache_flush() { return mb::alloc_cache().flush_current(); }
// Bytes held in cached (free) blocks of the current device.
size_t mb_alloc_cache_bytes() { return mb::alloc_cache().cached_bytes_current(); }

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
