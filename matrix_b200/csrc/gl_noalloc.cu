// A sumcheck round message that allocates nothing.
//
// Some hosts cannot let this library allocate: a prover that has handed every
// byte of device memory to its own arena at start-up, or a service loop that
// must never take the driver's allocation lock (cudaMalloc and cudaFree
// serialise against the whole device). The other entry points that finish
// their reduction on the device need a scratch buffer for per-block partial
// sums from somewhere. This one keeps that scratch in a fixed array that is
// part of the library image, so the call itself creates and frees nothing.
//
// The price is a fixed size and shared state: the array (about 85 KB) is
// resident on every GPU that loads the library until the process exits, every
// call on a device uses the same array, and two calls that overlap on the GPU
// (different streams or host threads) would overwrite each other's partial
// sums. Callers must serialise calls per device.
//
// Two conditions on "allocates nothing": the library's per-kernel timing must
// be off (mb_prof_enable(0), the default), because with it on every launch
// creates two CUDA events; and the array's address, looked up once per device
// and cached for the life of the process, does not survive a cudaDeviceReset
// of that device.
#include "gl_sumcheck_launch.cuh"
#include <mutex>

using namespace mb;
using namespace mb::sc;

namespace {

// Partial rows for at most NOALLOC_MAX_BLOCKS blocks of (MAX_D + 1) extension
// elements, followed by the ticket counter of the last-block reduction.
constexpr int NOALLOC_MAX_BLOCKS = 592;  // 4 blocks on each of 148 SMs
constexpr size_t NOALLOC_PARTIAL_WORDS = (size_t)NOALLOC_MAX_BLOCKS * (MAX_D + 1) * 2;
constexpr size_t NOALLOC_SCRATCH_WORDS = NOALLOC_PARTIAL_WORDS + 32;  // counter lives in the tail
// Largest table the entry point accepts: 2^30 pairs per table (tables of 2^31
// extension elements, 32 GiB each) -- far beyond one GPU, so in practice the
// limit that bites is d <= 8.
constexpr size_t NOALLOC_MAX_HALF = (size_t)1 << 30;

static __device__ __align__(256) uint64_t g_noalloc_scratch[NOALLOC_SCRATCH_WORDS];

// In host code the array's name is only a handle for the runtime, not a device
// address. The address is asked for once per device, with that device current.
constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
uint64_t* g_scratch_addr[MAX_DEVICES] = {nullptr};

int scratch_for_current_device(uint64_t** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MB_ERR_CUDA;
    if (dev < 0 || dev >= MAX_DEVICES) return MB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return MB_ERR_CUDA;
        g_scratch_addr[dev] = static_cast<uint64_t*>(p);
    }
    *out = g_scratch_addr[dev];
    return MB_OK;
}

}  // namespace

extern "C" {

// Whole round message of the extension-field sumcheck, no allocation.
//
//   d_polys    d tables, poly-major, `original_size` extension elements each
//   d_message  out: the d + 1 evaluations P(0..d), canonical, (c0, c1) each
//   half       live length / 2
//
// Same sums as sumcheck_round_message_ext2_ffi followed by adding up its
// partial rows. Returns 0; -2 for bad pointers or d outside 1..8; -3 when
// half exceeds 2^30 (the stated maximum) or the device index is above 63; -1
// on a CUDA error. The first call on each device looks up the scratch array's
// address; make that first call before any stream capture. Calls on one device
// must not overlap: they share the scratch, which keeps the previous call's
// partial sums (every row that is read is rewritten first, and the counter is
// cleared at the start of every call).
int sumcheck_round_message_ext2_noalloc_ffi(const uint64_t* d_polys, uint64_t* d_message, int d, size_t original_size,
                                            size_t half) {
    if (!d_polys || !d_message || d < 1 || d > MAX_D) return MB_ERR_ARG;
    if (half > NOALLOC_MAX_HALF) return MB_ERR_UNSUPPORTED;
    uint64_t* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != MB_OK) return rc;
    unsigned int* counter = reinterpret_cast<unsigned int*>(scratch + NOALLOC_PARTIAL_WORDS);
    MB_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned int), MB_STREAM));
    size_t need = (half + BLOCK - 1) / BLOCK;
    int blocks = (int)(need < (size_t)NOALLOC_MAX_BLOCKS ? (need ? need : 1) : (size_t)NOALLOC_MAX_BLOCKS);
    rc = launch_round_message<GlExt2>(d_polys, scratch, d, original_size, half, blocks, MB_STREAM, counter, d_message);
    return rc != MB_OK ? rc : finish_sync();
}

}  // extern "C"
