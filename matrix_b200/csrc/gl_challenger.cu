// Fiat-Shamir challenger on the device: n independent duplex sponges over
// Poseidon2 (width 8, rate 4, overwrite mode, LIFO output buffer), one thread
// per transcript. Reference: cuda/challenger.cuh:42-366 (state and semantics),
// declarations goldilocks-cuda-rs/src/ffi.rs:315-371, definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:1004-1110. The state layout (136 bytes) is
// the reference's DuplexChallengerState so that states copied to the host keep
// their meaning; all words are kept canonical.
#include "common.cuh"
#include "gl_poseidon2.cuh"

using namespace mb;

namespace {

struct ChallengerState {
    uint64_t sponge[8];
    uint64_t in_buf[4];
    uint64_t out_buf[4];
    int in_count;
    int out_count;
};
static_assert(sizeof(ChallengerState) == 136, "layout of cuda/challenger.cuh:42-49");

__device__ __forceinline__ void duplexing(ChallengerState& s) {
#pragma unroll
    for (int i = 0; i < 4; i++) s.sponge[i] = i < s.in_count ? s.in_buf[i] : 0;
    s.in_count = 0;
    gl::poseidon2_permute(s.sponge);
#pragma unroll
    for (int i = 0; i < 8; i++) s.sponge[i] = gl::canon(s.sponge[i]);
#pragma unroll
    for (int i = 0; i < 4; i++) s.out_buf[3 - i] = s.sponge[i];
    s.out_count = 4;
}
__device__ __forceinline__ void observe(ChallengerState& s, uint64_t v) {
    s.out_count = 0;
#pragma unroll
    for (int i = 0; i < 4; i++)
        if (i == s.in_count) s.in_buf[i] = gl::canon(v);
    s.in_count++;
    if (s.in_count == 4) duplexing(s);
}
__device__ __forceinline__ uint64_t sample(ChallengerState& s) {
    if (s.out_count == 0) duplexing(s);
    s.out_count--;
    uint64_t v = 0;
#pragma unroll
    for (int i = 0; i < 4; i++)
        if (i == s.out_count) v = s.out_buf[i];
    return v;
}

__global__ void init_kernel(ChallengerState* st, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    ChallengerState s;
    for (int k = 0; k < 8; k++) s.sponge[k] = 0;
    for (int k = 0; k < 4; k++) { s.in_buf[k] = 0; s.out_buf[k] = 0; }
    s.in_count = 0;
    s.out_count = 0;
    st[i] = s;
}
// values[i * count + k]
__global__ void observe_kernel(ChallengerState* st, const uint64_t* __restrict__ values, int count, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    ChallengerState s = st[i];
    for (int k = 0; k < count; k++) observe(s, values[(size_t)i * count + k]);
    st[i] = s;
}
// out[i * count + k]
__global__ void sample_kernel(ChallengerState* st, uint64_t* __restrict__ out, int count, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    ChallengerState s = st[i];
    for (int k = 0; k < count; k++) out[(size_t)i * count + k] = sample(s);
    st[i] = s;
}

int run_observe(void* d_states, const uint64_t* d_values, int count, int n) {
    if (!d_states || !d_values || n < 0 || count < 0) return MB_ERR_ARG;
    if (n == 0 || count == 0) return MB_OK;
    {
        MB_KERNEL("challenger_observe");
        observe_kernel<<<(n + 127) / 128, 128, 0, MB_STREAM>>>(static_cast<ChallengerState*>(d_states), d_values, count, n);
    }
    return finish_sync();
}
int run_sample(void* d_states, uint64_t* d_out, int count, int n) {
    if (!d_states || !d_out || n < 0 || count < 0) return MB_ERR_ARG;
    if (n == 0 || count == 0) return MB_OK;
    {
        MB_KERNEL("challenger_sample");
        sample_kernel<<<(n + 127) / 128, 128, 0, MB_STREAM>>>(static_cast<ChallengerState*>(d_states), d_out, count, n);
    }
    return finish_sync();
}

}  // namespace

extern "C" {

int challenger_state_size() { return (int)sizeof(ChallengerState); }

// The one entry point of the library that returns memory it allocated
// (as in the reference); release it with cuda_free.
int challenger_alloc_states(void** d_states, int n) {
    if (!d_states || n < 0) return MB_ERR_ARG;
    return cudaMalloc(d_states, (size_t)(n > 0 ? n : 1) * sizeof(ChallengerState)) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int challenger_init_states(void* d_states, int n) {
    if (!d_states || n < 0) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL("challenger_init");
        init_kernel<<<(n + 127) / 128, 128, 0, MB_STREAM>>>(static_cast<ChallengerState*>(d_states), n);
    }
    return finish_sync();
}
int challenger_observe_ffi(void* d_states, const uint64_t* d_values, int n) { return run_observe(d_states, d_values, 1, n); }
int challenger_observe_slice_ffi(void* d_states, const uint64_t* d_values, int count, int n) {
    return run_observe(d_states, d_values, count, n);
}
int challenger_observe_ext2_ffi(void* d_states, const uint64_t* d_values, int n) { return run_observe(d_states, d_values, 2, n); }
int challenger_sample_ffi(void* d_states, uint64_t* d_outputs, int n) { return run_sample(d_states, d_outputs, 1, n); }
int challenger_sample_array_ffi(void* d_states, uint64_t* d_outputs, int count, int n) {
    return run_sample(d_states, d_outputs, count, n);
}
int challenger_sample_ext2_ffi(void* d_states, uint64_t* d_outputs, int n) { return run_sample(d_states, d_outputs, 2, n); }
int challenger_sample_ext5_ffi(void* d_states, uint64_t* d_outputs, int n) { return run_sample(d_states, d_outputs, 5, n); }
int challenger_copy_state_to_host(void* h_state, const void* d_state) {
    if (!h_state || !d_state) return MB_ERR_ARG;
    MB_CUDA(cudaMemcpyAsync(h_state, d_state, sizeof(ChallengerState), cudaMemcpyDeviceToHost, MB_STREAM));
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
int challenger_copy_state_to_device(void* d_state, const void* h_state) {
    if (!h_state || !d_state) return MB_ERR_ARG;
    MB_CUDA(cudaMemcpyAsync(d_state, h_state, sizeof(ChallengerState), cudaMemcpyHostToDevice, MB_STREAM));
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}

}  // extern "C"
