// C-ABI entry points of the almost-Goldilocks library: field batches, sumcheck,
// eq tables, partial evaluation (reference declarations
// almost-goldilocks-cuda-rs/src/ffi.rs:103-263, definitions
// almost-goldilocks-cuda-rs/cuda/wrapper.cu:330-860). Declarations:
// include/almost_goldilocks_cuda_wrapper.h.
#include "agl_traits.cuh"
#include "eq_kernels.cuh"
#include "gl_sumcheck_launch.cuh"
#include "peval_kernels.cuh"
#include "fused_peval_kernels.cuh"

using namespace mb;
using namespace mb::sc;

namespace {

enum BatchOp { OP_ADD, OP_SUB, OP_MUL, OP_INV };

template <int OP>
__global__ void agl_batch_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b, uint64_t* __restrict__ r,
                                 size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        uint64_t x = a[i], v;
        if (OP == OP_ADD) v = agl::add(x, b[i]);
        else if (OP == OP_SUB) v = agl::sub(x, b[i]);
        else if (OP == OP_MUL) v = agl::mul(x, b[i]);
        else v = agl::inv(x);
        r[i] = agl::canon(v);
    }
}

__global__ void aext2_batch_mul_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b,
                                       uint64_t* __restrict__ r, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        agl::e2_store(r + 2 * i, agl::e2_canon(agl::e2_mul(agl::e2_load(a + 2 * i), agl::e2_load(b + 2 * i))));
}

__global__ void aext2_batch_inverse_kernel(const uint64_t* __restrict__ a, uint64_t* __restrict__ r, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        agl::e2_store(r + 2 * i, agl::e2_canon(agl::e2_inv(agl::e2_load(a + 2 * i))));
}

template <int OP>
int batch(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) {
    if (n < 0 || !a || !r || (OP != OP_INV && !b)) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL("agl_batch");
        agl_batch_kernel<OP><<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(a, b, r, (size_t)n);
    }
    return finish_sync();
}

}  // namespace

extern "C" {

// wrapper.cu:111-116
int almost_goldilocks_cuda_init() {
    int n = 0;
    return (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? MB_OK : MB_ERR_CUDA;
}

int agl_batch_add_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return batch<OP_ADD>(a, b, r, n); }
int agl_batch_sub_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return batch<OP_SUB>(a, b, r, n); }
int agl_batch_mul_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return batch<OP_MUL>(a, b, r, n); }
int agl_batch_inverse_ffi(const uint64_t* a, uint64_t* r, int n) { return batch<OP_INV>(a, nullptr, r, n); }
int aext2_batch_mul_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) {
    if (n < 0 || !a || !b || !r) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL("aext2_batch_mul");
        aext2_batch_mul_kernel<<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(a, b, r, (size_t)n);
    }
    return finish_sync();
}
int aext2_batch_inverse_ffi(const uint64_t* a, uint64_t* r, int n) {
    if (n < 0 || !a || !r) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL("aext2_batch_inverse");
        aext2_batch_inverse_kernel<<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(a, r, (size_t)n);
    }
    return finish_sync();
}

// ---- sumcheck: ffi.rs:221-263 (wrapper.cu:812-860) ----
int agl_sumcheck_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                                   size_t half, int num_blocks) {
    int rc = launch_round_message<AglBase>(d_polys, d_partial, d, original_size, half, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}
int agl_sumcheck_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge, int d, size_t original_size,
                          size_t half) {
    int rc = launch_fold<AglBase>(d_input, d_output, agl::canon(challenge), d, original_size, half, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}
int aext2_sumcheck_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                                     size_t half, int num_blocks) {
    int rc = launch_round_message<AglExt2>(d_polys, d_partial, d, original_size, half, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}
int aext2_sumcheck_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t c0, uint64_t c1, int d,
                            size_t original_size, size_t half) {
    agl::E2 r{agl::canon(c0), agl::canon(c1)};
    int rc = launch_fold<AglExt2>(d_input, d_output, r, d, original_size, half, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}
// additions: fold fused with the next round's message (see the Goldilocks twins)
int aext2_sumcheck_fold_round_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t c0, uint64_t c1, int d,
                                  size_t original_size, size_t quarter, uint64_t* d_partial, int num_blocks) {
    agl::E2 r{agl::canon(c0), agl::canon(c1)};
    int rc = launch_fold_message<AglExt2, AglExt2>(d_input, d_output, r, nullptr, d, original_size, original_size,
                                                   quarter, d_partial, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}
int aext2_sumcheck_fold_round_mixed_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t c0, uint64_t c1, int d,
                                        size_t original_size, size_t quarter, uint64_t* d_partial, int num_blocks) {
    agl::E2 r{agl::canon(c0), agl::canon(c1)};
    int rc = launch_fold_message<AglBase, AglExt2>(d_input, d_output, r, nullptr, d, original_size, original_size,
                                                   quarter, d_partial, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// ---- eq tables: ffi.rs (agl_eq_dp_all_ffi, aext2_eq_dp_all_ffi) ----
int agl_eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result) {
    if (!d_result) return MB_ERR_ARG;
    int rc = eq::build<AglBase>(d_r, d_buf_a, d_buf_b, log_n, MB_STREAM);
    if (rc != MB_OK) return rc;
    *d_result = d_buf_a;
    return finish_sync();
}
int aext2_eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result) {
    if (!d_result) return MB_ERR_ARG;
    int rc = eq::build<AglExt2>(d_r, d_buf_a, d_buf_b, log_n, MB_STREAM);
    if (rc != MB_OK) return rc;
    *d_result = d_buf_a;
    return finish_sync();
}

// ---- partial evaluation: wrapper.cu:713-749 ----
// In place: the 2^(log_n - m) results end up at the start of d_data.
int agl_partial_eval_ffi(uint64_t* d_data, const uint64_t* d_r, int log_n, int m) {
    if (log_n < 0 || log_n > 40 || m < 0 || m > log_n || !d_data) return MB_ERR_ARG;
    if (m == 0) return MB_OK;
    size_t n = (size_t)1 << log_n;
    uint64_t *t0 = nullptr, *t1 = nullptr;
    MB_CUDA(pool_alloc((void**)&t0, sizeof(uint64_t) * (n >> 1)));
    if (pool_alloc((void**)&t1, sizeof(uint64_t) * (n >> 1)) != cudaSuccess) { pool_free(t0); return MB_ERR_CUDA; }
    int rc = pe::partial_eval<AglBase, AglBase>(d_data, t0, t1, d_r, log_n, m, MB_STREAM);
    if (rc == MB_OK &&
        cudaMemcpyAsync(d_data, t0, sizeof(uint64_t) << (log_n - m), cudaMemcpyDeviceToDevice, MB_STREAM) != cudaSuccess)
        rc = MB_ERR_CUDA;
    if (rc == MB_OK) rc = finish_sync();
    pool_free(t0);
    pool_free(t1);
    return rc;
}
// Base-field table in, extension challenges, extension table out.
int agl_partial_eval_ext2_from_base_ffi(const uint64_t* d_input, uint64_t* d_output, const uint64_t* d_r, int log_n,
                                        int m) {
    if (log_n < 1 || log_n > 40 || m < 1 || m > log_n || !d_input || !d_output) return MB_ERR_ARG;
    size_t n = (size_t)1 << log_n;
    uint64_t* tmp = nullptr;
    MB_CUDA(pool_alloc((void**)&tmp, 2 * sizeof(uint64_t) * (n >> 1)));
    // d_output holds 2^(log_n - 1) extension elements in the reference's contract (first layer's size)
    int rc = pe::partial_eval<AglBase, AglExt2>(d_input, d_output, tmp, d_r, log_n, m, MB_STREAM);
    if (rc == MB_OK) rc = finish_sync();
    pool_free(tmp);
    return rc;
}

// ---- fused permute + partial evaluation: wrapper.cu:755-800 ----
int agl_fused_permute_partial_eval_ffi(const uint64_t* d_evals, uint64_t* d_output, const uint64_t* d_eq_table,
                                       const uint32_t* d_lo_lut, const uint32_t* d_hi_lut, int n, int m, int half,
                                       int output_size, int smem_bytes) {
    (void)smem_bytes;
    int rc = fp::launch<AglBase, AglExt2>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut, n, m, half, output_size,
                                          MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

}  // extern "C"
