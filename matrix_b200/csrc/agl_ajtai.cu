// C-ABI entry points of the Ajtai commitment (reference declarations
// almost-goldilocks-cuda-rs/src/ffi.rs:426-433,500-508,595-617, definitions
// almost-goldilocks-cuda-rs/cuda/wrapper.cu:1095-1204,1663-1670).
#include "ajtai_kernels.cuh"
#include "ajtai_tc.cuh"

using namespace mb;
using namespace mb::aj;

namespace {

// Columns per block of the scalar path: enough chunks to fill the machine.
uint64_t pick_cols_per_chunk(uint64_t N, int planes) {
    uint64_t target_blocks = (uint64_t)sm_count() * 4;
    uint64_t chunks = target_blocks / (uint64_t)planes;
    if (chunks < 1) chunks = 1;
    if (chunks > N) chunks = N;
    return (N + chunks - 1) / chunks;
}

template <int KIND>
int commit_scalar(const uint32_t* d_key, const void* d_z, uint64_t N, int planes, uint64_t col_offset, uint64_t* d_out) {
    if (!d_key || !d_z || !d_out || planes < 1 || planes > 64) return MB_ERR_ARG;
    const size_t width = (size_t)planes * KAPPA * D;
    if (N == 0) {
        MB_CUDA(cudaMemsetAsync(d_out, 0, width * sizeof(uint64_t), MB_STREAM));
        return finish_sync();
    }
    uint64_t cpc = pick_cols_per_chunk(N, planes);
    uint64_t chunks = (N + cpc - 1) / cpc;
    uint64_t* partial = nullptr;
    MB_CUDA(pool_alloc((void**)&partial, chunks * width * sizeof(uint64_t)));
    {
        MB_KERNEL("ajtai_commit_scalar");
        dim3 grid((unsigned)chunks, (unsigned)planes);
        commit_scalar_kernel<KIND><<<grid, 384, 0, MB_STREAM>>>(d_key, d_z, N, col_offset, cpc, partial);
    }
    {
        MB_KERNEL("ajtai_reduce_chunks");
        reduce_chunks_kernel<<<grid_for(width, 256, 4), 256, 0, MB_STREAM>>>(partial, chunks, width, d_out);
    }
    int rc = finish_sync();
    pool_free(partial);
    return rc;
}

bool valid_chunk(int chunk) { return chunk == 64 || chunk == 128 || chunk == 256 || chunk == 1024 || chunk == 4096; }

}  // namespace

extern "C" {

// Dense binary planes: d_z[b * N + j] is the bit mask of ring element j of
// witness b; d_out[b][i][r]. `chunk` is the reference's tuning knob: it is
// validated (-3 as in the reference) and otherwise ignored, the library sizes
// its own grid. B outside {1, 2, 4, 8, 16} returns -2 as in the reference.
int ajtai_commit_dense_batched_at_ffi(const uint32_t* d_key, const uint64_t* d_z, uint64_t N, int B, int chunk,
                                      uint64_t col_offset, uint64_t* d_out) {
    if (!valid_chunk(chunk)) return MB_ERR_UNSUPPORTED;
    if (B != 1 && B != 2 && B != 4 && B != 8 && B != 16) return MB_ERR_ARG;
    return commit_scalar<KIND_BITS>(d_key, d_z, N, B, col_offset, d_out);
}
int ajtai_commit_dense_batched_ffi(const uint32_t* d_key, const uint64_t* d_z, uint64_t N, int B, int chunk,
                                   uint64_t* d_out) {
    return ajtai_commit_dense_batched_at_ffi(d_key, d_z, N, B, chunk, 0, d_out);
}

// Wide witness: d_z_wide[j * 64 + l] field coefficients; d_out[i][r].
int ajtai_commit_wide_ffi(const uint32_t* d_key, const uint64_t* d_z_wide, uint64_t N, uint64_t col_offset, int chunk,
                          uint64_t* d_out) {
    if (!valid_chunk(chunk)) return MB_ERR_UNSUPPORTED;
    return commit_scalar<KIND_WIDE>(d_key, d_z_wide, N, 1, col_offset, d_out);
}

// M[j][i][k] for j < N.
int ajtai_materialize_m_ffi(const uint32_t* d_chacha_key, uint64_t* d_M, uint64_t N) {
    if (!d_chacha_key || !d_M) return MB_ERR_ARG;
    if (N == 0) return MB_OK;
    {
        MB_KERNEL("ajtai_materialize");
        materialize_kernel<<<grid_for(N * BLOCKS_PER_COL, 128, 16), 128, 0, MB_STREAM>>>(d_chacha_key, d_M, N, 0);
    }
    return finish_sync();
}

// Addition: signed 8-bit digit planes, d_digits[(p * N + j) * 64 + l] in
// [-128, 127]; d_out[p][i][r]. Scalar path (exact, any N).
int ajtai_commit_s8_scalar_ffi(const uint32_t* d_key, const int8_t* d_digits, uint64_t N, int planes,
                               uint64_t col_offset, uint64_t* d_out) {
    return commit_scalar<KIND_S8>(d_key, d_digits, N, planes, col_offset, d_out);
}

// Addition: the same signed-digit commit on the tensor cores (tcgen05 kind::i8).
// Digits must lie in [-127, 127] (-3 if a -128 is met: its negation, needed by
// the negacyclic wrap, is not an s8; use the scalar entry point then). Planes
// are processed four at a time.
int ajtai_commit_s8_ffi(const uint32_t* d_key, const int8_t* d_digits, uint64_t N, int planes, uint64_t col_offset,
                        uint64_t* d_out) {
    if (!d_key || !d_digits || !d_out || planes < 1 || planes > 64) return MB_ERR_ARG;
    const size_t plane_words = (size_t)KAPPA * D;
    if (N == 0) {
        MB_CUDA(cudaMemsetAsync(d_out, 0, planes * plane_words * sizeof(uint64_t), MB_STREAM));
        return finish_sync();
    }
    const size_t chunks = (N + TC_CHUNK_COLS - 1) / TC_CHUNK_COLS;
    uint64_t* partial = nullptr;
    int* d_err = nullptr;
    MB_CUDA(pool_alloc((void**)&partial, chunks * 3 * TC_MAX_PLANES * TC_ROWS * D * sizeof(uint64_t)));
    if (pool_alloc((void**)&d_err, sizeof(int)) != cudaSuccess) { pool_free(partial); return MB_ERR_CUDA; }
    int rc = MB_OK;
    if (cudaMemsetAsync(d_err, 0, sizeof(int), MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
    for (int p0 = 0; p0 < planes && rc == MB_OK; p0 += TC_MAX_PLANES) {
        int np = planes - p0 < TC_MAX_PLANES ? planes - p0 : TC_MAX_PLANES;
        size_t smem = tc_smem_bytes(np);
        if (cudaFuncSetAttribute(commit_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            rc = MB_ERR_CUDA;
            break;
        }
        {
            MB_KERNEL("ajtai_commit_tc");
            dim3 grid((unsigned)chunks, 3);
            commit_tc_kernel<<<grid, TC_THREADS, smem, MB_STREAM>>>(d_key, d_digits, N, p0, np, col_offset, partial, d_err);
        }
        {
            MB_KERNEL("ajtai_reduce_tc");
            reduce_tc_partials_kernel<<<grid_for((size_t)np * plane_words, 256, 4), 256, 0, MB_STREAM>>>(
                partial, chunks, np, d_out + (size_t)p0 * plane_words);
        }
        rc = finish_async();
    }
    int h_err = 0;
    if (rc == MB_OK && cudaMemcpyAsync(&h_err, d_err, sizeof(int), cudaMemcpyDeviceToHost, MB_STREAM) != cudaSuccess)
        rc = MB_ERR_CUDA;
    if (rc == MB_OK) rc = finish_sync();
    pool_free(partial);
    pool_free(d_err);
    if (rc != MB_OK) return rc;
    if (h_err == TC_ERR_TIMEOUT) return MB_ERR_CUDA;
    if (h_err == TC_ERR_DIGIT_RANGE) return MB_ERR_UNSUPPORTED;
    return MB_OK;
}

}  // extern "C"
