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
int commit_scalar(const uint32_t* d_key, const void* d_z, uint64_t N, int planes, uint64_t col_offset, uint64_t* d_out,
                  const uint64_t* d_premat = nullptr) {
    if ((!d_key && !d_premat) || !d_z || !d_out || planes < 1 || planes > 64) return MB_ERR_ARG;
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
        commit_scalar_kernel<KIND><<<grid, 384, 0, MB_STREAM>>>(d_key, d_z, N, col_offset, cpc, partial, d_premat);
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

}  // extern "C"

namespace {
constexpr int TC_PASS_PLANES = TC_MAX_PLANES;   // one MMA covers all planes of a pass: N = 64 np <= 256

template <int SRC, int NP>
int launch_tc_np(const uint32_t* d_key, const uint64_t* d_M, const uint8_t* d_T, const int8_t* d_digits, uint64_t N, int p0,
                 uint64_t col_offset, uint64_t* partial, int* d_err, uint8_t* materialize, size_t chunks, int chunk_cols) {
    dim3 grid((unsigned)chunks, 3);
    if (materialize) {   // the matrix as byte planes in operand order: the builder of the single-phase kernel, no MMAs
        const size_t smem = tc_pipe_smem_bytes(NP);
        if (cudaFuncSetAttribute(commit_tc_pipe_kernel<SRC, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return MB_ERR_CUDA;
        commit_tc_pipe_kernel<SRC, NP><<<grid, TCP_THREADS, smem, MB_STREAM>>>(d_key, d_M, d_T, d_digits, N, p0, col_offset, partial, d_err,
                                                                                 materialize, chunk_cols);
        return MB_OK;
    }
    const size_t smem = tc_ws_smem_bytes(SRC, NP);
    if (cudaFuncSetAttribute(commit_tc_ws_kernel<SRC, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return MB_ERR_CUDA;
    commit_tc_ws_kernel<SRC, NP><<<grid, ws_threads(SRC), smem, MB_STREAM>>>(d_key, d_M, d_T, d_digits, N, p0, col_offset, partial, d_err, chunk_cols);
    return MB_OK;
}
// Columns per CTA (a multiple of the four columns of an MMA stage, at most 512): one CTA runs per SM at a time
// and a grid has three CTAs per chunk, so the chunk width is chosen to make the grid a whole number of waves:
// as few waves as 512-column chunks allow (two at least, so that a short witness still spreads over every SM),
// then the widest chunks that fill them. 2^18 columns: 542 chunks of 484 columns = 1626 CTAs = 10.99 waves of
// 148 instead of 512 chunks = 10.4 waves, of which the last is two fifths full.
inline int tc_chunk_cols(uint64_t N) {
    const uint64_t sms = (uint64_t)sm_count();
    const uint64_t min_chunks = (N + TC_CHUNK_COLS - 1) / TC_CHUNK_COLS;
    uint64_t waves = (3 * min_chunks + sms - 1) / sms;
    if (waves < 2) waves = 2;
    uint64_t want_chunks = waves * sms / 3;
    if (want_chunks < 1) want_chunks = 1;
    uint64_t cols = (N + want_chunks - 1) / want_chunks;
    cols = (cols + TC_STAGE_COLS - 1) / TC_STAGE_COLS * TC_STAGE_COLS;
    if (cols < TC_CHUNK_MIN) cols = TC_CHUNK_MIN;
    if (cols > TC_CHUNK_COLS) cols = TC_CHUNK_COLS;
    return (int)cols;
}
template <int SRC>
int launch_tc(const uint32_t* d_key, const uint64_t* d_M, const uint8_t* d_T, const int8_t* d_digits, uint64_t N, int p0, int np,
              uint64_t col_offset, uint64_t* partial, int* d_err, uint8_t* materialize, size_t chunks, int chunk_cols) {
    switch (np) {
        case 1: return launch_tc_np<SRC, 1>(d_key, d_M, d_T, d_digits, N, p0, col_offset, partial, d_err, materialize, chunks, chunk_cols);
        case 2: return launch_tc_np<SRC, 2>(d_key, d_M, d_T, d_digits, N, p0, col_offset, partial, d_err, materialize, chunks, chunk_cols);
        case 3: return launch_tc_np<SRC, 3>(d_key, d_M, d_T, d_digits, N, p0, col_offset, partial, d_err, materialize, chunks, chunk_cols);
        default: return launch_tc_np<SRC, 4>(d_key, d_M, d_T, d_digits, N, p0, col_offset, partial, d_err, materialize, chunks, chunk_cols);
    }
}

// Signed 8-bit digit planes on the tensor cores, four planes per pass; the matrix comes from the key stream
// (d_key), from 64-bit coefficients (d_M) or from byte planes in operand order (d_T).
int commit_s8_tc(const uint32_t* d_key, const uint64_t* d_M, const uint8_t* d_T, const int8_t* d_digits, uint64_t N, int planes,
                 uint64_t col_offset, uint64_t* d_out) {
    if (!d_digits || !d_out || planes < 1 || planes > 64) return MB_ERR_ARG;
    const size_t plane_words = (size_t)KAPPA * D;
    if (N == 0) {
        MB_CUDA(cudaMemsetAsync(d_out, 0, planes * plane_words * sizeof(uint64_t), MB_STREAM));
        return finish_sync();
    }
    const int chunk_cols = tc_chunk_cols(N);
    const size_t chunks = (N + chunk_cols - 1) / chunk_cols;
    uint64_t* partial = nullptr;
    int* d_err = nullptr;
    MB_CUDA(pool_alloc((void**)&partial, chunks * 3 * TC_MAX_PLANES * TC_ROWS * D * sizeof(uint64_t)));
    if (pool_alloc((void**)&d_err, sizeof(int)) != cudaSuccess) { pool_free(partial); return MB_ERR_CUDA; }
    int rc = MB_OK;
    if (cudaMemsetAsync(d_err, 0, sizeof(int), MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
    for (int p0 = 0; p0 < planes && rc == MB_OK; p0 += TC_PASS_PLANES) {
        const int np = planes - p0 < TC_PASS_PLANES ? planes - p0 : TC_PASS_PLANES;
        {
            MB_KERNEL(d_T ? "ajtai_commit_tc_tiled" : d_M ? "ajtai_commit_tc_premat" : "ajtai_commit_tc");
            if (d_T) rc = launch_tc<TC_SRC_TILED>(nullptr, nullptr, d_T, d_digits, N, p0, np, 0, partial, d_err, nullptr, chunks, chunk_cols);
            else if (d_M) rc = launch_tc<TC_SRC_COEFFS>(nullptr, d_M, nullptr, d_digits, N, p0, np, 0, partial, d_err, nullptr, chunks, chunk_cols);
            else rc = launch_tc<TC_SRC_CHACHA>(d_key, nullptr, nullptr, d_digits, N, p0, np, col_offset, partial, d_err, nullptr, chunks, chunk_cols);
        }
        if (rc != MB_OK) break;
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
}  // namespace

extern "C" {

// Addition: the same signed-digit commit on the tensor cores (tcgen05 kind::i8).
// Digits must lie in [-127, 127] (-3 if a -128 is met: its negation, needed by
// the negacyclic wrap, is not an s8; use the scalar entry point then). Planes
// are processed four at a time.
int ajtai_commit_s8_ffi(const uint32_t* d_key, const int8_t* d_digits, uint64_t N, int planes, uint64_t col_offset,
                        uint64_t* d_out) {
    if (!d_key) return MB_ERR_ARG;
    return commit_s8_tc(d_key, nullptr, nullptr, d_digits, N, planes, col_offset, d_out);
}

// The same against a matrix materialised by ajtai_materialize_m_ffi (d_M[j][i][k], columns 0 .. N - 1): the
// tensor-core kernel streams the matrix instead of regenerating it. No reference counterpart for signed digits
// (the reference's premat entry point takes ternary planes, ajtai_commit_ternary_premat_ffi below).
int ajtai_commit_s8_premat_ffi(const uint64_t* d_M, const int8_t* d_digits, uint64_t N, int planes, uint64_t* d_out) {
    if (!d_M) return MB_ERR_ARG;
    return commit_s8_tc(nullptr, d_M, nullptr, d_digits, N, planes, 0, d_out);
}

// Additions (no reference counterpart): the matrix as byte planes in the order the tensor-core operand wants
// them. ajtai_tc_matrix_bytes(N) = size of that buffer for N columns; ajtai_materialize_tc_ffi fills it for
// columns col_offset .. col_offset + N - 1; ajtai_commit_s8_tiled_ffi commits against it (the kernel then only
// copies 28 KB per four columns and row group: its remaining work is the digit windows and the MMAs).
uint64_t ajtai_tc_matrix_bytes(uint64_t N) { return ((N + TC_STAGE_COLS - 1) / TC_STAGE_COLS) * 3 * (uint64_t)TCP_A_IMAGE; }

int ajtai_materialize_tc_ffi(const uint32_t* d_key, uint8_t* d_T, uint64_t N, uint64_t col_offset) {
    if (!d_key || (!d_T && N)) return MB_ERR_ARG;
    if (N == 0) return MB_OK;
    const int chunk_cols = tc_chunk_cols(N);
    const size_t chunks = (N + chunk_cols - 1) / chunk_cols;
    int* d_err = nullptr;
    MB_CUDA(pool_alloc((void**)&d_err, sizeof(int)));
    int rc = cudaMemsetAsync(d_err, 0, sizeof(int), MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    if (rc == MB_OK) {
        MB_KERNEL("ajtai_materialize_tc");
        rc = launch_tc<TC_SRC_CHACHA>(d_key, nullptr, nullptr, nullptr, N, 0, 1, col_offset, nullptr, d_err, d_T, chunks, chunk_cols);
    }
    if (rc == MB_OK) rc = finish_sync();
    pool_free(d_err);
    return rc;
}

int ajtai_commit_s8_tiled_ffi(const uint8_t* d_T, const int8_t* d_digits, uint64_t N, int planes, uint64_t* d_out) {
    if (!d_T) return MB_ERR_ARG;
    return commit_s8_tc(nullptr, nullptr, d_T, d_digits, N, planes, 0, d_out);
}

// Addition (measurement helper, no reference counterpart): the sustained int8 multiply-accumulate rate of the
// tensor pipes of the current device, from the commit kernel's own tcgen05 kind::i8 issue loop on operands that
// stay in shared memory (one CTA per SM, `groups` groups of eight M = 128, N = n_cols, K = 32 MMAs each). Writes
// multiply-accumulates per second. N = 256 (ajtai_tc_int8_peak_ffi) is the roofline denominator of the
// tensor-core commit; smaller N shows what the shape of an MMA costs.
int ajtai_tc_int8_peak_shape_ffi(int groups, int n_cols, int depth, double* mac_per_second) {
    if (depth < 1 || depth > PEAK_RING - 1) return MB_ERR_ARG;
    if (groups < 1 || groups > (1 << 20) || !mac_per_second || n_cols < 16 || n_cols > 256 || (n_cols & 15)) return MB_ERR_ARG;
    const size_t smem = TC_A_BYTES + 32 * (size_t)TC_SBO;
    if (cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return MB_ERR_CUDA;
    int* d_err = nullptr;
    MB_CUDA(pool_alloc((void**)&d_err, sizeof(int)));
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) { pool_free(d_err); return MB_ERR_CUDA; }
    int rc = cudaMemsetAsync(d_err, 0, sizeof(int), MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    const int grid = sm_count();
    float ms = 0.f;
    int h_err = 0;
    if (rc == MB_OK) {
        int8_peak_kernel<<<grid, 128, smem, MB_STREAM>>>(groups / 8 > 0 ? groups / 8 : 1, n_cols, depth, d_err);   // warm-up
        cudaEventRecord(a, MB_STREAM);
        {
            MB_KERNEL("int8_peak");
            int8_peak_kernel<<<grid, 128, smem, MB_STREAM>>>(groups, n_cols, depth, d_err);
        }
        cudaEventRecord(b, MB_STREAM);
        if (cudaMemcpyAsync(&h_err, d_err, sizeof(int), cudaMemcpyDeviceToHost, MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
        if (rc == MB_OK) rc = finish_sync();
        if (rc == MB_OK && cudaEventElapsedTime(&ms, a, b) != cudaSuccess) rc = MB_ERR_CUDA;
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    pool_free(d_err);
    if (rc != MB_OK) return rc;
    if (h_err != 0 || ms <= 0.f) return MB_ERR_CUDA;
    *mac_per_second = (double)grid * (double)groups * 8.0 * 128.0 * (double)n_cols * 32.0 / ((double)ms * 1e-3);
    return MB_OK;
}
int ajtai_tc_int8_peak_n_ffi(int groups, int n_cols, double* mac_per_second) { return ajtai_tc_int8_peak_shape_ffi(groups, n_cols, 6, mac_per_second); }
int ajtai_tc_int8_peak_ffi(int groups, double* mac_per_second) { return ajtai_tc_int8_peak_shape_ffi(groups, 256, 6, mac_per_second); }

// ---- ternary planes, sparse positions (ffi.rs:352-359,603-625,649-655; wrapper.cu:959-969,1642-1699,1741-1758) ----
namespace {
constexpr int SPLIT_K = 13;  // ternary planes per witness (cuda_almost_goldilocks/ajtai.cuh commit_ternary_kernel)

int expand_ternary(const uint64_t* d_pos, const uint64_t* d_neg, uint64_t N_ring, int8_t** d_digits) {
    const size_t words = (size_t)SPLIT_K * N_ring;
    if (pool_alloc((void**)d_digits, words * 64) != cudaSuccess) return MB_ERR_CUDA;
    MB_KERNEL("ajtai_ternary_expand");
    ternary_expand_kernel<<<grid_for(words * 4, 256, 8), 256, 0, MB_STREAM>>>(d_pos, d_neg, words, *d_digits);
    return finish_async();
}
}  // namespace

// 13 ternary planes: d_pos / d_neg[i * N_ring + j] are the bit masks of the +1 / -1 coefficients of ring
// element j of plane i; d_out[13][42][64]. The planes are expanded to signed digits and committed on the
// tensor cores (one matrix generation per four planes).
int ajtai_commit_ternary_ffi(const uint32_t* d_key, const uint64_t* d_pos, const uint64_t* d_neg, uint64_t N_ring, int chunk,
                             uint64_t* d_out) {
    if (!valid_chunk(chunk)) return MB_ERR_UNSUPPORTED;
    if (!d_key || !d_pos || !d_neg || !d_out) return MB_ERR_ARG;
    if (N_ring == 0) return ajtai_commit_s8_ffi(d_key, reinterpret_cast<const int8_t*>(d_pos), 0, SPLIT_K, 0, d_out);
    int8_t* d_digits = nullptr;
    int rc = expand_ternary(d_pos, d_neg, N_ring, &d_digits);
    if (rc == MB_OK) rc = ajtai_commit_s8_ffi(d_key, d_digits, N_ring, SPLIT_K, 0, d_out);
    pool_free(d_digits);
    return rc;
}

// The same against a matrix materialised by ajtai_materialize_m_ffi (d_M[j][i][k]).
int ajtai_commit_ternary_premat_ffi(const uint64_t* d_M, const uint64_t* d_pos, const uint64_t* d_neg, uint64_t N_ring,
                                    int chunk, uint64_t* d_out) {
    if (!valid_chunk(chunk)) return MB_ERR_UNSUPPORTED;
    if (!d_M || !d_pos || !d_neg || !d_out) return MB_ERR_ARG;
    if (N_ring == 0) return commit_scalar<KIND_S8>(nullptr, d_pos, 0, SPLIT_K, 0, d_out, d_M);
    int8_t* d_digits = nullptr;
    int rc = expand_ternary(d_pos, d_neg, N_ring, &d_digits);
    if (rc == MB_OK) rc = commit_s8_tc(nullptr, d_M, nullptr, d_digits, N_ring, SPLIT_K, 0, d_out);
    pool_free(d_digits);
    return rc;
}

// d_wide[n_ring][64] signed 16-bit coefficients to k_chunks ternary planes; *d_err is set when a
// coefficient does not fit k_chunks bits. More than 16 planes: -1 as in the reference.
int aext2_wide_to_ternary_ffi(const int16_t* d_wide, uint64_t* d_pos, uint64_t* d_neg, int* d_err, size_t n_ring, int k_chunks) {
    if (k_chunks > 16) return MB_ERR_CUDA;
    if (!d_wide || !d_pos || !d_neg || !d_err || k_chunks < 1) return MB_ERR_ARG;
    if (n_ring == 0) return MB_OK;
    MB_KERNEL("wide_to_ternary");
    wide_to_ternary_kernel<<<grid_for(n_ring, 128, 8), 128, 0, MB_STREAM>>>(d_wide, d_pos, d_neg, d_err, n_ring, k_chunks);
    return finish_async();
}

// K positions p in [0, 64 N): c_i = sum_p X^(p mod 64) M[i][p / 64]; d_out[42][64].
int ajtai_commit_sparse_ffi(const uint32_t* d_key, const uint64_t* d_positions, uint64_t K, int chunk, uint64_t* d_out) {
    if (!valid_chunk(chunk)) return MB_ERR_UNSUPPORTED;
    if (!d_key || !d_out || (!d_positions && K)) return MB_ERR_ARG;
    const size_t width = (size_t)KAPPA * D;
    if (K == 0) {
        MB_CUDA(cudaMemsetAsync(d_out, 0, width * sizeof(uint64_t), MB_STREAM));
        return finish_sync();
    }
    uint64_t blocks = (uint64_t)sm_count() * 4;
    if (blocks > K) blocks = K;
    const uint64_t per_chunk = (K + blocks - 1) / blocks;
    const uint64_t chunks = (K + per_chunk - 1) / per_chunk;
    uint64_t* partial = nullptr;
    MB_CUDA(pool_alloc((void**)&partial, chunks * width * sizeof(uint64_t)));
    {
        MB_KERNEL("ajtai_commit_sparse");
        commit_sparse_kernel<<<(unsigned)chunks, 384, 0, MB_STREAM>>>(d_key, d_positions, K, per_chunk, partial);
    }
    {
        MB_KERNEL("ajtai_reduce_chunks");
        reduce_chunks_kernel<<<grid_for(width, 256, 4), 256, 0, MB_STREAM>>>(partial, chunks, width, d_out);
    }
    int rc = finish_sync();
    pool_free(partial);
    return rc;
}

}  // extern "C"
