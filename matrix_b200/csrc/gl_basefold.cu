// C-ABI entry points of the Basefold path over Goldilocks and of the eq tables
// (reference declarations goldilocks-cuda-rs/src/ffi.rs:396-543, definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:1216-1590 and :2040-2110).
#include "basefold_kernels.cuh"
#include "eq_kernels.cuh"
#include "peval_kernels.cuh"
#include "fused_peval_kernels.cuh"

using namespace mb;
using namespace mb::bf;

namespace {

inline int gs(size_t items) { return grid_for(items, BLOCK, 8); }

// Applies Op on bits [first_bit, first_bit + count) of a 2^log_n array, up to
// TILE_LOG bits per pass; the first pass reads `in`, later ones run in place.
template <class Op>
int run_layers(const uint64_t* in, uint64_t* out, int log_n, int first_bit, int count, cudaStream_t st) {
    const uint64_t* src = in;
    int bit = first_bit, left = count;
    if (count == 0) {
        if (in != out)
            MB_CUDA(cudaMemcpyAsync(out, in, sizeof(uint64_t) << log_n, cudaMemcpyDeviceToDevice, st));
        return MB_OK;
    }
    const int tile_log = log_n < TILE_LOG ? log_n : TILE_LOG;
    while (left > 0) {
        // Row bits first (as many layers per pass as the tile allows), but keep
        // runs of at least 4 consecutive elements (one 32-byte sector) when the
        // rows are strided; leftover tile capacity widens the runs.
        int cmin = bit < 2 ? bit : 2;
        int nbits = left < tile_log - cmin ? left : tile_log - cmin;
        int cbits = bit < tile_log - nbits ? bit : tile_log - nbits;
        size_t tiles = (size_t)1 << (log_n - nbits - cbits);
        size_t smem = sizeof(uint64_t) << (nbits + cbits);
        int grid = (int)(tiles < (size_t)sm_count() * 4 ? tiles : (size_t)sm_count() * 4);
        {
            MB_KERNEL_ON("bit_layers", st);
            bit_layers_kernel<Op><<<grid, BLOCK, smem, st>>>(src, out, log_n, bit, nbits, cbits);
        }
        src = out;
        bit += nbits;
        left -= nbits;
    }
    return finish_async();
}

int bit_reverse_out_of_place(const uint64_t* in, uint64_t* out, int log_n, int copies, cudaStream_t st) {
    size_t n = (size_t)1 << log_n;
    if (log_n >= 12) {
        size_t tiles = (size_t)1 << (log_n - 12);
        int grid = (int)(tiles < (size_t)sm_count() * 4 ? tiles : (size_t)sm_count() * 4);
        {
            MB_KERNEL_ON("bit_reverse_tiled", st);
            bit_reverse_tiled_kernel<<<grid, 256, 0, st>>>(in, out, log_n, copies);
        }
    } else {
        {
            MB_KERNEL_ON("bit_reverse_copy", st);
            bit_reverse_copy_kernel<<<gs(n), BLOCK, 0, st>>>(in, out, log_n, copies);
        }
    }
    return finish_async();
}

}  // namespace

namespace mb {
namespace bf {

// evals -> coefficients (d_coeffs) and the bit-reversed copy of the evaluations
// (d_bh_evals); either output may be null.
int interpolate_async(const uint64_t* d_evals, uint64_t* d_coeffs, uint64_t* d_bh_evals, int nv, cudaStream_t st) {
    if (nv < 0 || nv > 32 || !d_evals) return MB_ERR_ARG;
    int rc = MB_OK;
    if (d_coeffs) rc = run_layers<InterpOp>(d_evals, d_coeffs, nv, 0, nv, st);
    if (rc == MB_OK && d_bh_evals) rc = bit_reverse_out_of_place(d_evals, d_bh_evals, nv, 1, st);
    return rc;
}

// coefficients -> codeword of 2^(nv+lr): butterflies on 2^nv elements in
// d_work (2^nv u64 of scratch, may equal d_coeffs if it can be overwritten),
// then the reversal writes the 2^lr equal blocks.
int encode_async(const uint64_t* d_coeffs, uint64_t* d_work, uint64_t* d_codeword, int nv, int lr, cudaStream_t st) {
    if (nv < 0 || lr < 0 || nv + lr > 32 || !d_coeffs || !d_work || !d_codeword) return MB_ERR_ARG;
    int rc = run_layers<CodeOp>(d_coeffs, d_work, nv, 0, nv, st);
    if (rc != MB_OK) return rc;
    return bit_reverse_out_of_place(d_work, d_codeword, nv, 1 << lr, st);
}

}  // namespace bf
}  // namespace mb

extern "C" {

int basefold_bit_reverse_gl_ffi(uint64_t* d_data, int log_n) {
    if (log_n < 0 || log_n > 40 || !d_data) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("bit_reverse_inplace", MB_STREAM);
        bit_reverse_inplace_kernel<1><<<gs((size_t)1 << log_n), BLOCK, 0, MB_STREAM>>>(d_data, log_n);
    }
    return finish_sync();
}
int basefold_bit_reverse_ext2_ffi(uint64_t* d_data, int log_n) {
    if (log_n < 0 || log_n > 40 || !d_data) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("bit_reverse_inplace", MB_STREAM);
        bit_reverse_inplace_kernel<2><<<gs((size_t)1 << log_n), BLOCK, 0, MB_STREAM>>>(d_data, log_n);
    }
    return finish_sync();
}

int basefold_bhc_interpolate_ffi(const uint64_t* d_evals, uint64_t* d_coeffs, uint64_t* d_bh_evals, int num_vars) {
    if (!d_coeffs || !d_bh_evals) return MB_ERR_ARG;
    int rc = interpolate_async(d_evals, d_coeffs, d_bh_evals, num_vars, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// The butterflies need 2^num_vars words of scratch besides the caller's two
// buffers (every block of the codeword is written from every tile of the
// reversal, so the codeword buffer cannot double as scratch); it is taken from
// the device allocator for the duration of the call.
int basefold_encode_ffi(const uint64_t* d_coeffs, uint64_t* d_codeword, int num_vars, int log_rate) {
    if (num_vars < 0 || log_rate < 0 || num_vars + log_rate > 32) return MB_ERR_ARG;
    uint64_t* work = nullptr;
    MB_CUDA(cudaMalloc(&work, sizeof(uint64_t) << num_vars));
    int rc = encode_async(d_coeffs, work, d_codeword, num_vars, log_rate, MB_STREAM);
    if (rc == MB_OK) rc = finish_sync();
    cudaFree(work);
    return rc;
}

int basefold_fold_gl_ffi(const uint64_t* d_codeword, const uint64_t* d_table, uint64_t challenge, uint64_t* d_output,
                         int pair_count) {
    if (pair_count < 1 || !d_codeword || !d_table || !d_output) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("fold_gl", MB_STREAM);
        fold_gl_kernel<<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_codeword, d_table, gl::canon(challenge), d_output, pair_count);
    }
    return finish_sync();
}
int basefold_fold_mixed_ffi(const uint64_t* d_codeword, const uint64_t* d_table, uint64_t c0, uint64_t c1,
                            uint64_t* d_output, int pair_count) {
    if (pair_count < 1 || !d_codeword || !d_table || !d_output) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("fold_mixed", MB_STREAM);
        fold_mixed_kernel<<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_codeword, d_table, gl::E2{gl::canon(c0), gl::canon(c1)},
                                                                 d_output, pair_count);
    }
    return finish_sync();
}
int basefold_fold_ext2_ffi(const uint64_t* d_codeword, const uint64_t* d_table, uint64_t c0, uint64_t c1,
                           uint64_t* d_output, int pair_count) {
    if (pair_count < 1 || !d_codeword || !d_table || !d_output) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("fold_ext2", MB_STREAM);
        fold_ext2_kernel<<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_codeword, d_table, gl::E2{gl::canon(c0), gl::canon(c1)},
                                                                d_output, pair_count);
    }
    return finish_sync();
}

int basefold_sumcheck_interp_gl_ffi(uint64_t* d_data, int pair_count) {
    if (pair_count < 1 || !d_data) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("sc_interp", MB_STREAM);
        sc_interp_kernel<1><<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_data, pair_count);
    }
    return finish_sync();
}
int basefold_sumcheck_interp_ext2_ffi(uint64_t* d_data, int pair_count) {
    if (pair_count < 1 || !d_data) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("sc_interp", MB_STREAM);
        sc_interp_kernel<2><<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_data, pair_count);
    }
    return finish_sync();
}

#define MB_PRODUCT_FFI(NAME, KERNEL)                                                                          \
    int NAME(const uint64_t* d_eq, const uint64_t* d_bh, uint64_t* p0, uint64_t* p1, uint64_t* p2, int pair_count, \
             int num_blocks) {                                                                                \
        if (pair_count < 1 || num_blocks < 1 || !d_eq || !d_bh || !p0 || !p1 || !p2) return MB_ERR_ARG;       \
        { MB_KERNEL(#KERNEL); KERNEL<<<num_blocks, BLOCK, 0, MB_STREAM>>>(d_eq, d_bh, p0, p1, p2, (size_t)pair_count); } \
        return finish_sync();                                                                                 \
    }
MB_PRODUCT_FFI(basefold_sumcheck_product_gl_ffi, sc_product_gl_kernel)
MB_PRODUCT_FFI(basefold_sumcheck_product_mixed_ffi, sc_product_mixed_kernel)
MB_PRODUCT_FFI(basefold_sumcheck_product_ext2_ffi, sc_product_ext2_kernel)

int basefold_sumcheck_eval_gl_ffi(const uint64_t* d_data, uint64_t challenge, uint64_t* d_output, int pair_count) {
    if (pair_count < 1 || !d_data || !d_output) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("sc_eval_gl", MB_STREAM);
        sc_eval_gl_kernel<<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_data, gl::canon(challenge), d_output, pair_count);
    }
    return finish_sync();
}
int basefold_sumcheck_eval_mixed_ffi(const uint64_t* d_data, uint64_t c0, uint64_t c1, uint64_t* d_output, int pair_count) {
    if (pair_count < 1 || !d_data || !d_output) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("sc_eval_mixed", MB_STREAM);
        sc_eval_mixed_kernel<<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_data, gl::E2{gl::canon(c0), gl::canon(c1)}, d_output,
                                                                    pair_count);
    }
    return finish_sync();
}
int basefold_sumcheck_eval_ext2_ffi(const uint64_t* d_data, uint64_t c0, uint64_t c1, uint64_t* d_output, int pair_count) {
    if (pair_count < 1 || !d_data || !d_output) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("sc_eval_ext2", MB_STREAM);
        sc_eval_ext2_kernel<<<gs(pair_count), BLOCK, 0, MB_STREAM>>>(d_data, gl::E2{gl::canon(c0), gl::canon(c1)}, d_output,
                                                                   pair_count);
    }
    return finish_sync();
}

int fused_sumcheck_round_ext2_ffi(const uint64_t* d_eq_in, const uint64_t* d_bh_in, uint64_t c0, uint64_t c1,
                                  uint64_t* d_eq_out, uint64_t* d_bh_out, uint64_t* p0, uint64_t* p1, uint64_t* p2,
                                  int pair_count, int num_blocks) {
    if (pair_count < 1 || num_blocks < 1 || !d_eq_in || !d_bh_in || !d_eq_out || !d_bh_out || !p0 || !p1 || !p2)
        return MB_ERR_ARG;
    {
        MB_KERNEL_ON("sc_fused_round_ext2", MB_STREAM);
        sc_fused_round_ext2_kernel<<<num_blocks, BLOCK, 0, MB_STREAM>>>(d_eq_in, d_bh_in, gl::E2{gl::canon(c0), gl::canon(c1)},
                                                                       d_eq_out, d_bh_out, p0, p1, p2, (size_t)pair_count);
    }
    return finish_sync();
}

int basefold_dot_product_gl_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_partial, int n, int num_blocks) {
    if (n < 0 || num_blocks < 1 || !d_a || !d_b || !d_partial) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("dot_gl", MB_STREAM);
        dot_gl_kernel<<<num_blocks, BLOCK, 0, MB_STREAM>>>(d_a, d_b, d_partial, (size_t)n);
    }
    return finish_sync();
}
int basefold_dot_product_mixed_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_partial, int n, int num_blocks) {
    if (n < 0 || num_blocks < 1 || !d_a || !d_b || !d_partial) return MB_ERR_ARG;
    {
        MB_KERNEL_ON("dot_mixed", MB_STREAM);
        dot_mixed_kernel<<<num_blocks, BLOCK, 0, MB_STREAM>>>(d_a, d_b, d_partial, (size_t)n);
    }
    return finish_sync();
}

// ---- eq tables: ffi.rs:396-410 ----
// The result is always left in d_buf_a; d_buf_b is used as scratch.
int eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result) {
    if (!d_result) return MB_ERR_ARG;
    int rc = eq::build<sc::GlBase>(d_r, d_buf_a, d_buf_b, log_n, MB_STREAM);
    if (rc != MB_OK) return rc;
    *d_result = d_buf_a;
    return finish_sync();
}
int ext2_eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result) {
    if (!d_result) return MB_ERR_ARG;
    int rc = eq::build<sc::GlExt2>(d_r, d_buf_a, d_buf_b, log_n, MB_STREAM);
    if (rc != MB_OK) return rc;
    *d_result = d_buf_a;
    return finish_sync();
}

// ---- fused permute + partial evaluation: ffi.rs:657-668 (cuda/fused_permute_peval.cuh:31-120) ----
// smem_bytes is the reference's launch parameter; the library sizes its own shared memory.
int fused_permute_partial_eval_ffi(const uint64_t* d_evals, uint64_t* d_output, const uint64_t* d_eq_table,
                                   const uint32_t* d_lo_lut, const uint32_t* d_hi_lut, int n, int m, int half,
                                   int output_size, int smem_bytes) {
    (void)smem_bytes;
    int rc = fp::launch<sc::GlBase, sc::GlExt2>(d_evals, d_output, d_eq_table, d_lo_lut, d_hi_lut, n, m, half, output_size,
                                                MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// ---- partial evaluation: ffi.rs:377-390 (cuda/partial_eval.cuh:113-219) ----
// In place: the 2^(log_n - m) results end up at the start of d_data.
int partial_eval_gl_ffi(uint64_t* d_data, const uint64_t* d_r, int log_n, int m) {
    if (log_n < 0 || log_n > 40 || m < 0 || m > log_n || !d_data) return MB_ERR_ARG;
    if (m == 0) return MB_OK;
    size_t n = (size_t)1 << log_n;
    uint64_t *t0 = nullptr, *t1 = nullptr;
    MB_CUDA(pool_alloc((void**)&t0, sizeof(uint64_t) * (n >> 1)));
    if (pool_alloc((void**)&t1, sizeof(uint64_t) * (n >> 1)) != cudaSuccess) { pool_free(t0); return MB_ERR_CUDA; }
    int rc = pe::partial_eval<sc::GlBase, sc::GlBase>(d_data, t0, t1, d_r, log_n, m, MB_STREAM);
    if (rc == MB_OK &&
        cudaMemcpyAsync(d_data, t0, sizeof(uint64_t) << (log_n - m), cudaMemcpyDeviceToDevice, MB_STREAM) != cudaSuccess)
        rc = MB_ERR_CUDA;
    if (rc == MB_OK) rc = finish_sync();
    pool_free(t0);
    pool_free(t1);
    return rc;
}
// Base-field table in, extension challenges (m pairs), 2^(log_n - m) extension elements out.
int partial_eval_ext2_from_gl_ffi(const uint64_t* d_input, uint64_t* d_output, const uint64_t* d_r, int log_n, int m) {
    if (log_n < 1 || log_n > 40 || m < 1 || m > log_n || !d_input || !d_output) return MB_ERR_ARG;
    size_t n = (size_t)1 << log_n;
    uint64_t* tmp = nullptr;
    MB_CUDA(pool_alloc((void**)&tmp, 2 * sizeof(uint64_t) * (n >> 1)));
    int rc = pe::partial_eval<sc::GlBase, sc::GlExt2>(d_input, d_output, tmp, d_r, log_n, m, MB_STREAM);
    if (rc == MB_OK) rc = finish_sync();
    pool_free(tmp);
    return rc;
}

}  // extern "C"
