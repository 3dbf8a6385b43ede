/*
 * C-ABI of libalmost_goldilocks_cuda_wrapper: almost-Goldilocks
 * (q = 2^64 - 2^32 - 31, extension X^2 = 3) hot path on B200 (sm_100a).
 *
 * Conventions as in goldilocks_cuda_wrapper.h: int return (0 ok, -1 CUDA error,
 * -2 rejected argument, -3 unsupported size), d_* device pointers owned by the
 * caller, loose u64 inputs, canonical outputs, calls run on the calling thread's
 * stream and return when done. Each declaration cites the reference interface it
 * replaces: almost-goldilocks-cuda-rs/src/ffi.rs (declaration) and
 * almost-goldilocks-cuda-rs/cuda/wrapper.cu (definition).
 */
#ifndef ALMOST_GOLDILOCKS_CUDA_WRAPPER_H
#define ALMOST_GOLDILOCKS_CUDA_WRAPPER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- init, memory, device: ffi.rs:77-100 (wrapper.cu:111-116, 205-330) ---- */
int almost_goldilocks_cuda_init(void);
/* Freed blocks are cached per device and reused (best fit, at most 25 % + 2 MiB larger; released and retried
 * when the driver is out of memory; AGL_ALLOC_CACHE=0 disables): almost-goldilocks-cuda-rs/cuda/wrapper.cu:118-235 */
int cuda_malloc(void** ptr, size_t size);
int cuda_free(void* ptr);
/* additions: release the current device's cached blocks; bytes they hold */
int mb_alloc_cache_flush(void);
size_t mb_alloc_cache_bytes(void);
int cuda_memcpy_htod(void* dst, const void* src, size_t size);
int cuda_memcpy_dtoh(void* dst, const void* src, size_t size);
int cuda_memcpy_dtod(void* dst, const void* src, size_t size);
int cuda_device_synchronize(void);
int cuda_get_last_error(void);
int cuda_peek_at_last_error(void);
int cuda_mem_get_info(size_t* free_bytes, size_t* total_bytes);
int cuda_set_device(int device);
int cuda_get_device(int* device);
int cuda_get_device_count(int* count);

/* ---- field batches: ffi.rs:103-135 ---- */
int agl_batch_add_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int agl_batch_sub_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int agl_batch_mul_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int agl_batch_inverse_ffi(const uint64_t* a, uint64_t* r, int n);
int aext2_batch_mul_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int aext2_batch_inverse_ffi(const uint64_t* a, uint64_t* r, int n);
/* ffi.rs:106-138,687: the remaining element-wise operations, asynchronous on the caller's stream */
int agl_batch_div_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int agl_batch_neg_ffi(const uint64_t* a, uint64_t* r, int n);
int agl_batch_square_ffi(const uint64_t* a, uint64_t* r, int n);
int agl_batch_double_ffi(const uint64_t* a, uint64_t* r, int n);
int agl_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* a, uint64_t* r, int n);
int agl_batch_exp_ffi(const uint64_t* a, uint64_t exp, uint64_t* r, int n);
int aext2_batch_add_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int aext2_batch_sub_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n);
int aext2_batch_neg_ffi(const uint64_t* a, uint64_t* r, int n);
int aext2_batch_square_ffi(const uint64_t* a, uint64_t* r, int n);
int aext2_batch_frobenius_ffi(const uint64_t* a, uint64_t* r, int n);
int aext2_batch_conjugate_ffi(const uint64_t* a, uint64_t* r, int n);
int aext2_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* a, uint64_t* r, int n);
int aext2_batch_exp_ffi(const uint64_t* a, uint64_t exp, uint64_t* r, int n);
int aext2_scale_accumulate_ffi(uint64_t scalar_c0, uint64_t scalar_c1, const uint64_t* src, uint64_t* acc, int n);
int agl_to_aext2_batch_ffi(const uint64_t* input, uint64_t* output, int n);
int aext2_to_agl_batch_ffi(const uint64_t* input, uint64_t* output, int n);
int agl_zero_buffer_ffi(uint64_t* d_buf, size_t n);
int agl_bit_permute_ffi(const uint64_t* d_input, uint64_t* d_output, const int* d_perm_map, int n_bits, int total);

/* ---- streams, copies, pool: ffi.rs:61-64,77-100,342-350 (wrapper.cu:259-411) ---- */
const char* agl_cuda_error_string(int code);
int cuda_memset(void* dst, int value, size_t size);
int cuda_sync_mine(void); /* the caller's own per-thread stream only */
int cuda_stream_create(void** stream);
int cuda_stream_destroy(void* stream);
int cuda_stream_synchronize(void* stream);
int cuda_memcpy_dtod_async(void* dst, const void* src, size_t size, void* stream);
int cuda_memcpy_htod_async(void* dst, const void* src, size_t size, void* stream);
int cuda_memcpy_peer(void* dst, int dst_dev, const void* src, int src_dev, size_t size);
int cuda_enable_peer_access(int peer);
int cuda_pool_trim(size_t min_bytes_to_keep);
size_t agl_cached_bytes(void);
/* pageable host memory through two pinned 64 MiB buffers per device */
int agl_d2h_staged(void* h_dst, const void* d_src, size_t bytes);
int agl_h2d_staged(void* d_dst, const void* h_src, size_t bytes);

/* ---- sumcheck: ffi.rs:221-263 (wrapper.cu:812-860); layouts as the Goldilocks twins ---- */
int agl_sumcheck_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                                   size_t half, int num_blocks);
int agl_sumcheck_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge, int d,
                          size_t original_size, size_t half);
int aext2_sumcheck_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                                     size_t half, int num_blocks);
int aext2_sumcheck_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                            uint64_t challenge_c1, int d, size_t original_size, size_t half);
/* additions: fold fused with the next round's message */
int aext2_sumcheck_fold_round_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                                  uint64_t challenge_c1, int d, size_t original_size, size_t quarter,
                                  uint64_t* d_partial, int num_blocks);
int aext2_sumcheck_fold_round_mixed_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                                        uint64_t challenge_c1, int d, size_t original_size, size_t quarter,
                                        uint64_t* d_partial, int num_blocks);

/* ---- eq tables: ffi.rs (agl_eq_dp_all_ffi, aext2_eq_dp_all_ffi), wrapper.cu:640-700 ---- */
int agl_eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result);
int aext2_eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result);

/* ---- partial evaluation: wrapper.cu:713-749 ---- */
int agl_partial_eval_ffi(uint64_t* d_data, const uint64_t* d_r, int log_n, int m);
int agl_partial_eval_ext2_from_base_ffi(const uint64_t* d_input, uint64_t* d_output, const uint64_t* d_r, int log_n,
                                        int m);

/* ---- fused bit-permutation + partial evaluation: wrapper.cu:755-800 ----
 * out[j] = sum_b evals[lo_lut[x & (2^half - 1)] | hi_lut[x >> half]] * eq[b], x = j 2^m + b; base-field
 * evals, extension eq table and output; smem_bytes is accepted for compatibility and ignored. */
int agl_fused_permute_partial_eval_ffi(const uint64_t* d_evals, uint64_t* d_output, const uint64_t* d_eq_table, const uint32_t* d_lo_lut,
       const uint32_t* d_hi_lut, int n, int m, int half, int output_size, int smem_bytes);

/* ---- Ajtai ring commitment: ffi.rs:426-433, 500-508, 595-617 (wrapper.cu:1095-1204, 1663-1670) ----
 * c_i = sum_j M[i][col_offset + j] * z_j in F_q[X]/(X^64 + 1), i < 42; M from
 * ChaCha8 keyed by d_key (8 u32). Dense: d_z[b*N + j] bit masks, d_out[b][42][64],
 * B in {1,2,4,8,16} (else -2). Wide: d_z_wide[j*64 + l] field coefficients,
 * d_out[42][64]. chunk in {64,128,256,1024,4096} (else -3); it is the
 * reference's tuning knob and does not change the result. */
int ajtai_commit_dense_batched_ffi(const uint32_t* d_key, const uint64_t* d_z, uint64_t N, int B, int chunk,
                                   uint64_t* d_out);
int ajtai_commit_dense_batched_at_ffi(const uint32_t* d_key, const uint64_t* d_z, uint64_t N, int B, int chunk,
                                      uint64_t col_offset, uint64_t* d_out);
int ajtai_commit_wide_ffi(const uint32_t* d_key, const uint64_t* d_z_wide, uint64_t N, uint64_t col_offset, int chunk,
                          uint64_t* d_out);
/* d_M[j][i][k], j < N (42 * 64 * 8 bytes per column) */
int ajtai_materialize_m_ffi(const uint32_t* d_chacha_key, uint64_t* d_M, uint64_t N);
/* ffi.rs:603-625: 13 ternary planes given as bit masks of the +1 / -1 coefficients, d_pos / d_neg[i * N_ring + j];
 * d_out[13][42][64] (kernel cuda_almost_goldilocks/ajtai.cuh:1262-1370). The premat form reads a matrix made by
 * ajtai_materialize_m_ffi. `chunk` is validated (-3) and otherwise ignored. */
int ajtai_commit_ternary_ffi(const uint32_t* d_key, const uint64_t* d_pos, const uint64_t* d_neg, uint64_t N_ring, int chunk,
                             uint64_t* d_out);
int ajtai_commit_ternary_premat_ffi(const uint64_t* d_M, const uint64_t* d_pos, const uint64_t* d_neg, uint64_t N_ring,
                                    int chunk, uint64_t* d_out);
/* ffi.rs:649-655: K positions p in [0, 64 N), c_i = sum_p X^(p mod 64) M[i][p / 64]; d_out[42][64]
 * (CPU twin cuda_almost_goldilocks/ajtai_cpu_reference.cuh:192-219) */
int ajtai_commit_sparse_ffi(const uint32_t* d_key, const uint64_t* d_positions, uint64_t K, int chunk, uint64_t* d_out);
/* ffi.rs:352-359: signed 16-bit coefficients d_wide[n_ring][64] to k_chunks <= 16 ternary planes (bit i of |v| goes to
 * plane i of pos or neg by sign); *d_err = 1 when a coefficient needs more bits (almost_sumcheck_prover.cuh:447-478) */
int aext2_wide_to_ternary_ffi(const int16_t* d_wide, uint64_t* d_pos, uint64_t* d_neg, int* d_err, size_t n_ring, int k_chunks);

/* ---- folding of witnesses and commitments by ring challenges: ffi.rs:435-492,635-647 (wrapper.cu:1468-1629,1717-1739;
 * kernels cuda_almost_goldilocks/ajtai.cuh:700-1255, ajtai_tc.cuh:44-411). Products are negacyclic (X^64 = -1);
 * challenges are 64 signed bytes (the protocol uses {-1, 0, 1, 2}). ---- */
/* d_out[N_ring][64] = z1 + r z2 as canonical field elements; z1, z2 bit masks; r_coeffs on the HOST */
int ajtai_fold_witness_ffi(const uint64_t* d_z1, const uint64_t* d_z2, const int8_t* r_coeffs, uint64_t N_ring, int chunk,
                           uint64_t* d_out);
/* d_out[42][64] = c1 + r c2; r_coeffs on the HOST */
int ajtai_fold_commitment_ffi(const uint64_t* d_c1, const uint64_t* d_c2, const int8_t* r_coeffs, uint64_t* d_out);
/* d_out[42][64] = sum_m r_m c_m; d_c_packed[m][42][64], d_r_all[m][64] on the device */
int ajtai_multifold_commitment_ffi(const uint64_t* d_c_packed, const int8_t* d_r_all, int num_instances, uint64_t* d_out);
/* d_out[N_ring][64] (16-bit) = sum_i r_i z_i: binary masks d_z[i * N_ring + j], then ternary (pos, neg) pairs; challenges in
 * that order on the device. All four run the tcgen05 int8 kernel (exact); chunk_size is ignored. */
int ajtai_multifold_witness_ffi(const uint64_t* d_z_packed, const int8_t* d_r_all, int16_t* d_out, int num_instances, uint64_t N_ring,
                                uint64_t chunk_size);
int ajtai_multifold_mixed_witness_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed, const uint64_t* d_neg_packed,
                                      const int8_t* d_r_all, int16_t* d_out, int num_binary, int num_ternary, uint64_t N_ring,
                                      uint64_t chunk_size);
int ajtai_multifold_mixed_witness_tc_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed, const uint64_t* d_neg_packed,
                                         const int8_t* d_r_all, int16_t* d_out, int num_binary, int num_ternary, uint64_t N_ring);
int ajtai_multifold_mixed_witness_tc_fused_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed,
                                               const uint64_t* d_neg_packed, const int8_t* d_r_all, int16_t* d_out, int num_binary,
                                               int num_ternary, uint64_t N_ring);
/* addition: the scalar form of the same fold, an independent check of the tensor-core path */
int ajtai_multifold_mixed_witness_scalar_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed,
                                             const uint64_t* d_neg_packed, const int8_t* d_r_all, int16_t* d_out, int num_binary,
                                             int num_ternary, uint64_t N_ring);
/* 16-bit coefficients d_z_wide[N_ring][64] to 13 ternary planes d_pos / d_neg[i * N_ring + j] */
int ajtai_split_witness_ffi(const int16_t* d_z_wide, uint64_t* d_pos_chunks, uint64_t* d_neg_chunks, uint64_t N_ring);

/* addition: signed 8-bit digit planes d_digits[(p*N + j)*64 + l] in [-128, 127], d_out[p][42][64];
 * scalar path, exact for any N */
int ajtai_commit_s8_scalar_ffi(const uint32_t* d_key, const int8_t* d_digits, uint64_t N, int planes,
                               uint64_t col_offset, uint64_t* d_out);

/* addition: the signed-digit commit on the tensor cores (tcgen05 kind::i8, exact s32 accumulation, byte-plane
 * recombination mod q); digits in [-127, 127] (-3 if a -128 is present), any number of planes */
int ajtai_commit_s8_ffi(const uint32_t* d_key, const int8_t* d_digits, uint64_t N, int planes, uint64_t col_offset,
                        uint64_t* d_out);
/* Addition (no reference counterpart for signed digits): the same commit against the matrix materialised by
 * ajtai_materialize_m_ffi (d_M[j][i][k], columns 0 .. N - 1); the tensor-core kernel streams d_M instead of
 * regenerating the matrix. ajtai_commit_ternary_premat_ffi (the reference's entry point) runs through it. */
int ajtai_commit_s8_premat_ffi(const uint64_t* d_M, const int8_t* d_digits, uint64_t N, int planes, uint64_t* d_out);
/* Additions (no reference counterpart): the matrix as unsigned byte planes in the order of the tensor-core operand
 * (per four columns and group of 14 rows one 28 KB image). ajtai_tc_matrix_bytes(N): size of d_T for N columns;
 * ajtai_materialize_tc_ffi: fill it for columns col_offset .. col_offset + N - 1; ajtai_commit_s8_tiled_ffi: the
 * signed-digit commit against it (the kernel copies the images; its work is the digit windows and the MMAs). */
uint64_t ajtai_tc_matrix_bytes(uint64_t N);
int ajtai_materialize_tc_ffi(const uint32_t* d_key, uint8_t* d_T, uint64_t N, uint64_t col_offset);
int ajtai_commit_s8_tiled_ffi(const uint8_t* d_T, const int8_t* d_digits, uint64_t N, int planes, uint64_t* d_out);
/* Addition (measurement helper, no reference counterpart): sustained int8 multiply-accumulates per second of the
 * tensor pipes of the current device, from the commit kernel's own tcgen05 kind::i8 issue loop on operands that
 * stay in shared memory (one CTA per SM, `groups` groups of eight M = 128, N = 256, K = 32 MMAs). */
int ajtai_tc_int8_peak_ffi(int groups, double* mac_per_second);
/* the same with MMAs of N = n_cols (a multiple of 16 up to 256): what the shape of an MMA costs */
int ajtai_tc_int8_peak_n_ffi(int groups, int n_cols, double* mac_per_second);
/* the same with `depth` (1..7) committed groups in flight before the issuing thread waits (the two calls above use
 * 6): with depth 1 the figure for narrow MMAs is the commit-to-wait round trip, not the pipe */
int ajtai_tc_int8_peak_shape_ffi(int groups, int n_cols, int depth, double* mac_per_second);

/* ---- batched same-point sumcheck family (sum_x eq(x) f(x) per leaf, messages at c = 0, 1, 2): ffi.rs:177-195,265-423
 * (wrapper.cu:674-707,851-1060; kernels cuda_almost_goldilocks/almost_sumcheck_prover.cuh:233-1007). Tables are Ext2
 * (two words per element) with stride original_size elements; folds bind the low variable; message kernels write
 * d_partial[block][leaf][c][2] for the caller to add; all calls are asynchronous on the caller's stream. ---- */
/* interleaved layout: d_polys[leaf] = eq table, then f table */
int aext2_sumcheck_batched_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, size_t original_size, size_t half,
                                             int num_leaves, int num_blocks_x);
int aext2_sumcheck_batched_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0, uint64_t challenge_c1,
                                    size_t original_size, size_t half, int num_leaves);
/* round 0 with f still binary (packed bits, packed_size_u64 words per leaf): no lift, f' in {0, 1, r, 1 - r} */
int aext2_sumcheck_batched_round0_binary_msg_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_partial,
                                                 size_t original_size, size_t half, int num_leaves, int num_blocks_x,
                                                 size_t packed_size_u64);
int aext2_sumcheck_batched_round0_binary_fold_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_output,
                                                  uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size, size_t half,
                                                  int num_leaves, size_t packed_size_u64);
/* additions (no reference counterpart): the fold on the challenge and the message of the NEXT round in one pass over
 * the tables; `half` is the half of the input tables and must be even; d_partial as for the message kernels */
int aext2_sumcheck_batched_fold_message_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0, uint64_t challenge_c1,
                                            size_t original_size, size_t half, int num_leaves, int num_blocks_x, uint64_t* d_partial);
int aext2_sumcheck_batched_round0_binary_fold_message_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_output,
                                                          uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size, size_t half,
                                                          int num_leaves, int num_blocks_x, size_t packed_size_u64, uint64_t* d_partial);
/* shared eq: eq tables of the distinct points in d_eq, f tables in d_f, leaf -> point map */
int aext2_sharedeq_msg_ffi(const uint64_t* d_eq, const uint64_t* d_f, const int* d_leaf_to_unique, uint64_t* d_partial,
                           size_t original_size, size_t half, int num_leaves, int num_blocks_x);
int aext2_fold_single_ffi(const uint64_t* d_in, uint64_t* d_out, uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size,
                          size_t half, int count);
/* factored eq: suffix tables eqsuf_t (element offset 2^(log_n - t) - 1 inside each point's region) built once;
 * a round returns d_partial[block][point][A, B][2], A = sum_y eqsuf[y] F[2y], B = sum_y eqsuf[y] F[2y + 1] */
int aext2_eq_suffix_dp_ffi(const uint64_t* d_r_all, uint64_t* d_eqsuf, int log_n, int num_unique, size_t eqsuf_stride_u64);
int aext2_sharedeq_factored_msg_ffi(const uint64_t* d_eqsuf, const uint64_t* d_fu, uint64_t* d_partial, size_t eqsuf_off_elems,
                                    size_t eqsuf_stride_u64, size_t poly_stride_u64, size_t half, int num_unique, int num_blocks_x);
/* F_u[x] = sum over the leaves of point u of alpha_leaf f_leaf[x]; leaves sorted by point, offsets[num_unique + 1] */
int aext2_build_fu_ffi(const uint64_t* d_packed, const uint64_t* d_alphas, const int* d_leaf_idx_sorted, const int* d_unique_offsets,
                       uint64_t* d_Fu, size_t original_size, int num_unique, size_t packed_size_u64);
int aext2_build_fu_ternary_ffi(const uint64_t* d_pos, const uint64_t* d_neg, const uint64_t* d_alphas, const int* d_leaf_idx_sorted,
                               const int* d_unique_offsets, uint64_t* d_Fu, size_t original_size, int num_unique, size_t packed_size_u64);
/* packed planes to Ext2 tables: into the f slot of the interleaved layout, a contiguous array, or pos - neg */
int aext2_batched_lift_binary_ffi(const uint64_t* d_packed, uint64_t* d_polys, size_t original_size, int num_leaves, size_t packed_size_u64);
int aext2_lift_binary_contig_ffi(const uint64_t* d_packed, uint64_t* d_f, size_t original_size, int num_leaves, size_t packed_size_u64);
int aext2_batched_lift_ternary_single_ffi(const uint64_t* d_pos, const uint64_t* d_neg, uint64_t* d_polys, size_t original_size,
                                          int num_leaves, size_t packed_size_u64);
/* d_partial[block][plane][2]: sum of eq[i] over the set bits of each plane */
int aext2_selective_add_batched_planes_ffi(const uint64_t* d_eq, const uint64_t* d_packed_planes, uint64_t* d_partial, size_t total,
                                           int n_planes, size_t packed_size_u64, int num_blocks_x);
/* eq tables on a caller stream; the table is returned in d_buf_a (d_buf_b is scratch) */
int aext2_eq_dp_all_stream_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result, void* stream);
int aext2_eq_dp_all_batched_ffi(const uint64_t* d_r_all, uint64_t* d_buf_a_all, uint64_t* d_buf_b_all, int log_n, int num_leaves,
                                size_t leaf_stride, uint64_t** d_result, void* stream);

/* ---- K = F_q[Theta]/(Theta^8 - 3) product sumcheck and table helpers: ffi.rs:65-75 (wrapper.cu:3815-3905;
 * kernels cuda_almost_goldilocks/morpheus_piop.cuh:140-282; CPU zk-torch-4/src/morpheus/piop/mod.rs:785-840,
 * field zk-torch-4/src/morpheus/field8.rs). Elements are 8 canonical words; tables live on the device,
 * h_tabs / h_outs are host arrays of device pointers, challenges / points / sums are host words.
 * -3: more than 6 tables or degree above 6 (or len < 4 for the fused form). ---- */
int agl_mpiop_sc_round(const uint64_t* const* h_tabs, int ntab, uint64_t len, int d, uint64_t* h_out);
int agl_mpiop_sc_fold(const uint64_t* d_in, uint64_t* d_out, uint64_t len, const uint64_t* h_r);
int agl_mpiop_sc_fold_round(const uint64_t* const* h_tabs, uint64_t* const* h_outs, int ntab, uint64_t len,
                            const uint64_t* h_r, int d, uint64_t* h_out);
int agl_mpiop_eq(const uint64_t* h_point, int n, uint64_t* d_out);
int agl_mpiop_eq_outer(const uint64_t* d_lo, int nlo, const uint64_t* d_hi, int nhi, uint64_t* d_out);
int agl_mpiop_axpy(uint64_t* d_out, const uint64_t* d_in, uint64_t n, const uint64_t* h_c);
int agl_mpiop_lift(const uint64_t* d_in, uint64_t n, uint64_t* d_out);
/* ffi.rs:65-68 (wrapper.cu:3753-3837; kernels morpheus_piop.cuh:20-172): helpers over base-field tables.
 * pe: d_out[r] = sum_f d_vals[deposit(r, rest_pos) | deposit(f, fix_pos)] d_e[f] (bit j of r / f goes to bit pos[j];
 * rest_pos, fix_pos are host arrays); mle: h_out[8] = sum_x d_vals[x] eq(x, h_point); gather: d_out[x] = d_in[idx],
 * bit j of idx = bit pos[j] of x; sel_lookup: d_out[i] = d_table[(d_sel[i] >> shift) & mask]. */
int agl_mpiop_pe(const uint64_t* d_vals, const int* rest_pos, int nrest_v, const int* fix_pos, int nfix_v, const uint64_t* d_e,
                 uint64_t* d_out);
int agl_mpiop_mle(const uint64_t* d_vals, const uint64_t* h_point, int n, uint64_t* h_out);
int agl_mpiop_gather(const uint64_t* d_in, const int* pos, int nv, uint64_t n, uint64_t* d_out);
int agl_mpiop_sel_lookup(const uint64_t* d_sel, uint64_t n, int shift, uint64_t mask, const uint64_t* d_table, uint64_t* d_out);

/* ---- exact module commitment over F_q[Y]/(Y^4096 + 1) ----
 * Replaces almost-goldilocks-cuda-rs/src/ffi.rs:18-21 (definitions cuda/wrapper.cu:3129-3229; kernels
 * cuda_almost_goldilocks/morpheus_commit.cuh; CPU definition zk-torch-4/src/morpheus/commit.rs:48-83,
 * ring.rs, keys.rs:48-93; Rust caller zk-torch-4/src/morpheus/commit_gpu.rs:27-97).
 * C[v][row] = sum_c centre(A_kind[row][col_c]) * x[v][c] as integer negacyclic products, reduced mod q
 * at the end, exact while twice the largest |coefficient| stays below the product of the first k of the
 * five 31-bit primes 2147377153, 2147352577, 2147295233, 2147205121, 2147196929 (k = 3 for ternary
 * inputs, 5 for 37-bit ones). Buffers between the calls: d_key u32 [k][ncols][rows][4096], d_acc u32
 * [V][k][rows][4096]; their contents are transform-domain residues in this library's own order (a cache
 * built with k primes serves calls with fewer). rows <= 16, V <= 8, x_bytes 1 (int8) or 8 (int64). */
int agl_mcommit_keygen(const uint32_t* h_seed, uint32_t kind, int rows, uint64_t col0, int ncols, int k, uint32_t* d_key);
int agl_mcommit_partial(const uint32_t* d_key, int kcols, int rows, int k, const void* d_x, int x_bytes, int V, int C,
                        uint64_t x_vstride, const uint32_t* d_colidx, uint32_t* d_acc);
int agl_mcommit_add(uint32_t* d_dst, const uint32_t* d_src, int V, int k, int rows);
/* d_out u64 [V][rows][4096] canonical; d_err int64 [V][rows][4096] or null is added; d_acc is left unchanged. */
int agl_mcommit_finish(uint32_t* d_acc, int V, int k, int rows, const int64_t* d_err, uint64_t* d_out);

/* ---- sparse boolean-check sumcheck ----
 * Replaces almost-goldilocks-cuda-rs/src/ffi.rs:140-158 (definitions cuda/wrapper.cu:2650-2981; Rust state
 * almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:2186-2340). sum_t w_t sum_x eq(x) v_t(x) (v_t(x) - 1) over sorted
 * (position u32, value ext) entry lists, term t owning entries [d_term_off[t], d_term_off[t + 1]); a round binds the low
 * position bit. round_msg fills d_flags (1 = entry opens a group) and d_gid (exclusive prefix sum of the flags), returns
 * the four evaluations at 0..3 in h_msg (8 canonical words) and the number of groups in *h_total; d_eq is the eq table of
 * the current size. d_partial, grid_x and the scan scratch are accepted for signature compatibility and not used.
 * fold writes `total` merged entries and n_terms + 1 new offsets. n < 2^32 - 4096. */
int agl_bool_init_val_ffi(uint64_t* d_val, size_t n);
int agl_bool_round_msg_ffi(const uint32_t* d_idx, const uint64_t* d_val, const uint32_t* d_term_off, const uint64_t* d_w,
                           const uint64_t* d_eq, int n_terms, size_t n, uint32_t* d_flags, uint32_t* d_gid, uint64_t* d_partial,
                           int grid_x, uint32_t* d_scan_scratch, size_t scan_scratch_len, uint64_t* h_msg, uint32_t* h_total);
int agl_bool_fold_ffi(const uint32_t* d_idx, const uint64_t* d_val, const uint32_t* d_flags, const uint32_t* d_gid,
                      const uint32_t* d_term_off, int n_terms, size_t n, uint64_t r0, uint64_t r1, uint32_t total, int grid_x,
                      uint32_t* d_out_idx, uint64_t* d_out_val, uint32_t* d_new_off);
int agl_bool_finish_ffi(const uint32_t* d_idx, const uint64_t* d_val, const uint32_t* d_term_off, int n_terms, size_t n,
                        uint64_t* d_out);

/* ---- packed link sumcheck ----
 * Replaces almost-goldilocks-cuda-rs/src/ffi.rs:511-593 (definitions cuda/wrapper.cu:1213-1440, kernels
 * cuda_almost_goldilocks/link_sumcheck.cuh; CPU definition zk-torch-4/src/pcs/link.rs:284-357).
 * Extension elements are two u64; tables are rows of `stride` elements per commitment; the HIGH index bit is
 * bound first (pairs (idx, half + idx)). Round messages: d_out = [S(0..3), E(0..2)], seven canonical elements,
 * S(k) = sum_e tag_e sum_idx eq[idx] R(w_e(k)[idx]) with R(u) = u^3 - u, E(k) = sum_e sum_idx omega_e(k)[idx]
 * w_e(k)[idx]; with first_round != 0 (and in the round0_bits forms) S(0) = S(1) = 0. d_partial is scratch of
 * n_commit * chunks * 7 elements; chunks = grid width per commitment. Support lists: d_list slices
 * [d_list_off[e], + d_list_len[e]) of pair indices, eq then indexed by list position. Interleaved layout: block
 * b = idx & block_mask, weight = scale[e][b] * eq(idx >> block_bits, pts[e][b][round .. leaf_arity)). */
int link_round_message_ffi(const uint64_t* d_w, const uint64_t* d_omega, const uint64_t* d_eq_suffix, const uint64_t* d_tags,
                           uint64_t stride, uint64_t omega_stride, uint64_t half, uint64_t n_commit, int first_round,
                           uint64_t* d_partial, uint64_t chunks, uint64_t* d_out);
int link_round_message_sparse_ffi(const uint64_t* d_w, const uint64_t* d_omega, const uint64_t* d_eq_suffix, const uint64_t* d_tags,
                                  const uint32_t* d_list, const uint64_t* d_list_off, const uint64_t* d_list_len, uint64_t stride,
                                  uint64_t omega_stride, uint64_t half, uint64_t n_commit, int first_round, uint64_t* d_partial,
                                  uint64_t chunks, uint64_t* d_out);
int link_round0_bits_ffi(const uint64_t* d_bits, const uint64_t* d_omega, const uint64_t* d_eq, const uint64_t* d_tags, uint64_t stride,
                         uint64_t half, uint64_t n_commit, uint64_t* d_partial, uint64_t chunks, uint64_t* d_out);
int link_round0_bits_sparse_ffi(const uint64_t* d_bits, const uint64_t* d_omega, const uint64_t* d_eq, const uint64_t* d_tags,
                                const uint32_t* d_list, const uint64_t* d_list_off, const uint64_t* d_list_len, uint64_t stride,
                                uint64_t half, uint64_t n_commit, uint64_t* d_partial, uint64_t chunks, uint64_t* d_out);
int link_round_interleaved_ffi(const uint64_t* d_bits, const uint64_t* d_w, const uint64_t* d_pts, const uint64_t* d_scale,
                               const uint64_t* d_eq, const uint64_t* d_tags, const uint32_t* d_list, const uint64_t* d_list_off,
                               const uint64_t* d_list_len, uint64_t w_stride, uint64_t bits_stride_words, uint64_t half,
                               uint64_t n_commit, uint32_t block_mask, int block_bits, int leaf_arity, int round, int first_round,
                               uint64_t* d_partial, uint64_t chunks, uint64_t* d_out);
/* t[i] = lo + r (hi - lo), in place on both tables (rows of stride / omega_stride). */
int link_fold_ffi(uint64_t* d_w, uint64_t* d_omega, uint64_t stride, uint64_t omega_stride, uint64_t half, uint64_t n_commit,
                  uint64_t r_c0, uint64_t r_c1);
int link_fold_sparse_ffi(uint64_t* d_w, uint64_t* d_omega, const uint32_t* d_list, const uint64_t* d_list_off,
                         const uint64_t* d_list_len, uint64_t stride, uint64_t half, uint64_t n_commit, uint64_t r_c0, uint64_t r_c1);
/* bits in (rows of stride bits), d_w_out rows of `half` elements, d_omega (rows of stride) folded in place. */
int link_fold0_bits_ffi(const uint64_t* d_bits, uint64_t* d_w_out, uint64_t* d_omega, uint64_t stride, uint64_t half, uint64_t n_commit,
                        uint64_t r_c0, uint64_t r_c1);
int link_fold_w_ffi(const uint64_t* d_bits, const uint64_t* d_w_in, uint64_t* d_w_out, uint64_t in_stride, uint64_t bits_stride_words,
                    uint64_t out_stride, uint64_t half, uint64_t n_commit, int first_round, uint64_t r_c0, uint64_t r_c1);
/* table[i], table[span + i] = v (1 - r), v r for i < span. */
int link_eq_expand_ffi(uint64_t* d_table, uint64_t span, uint64_t r_c0, uint64_t r_c1);
int link_omega_expand_ffi(uint64_t* d_omega, const uint64_t* d_bases, const uint64_t* d_rs, uint64_t span, uint64_t n_active);
int link_expand_bits_ffi(const uint64_t* d_bits, uint64_t* d_out, uint64_t n_words);
int link_eq_gather_ffi(const uint64_t* d_alpha, uint64_t n_vars, const uint32_t* d_list, uint64_t* d_out, uint64_t total);

/* ---- host side: Monolith over almost-Goldilocks and the transcript on it ----
 * The reference keeps these in Rust: permutation and SHA-256-derived round constants
 * zk-torch-4/src/crypto/monolith.rs:66-208, transcript zk-torch-4/src/transcript.rs:22-243 (width 12,
 * rate 8, overwrite mode, LIFO outputs; a label is absorbed as its length then its bytes, an empty label
 * absorbs nothing; the constructor absorbs its label bytes without a length; appended values are
 * reduced mod q). No device work. */
int agl_monolith_permute_host(uint64_t* state12);
int agl_monolith_round_constants(uint64_t* out84); /* [7][12] */
int agl_transcript_create(const uint8_t* label, size_t label_len, void** transcript);
int agl_transcript_destroy(void* transcript);
/* transcript.rs:168-173: a copy that has absorbed the family label and the branch id */
int agl_transcript_fork(const void* transcript, const uint8_t* family, size_t family_len, uint64_t branch_id,
                        void** forked);
int agl_transcript_append_scalar(void* transcript, const uint8_t* label, size_t label_len, uint64_t v);
int agl_transcript_append_u64(void* transcript, const uint8_t* label, size_t label_len, uint64_t v);
int agl_transcript_append_u64_slice(void* transcript, const uint8_t* label, size_t label_len, const uint64_t* values,
                                    size_t n);
int agl_transcript_append_ext2(void* transcript, const uint8_t* label, size_t label_len, uint64_t c0, uint64_t c1);
int agl_transcript_challenge_scalar(void* transcript, const uint8_t* label, size_t label_len, uint64_t* out);
/* n = 2 is challenge_ext2 (c0 then c1) */
int agl_transcript_challenge_vector(void* transcript, const uint8_t* label, size_t label_len, uint64_t* out, size_t n);
int agl_transcript_state(const void* transcript, uint64_t* out12);

/* ---- addition: the device sequence of one einsum block's proof in one call (Einsum::prove_gpu,
 * zk-torch-4/src/basicblock/einsum.rs:1168-1310, which issues these steps from Rust one synchronising FFI call each):
 * per operand the partial evaluation at the output point's coordinates that belong to it alone (plain when those are its
 * low variables: d_lut_lo null; fused with the bit permutation of partial_eval.rs:283-321 otherwise), the eq table of the
 * output variables two operands share (a table of ones when num_shared = 0), the tables tiled over the variables an
 * operand does not depend on, then agl_sumcheck_prove_device_ffi over the num_operands + 1 tables of 2^rounds
 * elements on `transcript`. An operand's table variables are the lowest n - m of the block's. h_point: the output
 * point, (c0, c1) per variable; fixed_idx (per operand m entries from fixed_off) and shared_idx index its variables.
 * Host outputs as agl_sumcheck_prove_device_ffi with d = num_operands + 1. */
typedef struct mb_einsum_operand {
    const uint64_t* d_src;      /* 2^n base-field words */
    const uint32_t* d_lut_lo;   /* split index tables of the permutation, or null for the identity */
    const uint32_t* d_lut_hi;
    int n;                      /* variables of the operand */
    int m;                      /* of which fixed to coordinates of the point (the first m of the new order) */
    int fixed_off;              /* offset of this operand's m indices in fixed_idx */
    int reserved;
} mb_einsum_operand;
int agl_einsum_prove_device_ffi(int num_operands, const mb_einsum_operand* ops, const int* fixed_idx, int rounds, int num_shared,
                                const int* shared_idx, const uint64_t* h_point, int point_vars, void* transcript,
                                uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval);

/* ---- addition: the same-point sumcheck as a whole protocol (the host loop the reference keeps in Rust:
 * zk-torch-4/src/fold/same_point_sumcheck.rs:58-157 prover and labels, :1334-1553 device path over the batched
 * kernels above, :161-219 verifier). num_leaves instances of one arity, each with its own claim point and claim
 * y_i = f_i(r_i); the proof reduces them to one point R. h_claim_pts[num_leaves][arity][2],
 * h_claim_vals[num_leaves][2]; witness on the device: kind 0 binary packed (d_w0[num_leaves][words], words =
 * max(1, 2^(arity - 6)), bit j of word j / 64), 1 ternary single chunk (d_w0 = +1 masks, d_w1 = -1 masks), 2
 * extension tables (d_w0[num_leaves][2^arity][2]). `transcript` is a handle from agl_transcript_create and is
 * advanced exactly as the reference's prover advances it. Host outputs: round_msgs[arity][3][2] (degree 2),
 * challenges[arity][2] (may be null), f_evals[num_leaves][2] = f_i(R), final_eval[2]. Device memory: 2 x num_leaves x
 * 2^arity x 32 bytes. Instances of different arities stay on the CPU path, as in the reference. */
int agl_same_point_prove_device_ffi(int num_leaves, int arity, const uint64_t* h_claim_pts, const uint64_t* h_claim_vals, int kind,
                                    const uint64_t* d_w0, const uint64_t* d_w1, void* transcript, uint64_t* h_round_msgs,
                                    uint64_t* h_challenges, uint64_t* h_f_evals, uint64_t* h_final_eval);
/* the claims y_i = f_i(r_i) the protocol starts from (FoldData::evaluate_at_ext2, zk-torch-4/src/fold/mod.rs:107-110),
 * on the device with the kernels of the proof: h_claim_vals[num_leaves][2] */
int agl_same_point_claims_device_ffi(int num_leaves, int arity, const uint64_t* h_claim_pts, int kind, const uint64_t* d_w0,
                                     const uint64_t* d_w1, uint64_t* h_claim_vals);
/* verify_same_point on the host; arity[i] <= num_vars may differ per instance (h_claim_pts: arity[i] pairs each, back
 * to back). *ok = 1 when the proof is accepted; challenges (num_vars pairs) are written when not null. */
int agl_same_point_verify_ffi(int num_instances, int num_vars, const int* arity, const uint64_t* h_claim_pts,
                              const uint64_t* h_claim_vals, const uint64_t* round_msgs, const uint64_t* f_evals,
                              const uint64_t* final_eval, void* transcript, uint64_t* challenges, int* ok);

/* ---- host layer: the whole linear sumcheck (the reference keeps these loops in Rust) ----
 * GpuLinearSumcheckProver::new + prove / prove_ext2 / prove_gpu_resident
 * (zk-torch-4/src/sumcheck/gpu_prover.rs:26-112), interoperable with CpuLinearSumcheckProverExt2
 * (zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100). d tables of 2^num_var elements, poly-major;
 * base_field != 0: one word per element, else (c0, c1). `transcript` is a handle from
 * agl_transcript_create and is advanced by the proof (append num_var, num_poly; per round the d+1
 * values under "round_message", then challenge_ext2("challenge")). Host outputs:
 * round_msgs[num_var][d+1][2], challenges[num_var][2] (may be NULL), final_evals[d][2] (may be
 * NULL), final_eval[2] = product of the final evaluations (SumcheckProof, sumcheck/mod.rs:32-36). */
int agl_sumcheck_prove_device_ffi(const uint64_t* d_tables, int d, int num_var, int base_field, void* transcript,
                                  uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals,
                                  uint64_t* final_eval);
int agl_sumcheck_prove_host_ffi(const uint64_t* h_tables, int d, int num_var, int base_field, void* transcript,
                                uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval);
/* SumcheckVerifier::verify (zk-torch-4/src/sumcheck/verifier.rs:14-113), on the host: *ok = 1 when the
 * proof is accepted against claimed_sum[2]; challenges[num_var][2] may be NULL. */
int agl_sumcheck_verify_ffi(const uint64_t* round_msgs, const uint64_t* final_eval, const uint64_t* claimed_sum, int d,
                            int num_var, void* transcript, uint64_t* challenges, int* ok);

/* ---- additions shared with the Goldilocks library ---- */
/* d_out[i] = splitmix64(seed) output i + 1 mod modulus: seeded synthetic inputs made on the device */
int mb_fill_splitmix(uint64_t* d_out, size_t n, uint64_t seed, uint64_t modulus);
int mb_event_create(void** ev);
int mb_event_record(void* ev);
int mb_event_sync(void* ev);
int mb_event_elapsed_ms(void* start, void* stop, float* ms);
int mb_event_destroy(void* ev);
int mb_stream_sync(void);
uint64_t mb_launch_count(void);


/* ---- out of scope: stubs ----
 * Declared by the reference's ffi.rs but outside the prover's field-arithmetic path. Exported so that the
 * crates link unchanged: every one returns -3 (unsupported) and touches nothing (the two profiler range
 * markers are no-ops). Parameter lists are those of ffi.rs and are not repeated here. */
#ifdef __cplusplus
#define MB_STUB_ARGS ...
#else
#define MB_STUB_ARGS
#endif
int agl_morpheus_gauss_words(MB_STUB_ARGS);
int agl_morpheus_gauss_dev(MB_STUB_ARGS);
int agl_mauth_wtable(MB_STUB_ARGS);
int agl_mauth_ev(MB_STUB_ARGS);
int agl_mauth_decode(MB_STUB_ARGS);
int agl_mauth_combine_multi(MB_STUB_ARGS);
int agl_mauth_combine(MB_STUB_ARGS);
int agl_mauth_norm(MB_STUB_ARGS);
int agl_mauth_pack37(MB_STUB_ARGS);
int agl_mauth_unpack37(MB_STUB_ARGS);
int agl_mlink_phase1(MB_STUB_ARGS);
int agl_mlink_fold(MB_STUB_ARGS);
int agl_morpheus_coins(MB_STUB_ARGS);
int agl_mlink2_consts(MB_STUB_ARGS);
int agl_mlink2_round(MB_STUB_ARGS);
int agl_mlink2_range_bin1(MB_STUB_ARGS);
int agl_mlink2_coarse_init(MB_STUB_ARGS);
int agl_i64_to_i32(MB_STUB_ARGS);
int agl_add_i32_i64(MB_STUB_ARGS);
int agl_mlink2_coarse_init2(MB_STUB_ARGS);
int agl_mlink2_b_build(MB_STUB_ARGS);
int agl_mlink2_b_halve(MB_STUB_ARGS);
int agl_mlink2_dense_expand(MB_STUB_ARGS);
int agl_mlink2_coarse_round(MB_STUB_ARGS);
int agl_mlink2_coarse_fold(MB_STUB_ARGS);
int agl_mlink2_onehot3(MB_STUB_ARGS);
int agl_mlink2_onehot_pre(MB_STUB_ARGS);
int agl_mlink2_onehot_bin(MB_STUB_ARGS);
int agl_mlink2_rep_reduce(MB_STUB_ARGS);
int agl_morpheus_permute(MB_STUB_ARGS);
int agl_morpheus_unpack2(MB_STUB_ARGS);
int agl_morpheus_permute2(MB_STUB_ARGS);
int agl_mauth_ev_packed_batch(MB_STUB_ARGS);
int agl_mauth_combine_tc(MB_STUB_ARGS);
int agl_mauth_combine_packed(MB_STUB_ARGS);
int agl_gauss_low_priority(MB_STUB_ARGS);
int agl_mlink2_index(MB_STUB_ARGS);
int agl_morpheus_gauss_scatter(MB_STUB_ARGS);
void agl_nvtx_push(MB_STUB_ARGS);
void agl_nvtx_pop(MB_STUB_ARGS);
int ajtai_tc_commit_probe_ffi(MB_STUB_ARGS);
int agl_einsum2_ffi(MB_STUB_ARGS);
int agl_einsum1_ffi(MB_STUB_ARGS);
int agl_relu_helper_ffi(MB_STUB_ARGS);
int agl_conv2d_ffi(MB_STUB_ARGS);
int agl_flatten_kernel2d_ffi(MB_STUB_ARGS);
int agl_conv3d_ffi(MB_STUB_ARGS);
int agl_flatten_kernel3d_ffi(MB_STUB_ARGS);
int agl_depthwise_conv2d_ffi(MB_STUB_ARGS);
int agl_conv_transpose2d_ffi(MB_STUB_ARGS);
int agl_conv_transpose3d_ffi(MB_STUB_ARGS);
int agl_conv_full_ffi(MB_STUB_ARGS);

#ifdef __cplusplus
}
#endif
#endif
