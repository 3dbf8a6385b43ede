/*
 * C-ABI of libgoldilocks_cuda_wrapper: Goldilocks (p = 2^64 - 2^32 + 1) hot path
 * on B200 (sm_100a).
 *
 * Every function returns int: 0 success, -1 CUDA error, -2 rejected argument,
 * -3 unsupported configuration. Pointers named d_* are device memory that the
 * caller owns (obtained from cuda_malloc, returned with cuda_free); h_* are host
 * memory. Inputs may be any u64 representative of a residue; everything
 * written out is canonical (< p). Calls run on the calling thread's stream
 * and return when their result is ready.
 *
 * Each declaration cites the reference interface it replaces: the Rust
 * `extern "C"` block in goldilocks-cuda-rs/src/ffi.rs (declaration) and
 * goldilocks-cuda-rs/cuda/wrapper.cu (definition). Entries marked "addition"
 * have no reference counterpart.
 */
#ifndef GOLDILOCKS_CUDA_WRAPPER_H
#define GOLDILOCKS_CUDA_WRAPPER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- initialisation: ffi.rs:10-11, :549 (wrapper.cu:27-46) ---- */
int goldilocks_cuda_init(void);
int poseidon2_cuda_init(void);
int monolith_cuda_init(void);

/* ---- element-wise batch operations: ffi.rs:31-58,165-285,629-655 (wrapper.cu:100-575,1807-1860,2446-2460).
 * Device pointers, n elements (extension elements are two consecutive words), canonical outputs,
 * asynchronous on the caller's stream like the reference's. Division and inversion map 0 to 0. ---- */
int gl_batch_add(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int gl_batch_sub(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int gl_batch_mul(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int gl_batch_div(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int gl_batch_inverse(const uint64_t* d_a, uint64_t* d_result, int n);
int gl_batch_neg(const uint64_t* d_a, uint64_t* d_result, int n);
int gl_batch_square(const uint64_t* d_a, uint64_t* d_result, int n);
int gl_batch_double(const uint64_t* d_a, uint64_t* d_result, int n);
int gl_batch_mul_scalar(uint64_t scalar, const uint64_t* d_a, uint64_t* d_result, int n);
int gl_batch_exp(const uint64_t* d_a, uint64_t exp, uint64_t* d_result, int n);
int ext2_batch_add_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int ext2_batch_sub_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int ext2_batch_mul_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int ext2_batch_inverse_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext2_batch_neg_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext2_batch_square_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext2_batch_frobenius_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext2_batch_conjugate_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext2_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* d_a, uint64_t* d_result, int n);
int ext2_batch_exp_ffi(const uint64_t* d_a, uint64_t exp, uint64_t* d_result, int n);
/* acc[i] += scalar * src[i] */
int ext2_scale_accumulate_ffi(uint64_t scalar_c0, uint64_t scalar_c1, const uint64_t* d_src, uint64_t* d_acc, int n);
int gl_to_ext2_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n);
int ext2_to_gl_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n);
/* Degree-5 extension F_p[X]/(X^5 - 3), five consecutive words per element
 * (goldilocks-cuda-rs/src/ffi.rs:229-281; arithmetic cuda/extension.cuh:299-700).
 * The inverse of zero is zero; the Frobenius map is x -> x^p. */
int ext5_batch_add_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int ext5_batch_sub_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int ext5_batch_mul_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_result, int n);
int ext5_batch_inverse_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext5_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* d_a, uint64_t* d_result, int n);
int ext5_batch_neg_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext5_batch_square_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext5_batch_frobenius_ffi(const uint64_t* d_a, uint64_t* d_result, int n);
int ext5_batch_exp_ffi(const uint64_t* d_a, uint64_t exp, uint64_t* d_result, int n);
int gl_to_ext5_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n);
int ext5_to_gl_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n);
int gl_zero_buffer(uint64_t* d_buf, int n);
/* out[new] = in[old] where bit b of new is bit d_perm_map[b] of old (wrapper.cu:1843-1860) */
int bit_permute_gl_ffi(const uint64_t* d_input, uint64_t* d_output, const int* d_perm_map, int n_bits, int total);

/* ---- memory: ffi.rs:17-25 (wrapper.cu:52-98) ---- */
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
/* ffi.rs:102 */
int gl_memset_zero(uint64_t* d_buf, size_t n_u64);

/* ---- device info: ffi.rs:305-308 ---- */
int cuda_set_device(int device);
int cuda_get_device(int* device);
int cuda_get_device_count(int* count);
int cuda_get_device_name(int device, char* name, int max_len);

/* ---- sumcheck, base field: ffi.rs:588-604 (wrapper.cu:1716-1749) ----
 * d tables of `original_size` u64 each, poly-major; `half` = live length / 2.
 * round_message writes num_blocks*(d+1) partial sums, d_partial[block*(d+1)+c];
 * the caller adds the rows. fold writes d_output[i*original_size + y].
 * Stricter than the reference in one respect: the tables are read with 128-bit
 * loads, so d_polys / d_input must be 16-byte aligned and original_size even for
 * base-field tables (-2 otherwise; the reference accepts any 8-byte-aligned
 * pointer). Buffers from cuda_malloc are 256-byte aligned; only a sub-slice that
 * starts at an odd u64 offset is refused. The same holds for the extension-field
 * and almost-Goldilocks forms below. */
int sumcheck_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                               size_t half, int num_blocks);
int sumcheck_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge, int d,
                      size_t original_size, size_t half);

/* ---- sumcheck, extension field: ffi.rs:610-627 (wrapper.cu:1751-1785) ----
 * Elements are (c0, c1) pairs; original_size counts extension elements. */
int sumcheck_round_message_ext2_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                                    size_t half, int num_blocks);
int sumcheck_fold_ext2_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                           uint64_t challenge_c1, int d, size_t original_size, size_t half);

/* ---- additions: fold fused with the next round's message ----
 * One pass folds every table on the challenge and accumulates the message of
 * the following round, so a round streams the tables through HBM once.
 * `quarter` = live length / 4. Partials as in round_message (extension). */
int sumcheck_fold_round_ext2_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                                 uint64_t challenge_c1, int d, size_t original_size, size_t quarter,
                                 uint64_t* d_partial, int num_blocks);
/* base-field tables in, extension tables out */
int sumcheck_fold_round_mixed_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                                  uint64_t challenge_c1, int d, size_t original_size, size_t quarter,
                                  uint64_t* d_partial, int num_blocks);
int sumcheck_fold_mixed_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                            uint64_t challenge_c1, int d, size_t original_size, size_t half);

/* ---- addition: a round message that allocates nothing ----
 * No counterpart in the reference. For hosts that cannot let the library
 * allocate (all device memory owned by their own arena, or a loop that must not
 * take the driver's allocation lock): the per-block partial sums live in a fixed
 * array inside the library image (about 85 KB per GPU, held until exit).
 * d_message receives the d + 1 evaluations P(0..d), canonical. Limits: d <= 8,
 * half <= 2^30 (-3 beyond). First call per device resolves the array's address
 * (do it before any stream capture). Calls on one device share the array and
 * must not overlap. "Allocates nothing" holds with the library's per-kernel
 * timing off (mb_prof_enable(0), the default): with it on, every launch creates
 * two CUDA events. The resolved address is cached for the life of the process
 * and is not valid after a cudaDeviceReset of that device. */
int sumcheck_round_message_ext2_noalloc_ffi(const uint64_t* d_polys, uint64_t* d_message, int d,
                                            size_t original_size, size_t half);

/* ---- additions: whole sumcheck proof (host layer) ----
 * The loop of GpuLinearSumcheckProver::prove (zk-torch-3/src/sumcheck/gpu_prover.rs:37-90)
 * with the transcript of zk-torch-3/src/transcript.rs started as Transcript::new(label).
 * Outputs (host): round_msgs[num_var][d+1][2], challenges[num_var][2],
 * final_evals[d][2], final_eval[2], transcript_state[8] (may be NULL). */
int gl_sumcheck_prove_device_ffi(const uint64_t* d_tables, int d, int num_var, int base_field,
                                 const uint8_t* label, size_t label_len, uint64_t* round_msgs,
                                 uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval,
                                 uint64_t* transcript_state);
int gl_sumcheck_prove_host_ffi(const uint64_t* h_tables, int d, int num_var, int base_field,
                               const uint8_t* label, size_t label_len, uint64_t* round_msgs,
                               uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval,
                               uint64_t* transcript_state);
/* The verifier of the same protocol on the host (zk-torch-3/src/sumcheck/verifier.rs): *ok = 1 when every round's
 * P(0) + P(1) equals the running claim and the last claim equals final_eval. round_msgs[num_var][d+1][2],
 * claimed_sum[2], final_eval[2]; challenges[num_var][2] may be NULL. No device call. */
int gl_sumcheck_verify_ffi(const uint64_t* round_msgs, const uint64_t* final_eval, const uint64_t* claimed_sum, int d,
                           int num_var, const uint8_t* label, size_t label_len, uint64_t* challenges, int* ok);

/* ---- Poseidon2: ffi.rs:287-300 (wrapper.cu:863-964) ----
 * hash_batch permutes n width-8 states (8 words in, 8 out); compress_batch and
 * merkle_layer write permute(left || right)[0..4]. */
int poseidon2_hash_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n);
int poseidon2_compress_batch_ffi(const uint64_t* d_left, const uint64_t* d_right, uint64_t* d_output, int n);
int poseidon2_merkle_layer_ffi(const uint64_t* d_input, uint64_t* d_output, int n);

/* ---- Merkle trees: ffi.rs:549-561 (wrapper.cu:1604-1713) ----
 * d_tree holds (2 * num_leaves - 1) digests: leaves, each layer, root last. */
int poseidon2_merkle_tree_gl_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves);
int poseidon2_merkle_tree_ext2_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves);

/* ---- Monolith width 12 Merkle trees: ffi.rs:565-582 (wrapper.cu:1889-2012); CPU twins
 * goldilocks-cuda-rs/src/cpu_monolith.rs:137-211. Same tree layout and leaf inputs as above, zero-padded
 * to 12 words; digest = first four words. ---- */
int monolith_merkle_tree_gl_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves);
int monolith_merkle_tree_ext2_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves);
/* one permutation of a host state on the device (host pointers, 12 words each) */
int monolith_permute_test_ffi(const uint64_t* h_input, uint64_t* h_output);
/* addition: n width-12 states on the device, permuted out of place, canonical outputs */
int monolith_permute_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n);

/* addition, tuning hook: one layer with an explicit kernel (0: permutation per thread, 1: eight lanes per
 * permutation); asynchronous on the caller's stream */
int mb_merkle_layer_variant(const uint64_t* d_input, uint64_t* d_output, int n, int variant);

/* ---- eq tables: ffi.rs:396-410 (wrapper.cu:2040-2110) ----
 * eq(r, x) for all x, bit i of x <-> r[i]; *d_result is set to the buffer that
 * holds the table (always d_buf_a here; d_buf_b is scratch). */
int eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result);
int ext2_eq_dp_all_ffi(const uint64_t* d_r, uint64_t* d_buf_a, uint64_t* d_buf_b, int log_n, uint64_t** d_result);

/* ---- Fiat-Shamir challenger: ffi.rs:315-371 (wrapper.cu:1004-1110, cuda/challenger.cuh:42-366) ----
 * n independent duplex sponges (Poseidon2 width 8, rate 4). d_states is opaque
 * (challenger_state_size() bytes each; challenger_alloc_states returns memory to
 * release with cuda_free). observe: d_values[i] (or [i*count + k], or (c0, c1)
 * pairs); sample: d_outputs[i] (or [i*count + k]). */
int challenger_state_size(void);
int challenger_alloc_states(void** d_states, int n);
int challenger_init_states(void* d_states, int n);
int challenger_observe_ffi(void* d_states, const uint64_t* d_values, int n);
int challenger_observe_slice_ffi(void* d_states, const uint64_t* d_values, int count, int n);
int challenger_sample_ffi(void* d_states, uint64_t* d_outputs, int n);
int challenger_sample_array_ffi(void* d_states, uint64_t* d_outputs, int count, int n);
int challenger_sample_ext2_ffi(void* d_states, uint64_t* d_outputs, int n);
int challenger_sample_ext5_ffi(void* d_states, uint64_t* d_outputs, int n);
int challenger_observe_ext2_ffi(void* d_states, const uint64_t* d_values, int n);
int challenger_copy_state_to_host(void* h_state, const void* d_state);
int challenger_copy_state_to_device(void* d_state, const void* h_state);

/* ---- partial evaluation: ffi.rs:377-390 (cuda/partial_eval.cuh:113-219) ----
 * Fixes the m low variables at d_r[0..m). In place for the base field (results
 * at the start of d_data); base table in, extension challenges and output for
 * the second form. */
int partial_eval_gl_ffi(uint64_t* d_data, const uint64_t* d_r, int log_n, int m);
int partial_eval_ext2_from_gl_ffi(const uint64_t* d_input, uint64_t* d_output, const uint64_t* d_r, int log_n, int m);

/* ---- fused bit-permutation + partial evaluation: ffi.rs:657-668 (cuda/fused_permute_peval.cuh:31-120) ----
 * out[j] = sum_b evals[lo_lut[x & (2^half - 1)] | hi_lut[x >> half]] * eq[b], x = j 2^m + b; base-field
 * evals, extension eq table and output; smem_bytes is accepted for compatibility and ignored. */
int fused_permute_partial_eval_ffi(const uint64_t* d_evals, uint64_t* d_output, const uint64_t* d_eq_table, const uint32_t* d_lo_lut,
       const uint32_t* d_hi_lut, int n, int m, int half, int output_size, int smem_bytes);

/* ---- Basefold kernels: ffi.rs:416-543 (wrapper.cu:1216-1590) ---- */
int basefold_bit_reverse_gl_ffi(uint64_t* d_data, int log_n);
int basefold_bit_reverse_ext2_ffi(uint64_t* d_data, int log_n);
int basefold_bhc_interpolate_ffi(const uint64_t* d_evals, uint64_t* d_coeffs, uint64_t* d_bh_evals, int num_vars);
int basefold_encode_ffi(const uint64_t* d_coeffs, uint64_t* d_codeword, int num_vars, int log_rate);
int basefold_fold_gl_ffi(const uint64_t* d_codeword, const uint64_t* d_table, uint64_t challenge, uint64_t* d_output,
                         int pair_count);
int basefold_fold_mixed_ffi(const uint64_t* d_codeword, const uint64_t* d_table, uint64_t challenge_c0,
                            uint64_t challenge_c1, uint64_t* d_output, int pair_count);
int basefold_fold_ext2_ffi(const uint64_t* d_codeword, const uint64_t* d_table, uint64_t challenge_c0,
                           uint64_t challenge_c1, uint64_t* d_output, int pair_count);
int basefold_sumcheck_interp_gl_ffi(uint64_t* d_data, int pair_count);
int basefold_sumcheck_interp_ext2_ffi(uint64_t* d_data, int pair_count);
int basefold_sumcheck_product_gl_ffi(const uint64_t* d_eq, const uint64_t* d_bh, uint64_t* d_partial_c0,
                                     uint64_t* d_partial_c1, uint64_t* d_partial_c2, int pair_count, int num_blocks);
int basefold_sumcheck_product_mixed_ffi(const uint64_t* d_eq, const uint64_t* d_bh, uint64_t* d_partial_c0,
                                        uint64_t* d_partial_c1, uint64_t* d_partial_c2, int pair_count, int num_blocks);
int basefold_sumcheck_product_ext2_ffi(const uint64_t* d_eq, const uint64_t* d_bh, uint64_t* d_partial_c0,
                                       uint64_t* d_partial_c1, uint64_t* d_partial_c2, int pair_count, int num_blocks);
int basefold_sumcheck_eval_gl_ffi(const uint64_t* d_data, uint64_t challenge, uint64_t* d_output, int pair_count);
int basefold_sumcheck_eval_mixed_ffi(const uint64_t* d_data, uint64_t challenge_c0, uint64_t challenge_c1,
                                     uint64_t* d_output, int pair_count);
int basefold_sumcheck_eval_ext2_ffi(const uint64_t* d_data, uint64_t challenge_c0, uint64_t challenge_c1,
                                    uint64_t* d_output, int pair_count);
int fused_sumcheck_round_ext2_ffi(const uint64_t* d_eq_in, const uint64_t* d_bh_in, uint64_t challenge_c0,
                                  uint64_t challenge_c1, uint64_t* d_eq_out, uint64_t* d_bh_out,
                                  uint64_t* d_partial_c0, uint64_t* d_partial_c1, uint64_t* d_partial_c2,
                                  int pair_count, int num_blocks);
int basefold_dot_product_gl_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_partial, int n, int num_blocks);
int basefold_dot_product_mixed_ffi(const uint64_t* d_a, const uint64_t* d_b, uint64_t* d_partial, int n,
                                   int num_blocks);

/* ---- additions: Basefold host layer ----
 * The objects the reference keeps in Rust: BasefoldTable (basefold.rs:267-362),
 * BasefoldCommitment::commit_device (:382-414) and open_ext2 (:578-863) with
 * the Poseidon2 transcript of zk-torch-3/src/transcript.rs. Handles are opaque.
 * Proof layout (u64 words): eval[2] | oracles[nv][3][2] | folded_roots[nv-1][4] |
 * final_codeword[2^lr][2] | per query: index, nv value pairs [2][2], sibling
 * digests of the commitment tree bottom-up, then of each folded tree. */
size_t basefold_proof_words(int num_vars, int log_rate, int num_queries);
/* Merkle hash of commitments made after the call: 0 Poseidon2 (default), 1 Monolith. The reference fixes it
 * at build time (cargo feature "monolith", goldilocks-cuda-rs/src/basefold.rs:11-14, merkle.rs:44-47); a
 * commitment is opened with the hash it was built with. */
int basefold_set_merkle_hash(int hash);
int basefold_table_create(int num_vars, int log_rate, int num_rounds, uint64_t seed, void** table);
int basefold_table_destroy(void* table);
size_t basefold_table_entries(const void* table);
int basefold_table_download(const void* table, uint64_t* h_entries);
const uint64_t* basefold_table_level_ptr(const void* table, int level);
int basefold_commit_device(const uint64_t* d_evals, int num_vars, int log_rate, void** commitment, uint64_t* h_root);
int basefold_commit_host(const uint64_t* h_evals, int num_vars, int log_rate, void** commitment, uint64_t* h_root);
int basefold_commitment_destroy(void* commitment);
const uint64_t* basefold_commitment_codeword(const void* commitment);
const uint64_t* basefold_commitment_bh_evals(const void* commitment);
const uint64_t* basefold_commitment_tree(const void* commitment);
int basefold_open_ext2(const void* commitment, const uint64_t* h_point, const void* table, const uint8_t* label,
                       size_t label_len, int num_queries, uint64_t* h_proof, uint64_t* h_transcript_state);
int basefold_prove_host(const uint64_t* h_evals, int num_vars, int log_rate, const uint64_t* h_point,
                        const void* table, const uint8_t* label, size_t label_len, int num_queries, uint64_t* h_root,
                        uint64_t* h_proof);
/* Verifier of an opening (BasefoldProver::verify_ext2, goldilocks-cuda-rs/src/basefold.rs:1759-1925, query checks
 * :2222-2402), on the host: transcript replay, the inner sumcheck's oracle chain, and per query the commitment path,
 * the fold consistency at every round, the folded trees' paths and the final codeword. The table's (point, weight)
 * pairs at the queried positions come from the device table in one gather. merkle_hash: 0 Poseidon2, 1 Monolith,
 * negative = the current basefold_set_merkle_hash setting. *result = 0 accepted; -1 claimed value, -(10+i) oracle
 * chain at round i, -100 query index, -101 commitment path, -(200+i) fold at round i, -(300+i) folded-tree path at
 * round i, -400 final codeword. The return value reports only argument / CUDA errors. */
int basefold_verify_host(const uint64_t* h_root, int num_vars, int log_rate, const uint64_t* h_point, const void* table,
                         const uint8_t* label, size_t label_len, int num_queries, int merkle_hash,
                         const uint64_t* h_proof, int* result);
/* The same verifier with the folding table in host memory (h_table: the (point, weight) pairs as
 * basefold_table_download writes them): no device call, for a verifier on a machine without a GPU. */
int basefold_verify_with_table_host(const uint64_t* h_root, int num_vars, int log_rate, const uint64_t* h_point,
                                    const uint64_t* h_table, const uint8_t* label, size_t label_len, int num_queries,
                                    int merkle_hash, const uint64_t* h_proof, int* result);

/* ---- additions: one commitment + opening shared by several GPUs ----
 * No counterpart in the reference, which runs one whole prover per device
 * (zk-torch-3/src/commit/basefold.rs:119-146). The ranks (one host thread or
 * process per GPU) talk through an mb_exchange: a gather of a few host words per
 * round and one device all-to-all per proof. Exchange objects: threads of one
 * process (local), or processes on one machine with a mailbox in POSIX shared
 * memory for the host words and a caller-supplied device all-to-all (shm). Every
 * wait is a bounded host wait (-4 = MB_ERR_EXCHANGE when it runs out). */
typedef struct mb_exchange {
    void* ctx;
    int rank;
    int world;
    int (*all_gather_host)(void* ctx, const uint64_t* mine, size_t words, uint64_t* all);
    int (*all_to_all_device)(void* ctx, const uint64_t* d_send, uint64_t* d_recv, size_t words_per_rank);
} mb_exchange;
typedef int (*mb_all_to_all_fn)(void* ctx, const uint64_t* d_send, uint64_t* d_recv, size_t words_per_rank);
int mb_exchange_local_create(int world, mb_exchange** out /* world pointers */);
int mb_exchange_shm_create(const char* name, int rank, int world, size_t slot_words, mb_all_to_all_fn a2a, void* a2a_ctx,
                           mb_exchange** out);
int mb_exchange_destroy(mb_exchange* ex);
int mb_exchange_all_gather_host(mb_exchange* ex, const uint64_t* mine, size_t words, uint64_t* all);
int mb_exchange_all_to_all_device(mb_exchange* ex, const uint64_t* d_send, uint64_t* d_recv, size_t words_per_rank);
/* Rank r passes evaluations [r n / world, (r + 1) n / world) of the polynomial; point, table, label and query count
 * are the same on every rank. h_root and h_proof receive, on every rank, exactly the words basefold_prove_host
 * writes for the whole polynomial. world: a power of two, 2^log_rate <= world <= 16 * 2^log_rate;
 * num_vars >= log2(world) + 3 (-3 otherwise). */
int basefold_prove_sharded_device(const uint64_t* d_evals_shard, int num_vars, int log_rate, const uint64_t* h_point,
                                  const void* table, const uint8_t* label, size_t label_len, int num_queries,
                                  const mb_exchange* ex, uint64_t* h_root, uint64_t* h_proof);
int basefold_prove_sharded_host(const uint64_t* h_evals_shard, int num_vars, int log_rate, const uint64_t* h_point,
                                const void* table, const uint8_t* label, size_t label_len, int num_queries,
                                const mb_exchange* ex, uint64_t* h_root, uint64_t* h_proof);

/* ---- additions: batched degree-3 sumcheck with a shared eq table, one shard ----
 * S = sum_k alpha^k sum_x eq(t, x) a_k(x) b_k(x). d_a, d_b: [K][2^n_loc] base-field
 * slices of this shard; h_point_low: n_loc (c0, c1) pairs; h_eq_scale: eq of the
 * sharded (top) coordinates at this shard's index, (1, 0) for a single shard.
 * claims: K local shares of the per-instance sums; round_message: local share of
 * m(0..3) (4 extension elements); fold binds the low variable on the challenge;
 * finals (after n_loc folds): eq, alpha^k a_k (K), b_k (K). The caller adds the
 * shards' shares and runs the transcript (matrix_b200/sharded.py).
 * Threads: create returns with the handle's tables complete, and a handle may then
 * be used from any host thread, one call at a time. Work is queued on the calling
 * thread's stream; claims, round_message and finals wait for it, fold does not, so
 * pass a handle to another thread only after one of the waiting calls. */
int gl_batched_state_create(const uint64_t* d_a, const uint64_t* d_b, const uint64_t* h_point_low,
                            const uint64_t* h_eq_scale, int K, int n_loc, void** state);
int gl_batched_state_destroy(void* state);
int gl_batched_state_claims(void* state, uint64_t* h_claims);
int gl_batched_state_set_alpha(void* state, uint64_t c0, uint64_t c1);
int gl_batched_state_round_message(void* state, uint64_t* h_msg);
int gl_batched_state_fold(void* state, uint64_t c0, uint64_t c1);
int gl_batched_state_finals(void* state, uint64_t* h_out);
/* The whole proof over the shards of an exchange object: round loop, recombination of the ranks' shares mod p,
 * transcript (labels of zk-torch-4/src/fold/same_point_sumcheck.rs:58-157 as zk-torch-3's transcript absorbs them)
 * and the last log2(world) rounds on the host, in one call per rank; no counterpart in the reference, whose
 * sumchecks run on one GPU each. Rank r passes the slices of a_k, b_k whose top log2(world) index bits equal r:
 * d_a, d_b = [K][2^(num_vars - log2 world)]; h_point = num_vars (c0, c1) pairs, the same on every rank; world = 1
 * takes an mb_exchange_local_create(1) object. Per local round the ranks gather 8 words each through
 * all_gather_host; the kernels write their share of the round polynomial straight into pinned host memory. Outputs
 * (each may be null) are identical on every rank: h_claims [K][2], h_alpha [2], h_round_msgs [num_vars][4][2],
 * h_challenges [num_vars][2], h_finals [2K + 1][2] (eq, a_k, b_k at the challenge point), h_final_eval [2],
 * h_transcript_state [8]; h_round_us [3]: with MB_SHARD_TIMING set in the environment, microseconds per local round
 * spent waiting for the kernel, in the exchange, and in recombination + transcript; -1 otherwise.
 * -3 when num_vars - log2(world) < 1; -4 when the exchange gives up. */
int gl_batched_prove_sharded(const mb_exchange* ex, const uint64_t* d_a, const uint64_t* d_b, int K, int num_vars,
                             const uint64_t* h_point, const uint8_t* label, size_t label_len, uint64_t* h_claims,
                             uint64_t* h_alpha, uint64_t* h_round_msgs, uint64_t* h_challenges, uint64_t* h_finals,
                             uint64_t* h_final_eval, uint64_t* h_transcript_state, double* h_round_us);
/* Verifier of that proof on the host (no device call): transcript replay, P(0) + P(1) against the running claim in
 * every round (first claim sum_k alpha^k y_k), P(r) by interpolation on 0..3, and at the end the last claim against
 * eq(R) sum_k alpha^k a_k(R) b_k(R), with eq(R) recomputed from h_point and the challenges (round i binds variable
 * i). h_challenges [num_vars][2] may be null. *ok = 1 when accepted. */
int gl_batched_verify_host(int K, int num_vars, const uint64_t* h_point, const uint8_t* label, size_t label_len,
                           const uint64_t* h_claims, const uint64_t* h_round_msgs, const uint64_t* h_finals,
                           uint64_t* h_challenges, int* ok);

/* ---- additions: the host transcript (zk-torch-3/src/transcript.rs:174-350) ---- */
int gl_transcript_create(const uint8_t* label, size_t label_len, void** transcript);
int gl_transcript_destroy(void* transcript);
int gl_transcript_append_u64(void* transcript, const char* label, uint64_t v);
int gl_transcript_append_ext2(void* transcript, const char* label, uint64_t c0, uint64_t c1);
int gl_transcript_challenge_ext2(void* transcript, const char* label, uint64_t* out2);
int gl_transcript_state(const void* transcript, uint64_t* out8);

/* ---- additions: pinned memory, stream and timing helpers ---- */
int mb_host_alloc(void** ptr, size_t size);
int mb_host_free(void* ptr);
int mb_memcpy_htod_async(void* dst, const void* src, size_t size);
int mb_memcpy_dtoh_async(void* dst, const void* src, size_t size);
int mb_stream_sync(void);
/* d_out[i] = splitmix64(seed) output i + 1 mod modulus: seeded synthetic inputs made on the device */
int mb_fill_splitmix(uint64_t* d_out, size_t n, uint64_t seed, uint64_t modulus);
int mb_event_create(void** ev);
int mb_event_record(void* ev);
int mb_event_sync(void* ev);
int mb_event_elapsed_ms(void* start, void* stop, float* ms);
int mb_event_destroy(void* ev);

/* ---- additions: launch accounting and per-kernel stopwatch ----
 * mb_launch_count: kernels this library launched in the process so far.
 * With profiling on, every launch is bracketed by CUDA events on its stream;
 * the report holds "name launches total_ms" lines (returns bytes needed). */
uint64_t mb_launch_count(void);
int mb_prof_enable(int on);
int mb_prof_reset(void);
size_t mb_prof_report(char* buf, size_t cap);


/* ---- out of scope: stubs ----
 * Declared by the reference's ffi.rs but outside the prover's field-arithmetic path. Exported so that the
 * crates link unchanged: every one returns -3 (unsupported) and touches nothing (the two profiler range
 * markers are no-ops). Parameter lists are those of ffi.rs and are not repeated here. */
#ifdef __cplusplus
#define MB_STUB_ARGS ...
#else
#define MB_STUB_ARGS
#endif
int gl_einsum2(MB_STUB_ARGS);
int gl_einsum1(MB_STUB_ARGS);
int gl_scale_down(MB_STUB_ARGS);
int gl_scale_up(MB_STUB_ARGS);
int gl_decompose_bits32(MB_STUB_ARGS);
int gl_conv2d(MB_STUB_ARGS);
int gl_flatten_kernel2d(MB_STUB_ARGS);
int gl_relu_helper(MB_STUB_ARGS);
int gl_conv3d(MB_STUB_ARGS);
int gl_flatten_kernel3d(MB_STUB_ARGS);
int gl_depthwise_conv2d(MB_STUB_ARGS);

#ifdef __cplusplus
}
#endif
#endif
