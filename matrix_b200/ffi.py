"""ctypes bindings of the C-ABI (see include/*.h for the declarations)."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIBDIR = os.path.join(HERE, "lib")

c_u64 = ctypes.c_uint64
c_u64p = ctypes.POINTER(ctypes.c_uint64)
c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_size_t = ctypes.c_size_t


class LibraryMissing(RuntimeError):
    """The CUDA library has not been built; there is no fallback."""


def _load(name):
    path = os.path.join(LIBDIR, name)
    if not os.path.exists(path):
        raise LibraryMissing(
            "%s not found: build it with `python -m matrix_b200.build` (needs nvcc). "
            "This package has no CPU fallback." % path)
    return ctypes.CDLL(path)


_GL = None

# name -> (restype, argtypes); pointers to device memory are passed as integers (c_void_p)
_GL_SIGNATURES = {
    "goldilocks_cuda_init": (c_int, []),
    "poseidon2_cuda_init": (c_int, []),
    "monolith_cuda_init": (c_int, []),
    "cuda_malloc": (c_int, [ctypes.POINTER(c_void_p), c_size_t]),
    "cuda_free": (c_int, [c_void_p]),
    "mb_alloc_cache_flush": (c_int, []),
    "mb_alloc_cache_bytes": (c_size_t, []),
    "cuda_memcpy_htod": (c_int, [c_void_p, c_void_p, c_size_t]),
    "cuda_memcpy_dtoh": (c_int, [c_void_p, c_void_p, c_size_t]),
    "cuda_memcpy_dtod": (c_int, [c_void_p, c_void_p, c_size_t]),
    "cuda_device_synchronize": (c_int, []),
    "cuda_get_last_error": (c_int, []),
    "cuda_peek_at_last_error": (c_int, []),
    "cuda_mem_get_info": (c_int, [ctypes.POINTER(c_size_t), ctypes.POINTER(c_size_t)]),
    "cuda_set_device": (c_int, [c_int]),
    "cuda_get_device": (c_int, [ctypes.POINTER(c_int)]),
    "cuda_get_device_count": (c_int, [ctypes.POINTER(c_int)]),
    "cuda_get_device_name": (c_int, [c_int, ctypes.c_char_p, c_int]),
    "gl_memset_zero": (c_int, [c_void_p, c_size_t]),
    "mb_host_alloc": (c_int, [ctypes.POINTER(c_void_p), c_size_t]),
    "mb_host_free": (c_int, [c_void_p]),
    "mb_memcpy_htod_async": (c_int, [c_void_p, c_void_p, c_size_t]),
    "mb_memcpy_dtoh_async": (c_int, [c_void_p, c_void_p, c_size_t]),
    "mb_stream_sync": (c_int, []),
    "mb_fill_splitmix": (c_int, [c_void_p, c_size_t, c_u64, c_u64]),
    "mb_event_create": (c_int, [ctypes.POINTER(c_void_p)]),
    "mb_event_record": (c_int, [c_void_p]),
    "mb_event_sync": (c_int, [c_void_p]),
    "mb_event_elapsed_ms": (c_int, [c_void_p, c_void_p, ctypes.POINTER(ctypes.c_float)]),
    "mb_event_destroy": (c_int, [c_void_p]),
    "mb_launch_count": (c_u64, []),
    "mb_prof_enable": (c_int, [c_int]),
    "mb_prof_reset": (c_int, []),
    "mb_prof_report": (c_size_t, [ctypes.c_char_p, c_size_t]),
    "sumcheck_round_message_ffi": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int]),
    "sumcheck_fold_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_size_t, c_size_t]),
    "sumcheck_round_message_ext2_ffi": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int]),
    "sumcheck_fold_ext2_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t]),
    "sumcheck_fold_round_ext2_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t, c_void_p, c_int]),
    "sumcheck_fold_round_mixed_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t, c_void_p, c_int]),
    "sumcheck_fold_mixed_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t]),
    "poseidon2_hash_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "poseidon2_compress_batch_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "poseidon2_merkle_layer_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "poseidon2_merkle_tree_gl_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "poseidon2_merkle_tree_ext2_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_batch_add": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "gl_batch_sub": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "gl_batch_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "gl_batch_div": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "ext2_batch_add_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "ext2_batch_sub_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "ext2_batch_mul_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "gl_batch_inverse": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_batch_neg": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_batch_square": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_batch_double": (c_int, [c_void_p, c_void_p, c_int]),
    "ext2_batch_inverse_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext2_batch_neg_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext2_batch_square_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext2_batch_frobenius_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext2_batch_conjugate_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_to_ext2_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext2_to_gl_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_batch_mul_scalar": (c_int, [c_u64, c_void_p, c_void_p, c_int]),
    "ext2_batch_mul_scalar_ffi": (c_int, [c_u64, c_void_p, c_void_p, c_int]),
    "gl_batch_exp": (c_int, [c_void_p, c_u64, c_void_p, c_int]),
    "ext2_batch_exp_ffi": (c_int, [c_void_p, c_u64, c_void_p, c_int]),
    "ext2_scale_accumulate_ffi": (c_int, [c_u64, c_u64, c_void_p, c_void_p, c_int]),
    "ext5_batch_add_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "ext5_batch_sub_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "ext5_batch_mul_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "ext5_batch_inverse_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext5_batch_neg_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext5_batch_square_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext5_batch_frobenius_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext5_batch_mul_scalar_ffi": (c_int, [c_u64, c_void_p, c_void_p, c_int]),
    "ext5_batch_exp_ffi": (c_int, [c_void_p, c_u64, c_void_p, c_int]),
    "gl_to_ext5_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "ext5_to_gl_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "gl_zero_buffer": (c_int, [c_void_p, c_int]),
    "bit_permute_gl_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "monolith_merkle_tree_gl_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "monolith_merkle_tree_ext2_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "monolith_permute_test_ffi": (c_int, [c_void_p, c_void_p]),
    "monolith_permute_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "mb_merkle_layer_variant": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "eq_dp_all_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "ext2_eq_dp_all_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "challenger_state_size": (c_int, []),
    "challenger_alloc_states": (c_int, [ctypes.POINTER(c_void_p), c_int]),
    "challenger_init_states": (c_int, [c_void_p, c_int]),
    "challenger_observe_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "challenger_observe_slice_ffi": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "challenger_sample_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "challenger_sample_array_ffi": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "challenger_sample_ext2_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "challenger_sample_ext5_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "challenger_observe_ext2_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "challenger_copy_state_to_host": (c_int, [c_void_p, c_void_p]),
    "challenger_copy_state_to_device": (c_int, [c_void_p, c_void_p]),
    "fused_permute_partial_eval_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "partial_eval_gl_ffi": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "partial_eval_ext2_from_gl_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "basefold_bit_reverse_gl_ffi": (c_int, [c_void_p, c_int]),
    "basefold_bit_reverse_ext2_ffi": (c_int, [c_void_p, c_int]),
    "basefold_bhc_interpolate_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "basefold_encode_ffi": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "basefold_fold_gl_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_void_p, c_int]),
    "basefold_fold_mixed_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_void_p, c_int]),
    "basefold_fold_ext2_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_void_p, c_int]),
    "basefold_sumcheck_interp_gl_ffi": (c_int, [c_void_p, c_int]),
    "basefold_sumcheck_interp_ext2_ffi": (c_int, [c_void_p, c_int]),
    "basefold_sumcheck_product_gl_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "basefold_sumcheck_product_mixed_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "basefold_sumcheck_product_ext2_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "basefold_sumcheck_eval_gl_ffi": (c_int, [c_void_p, c_u64, c_void_p, c_int]),
    "basefold_sumcheck_eval_mixed_ffi": (c_int, [c_void_p, c_u64, c_u64, c_void_p, c_int]),
    "basefold_sumcheck_eval_ext2_ffi": (c_int, [c_void_p, c_u64, c_u64, c_void_p, c_int]),
    "fused_sumcheck_round_ext2_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int]),
    "basefold_dot_product_gl_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "basefold_dot_product_mixed_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "basefold_proof_words": (c_size_t, [c_int, c_int, c_int]),
    "basefold_set_merkle_hash": (c_int, [c_int]),
    "basefold_table_create": (c_int, [c_int, c_int, c_int, c_u64, ctypes.POINTER(c_void_p)]),
    "basefold_table_destroy": (c_int, [c_void_p]),
    "basefold_table_entries": (c_size_t, [c_void_p]),
    "basefold_table_download": (c_int, [c_void_p, c_void_p]),
    "basefold_table_level_ptr": (c_void_p, [c_void_p, c_int]),
    "basefold_commit_device": (c_int, [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), c_void_p]),
    "basefold_commit_host": (c_int, [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), c_void_p]),
    "basefold_commitment_destroy": (c_int, [c_void_p]),
    "basefold_commitment_codeword": (c_void_p, [c_void_p]),
    "basefold_commitment_bh_evals": (c_void_p, [c_void_p]),
    "basefold_commitment_tree": (c_void_p, [c_void_p]),
    "basefold_open_ext2": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_char_p, c_size_t, c_int, c_void_p, c_void_p]),
    "basefold_prove_host": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_char_p, c_size_t, c_int,
                                    c_void_p, c_void_p]),
    "basefold_verify_host": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_char_p, c_size_t, c_int, c_int,
                                     c_void_p, ctypes.POINTER(c_int)]),
    "basefold_verify_with_table_host": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_char_p, c_size_t, c_int,
                                                c_int, c_void_p, ctypes.POINTER(c_int)]),
    "mb_exchange_local_create": (c_int, [c_int, ctypes.POINTER(c_void_p)]),
    "mb_exchange_shm_create": (c_int, [ctypes.c_char_p, c_int, c_int, c_size_t, c_void_p, c_void_p, ctypes.POINTER(c_void_p)]),
    "mb_exchange_destroy": (c_int, [c_void_p]),
    "mb_exchange_all_gather_host": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "mb_exchange_all_to_all_device": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "basefold_prove_sharded_device": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_char_p, c_size_t, c_int,
                                              c_void_p, c_void_p, c_void_p]),
    "basefold_prove_sharded_host": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_char_p, c_size_t, c_int,
                                            c_void_p, c_void_p, c_void_p]),
    "sumcheck_round_message_ext2_noalloc_ffi": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t]),
    "gl_batched_state_create": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(c_void_p)]),
    "gl_batched_state_destroy": (c_int, [c_void_p]),
    "gl_batched_state_claims": (c_int, [c_void_p, c_void_p]),
    "gl_batched_state_set_alpha": (c_int, [c_void_p, c_u64, c_u64]),
    "gl_batched_state_round_message": (c_int, [c_void_p, c_void_p]),
    "gl_batched_state_fold": (c_int, [c_void_p, c_u64, c_u64]),
    "gl_batched_state_finals": (c_int, [c_void_p, c_void_p]),
    "gl_batched_prove_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, ctypes.c_char_p, c_size_t,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gl_batched_verify_host": (c_int, [c_int, c_int, c_void_p, ctypes.c_char_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p,
                                       ctypes.POINTER(c_int)]),
    "gl_transcript_create": (c_int, [ctypes.c_char_p, c_size_t, ctypes.POINTER(c_void_p)]),
    "gl_transcript_destroy": (c_int, [c_void_p]),
    "gl_transcript_append_u64": (c_int, [c_void_p, ctypes.c_char_p, c_u64]),
    "gl_transcript_append_ext2": (c_int, [c_void_p, ctypes.c_char_p, c_u64, c_u64]),
    "gl_transcript_challenge_ext2": (c_int, [c_void_p, ctypes.c_char_p, c_void_p]),
    "gl_transcript_state": (c_int, [c_void_p, c_void_p]),
    "gl_sumcheck_prove_device_ffi": (c_int, [c_void_p, c_int, c_int, c_int, ctypes.c_char_p, c_size_t,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gl_sumcheck_prove_host_ffi": (c_int, [c_void_p, c_int, c_int, c_int, ctypes.c_char_p, c_size_t,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gl_sumcheck_verify_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_char_p, c_size_t, c_void_p,
                                       ctypes.POINTER(c_int)]),
}


def load_gl():
    """The Goldilocks library with argument types set. Raises LibraryMissing if it was not built."""
    global _GL
    if _GL is None:
        lib = _load("libgoldilocks_cuda_wrapper.so")
        for name, (res, args) in _GL_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _GL = lib
    return _GL


_AGL = None
_MEM = ["cuda_malloc", "cuda_free", "mb_alloc_cache_flush", "mb_alloc_cache_bytes", "cuda_memcpy_htod", "cuda_memcpy_dtoh", "cuda_memcpy_dtod", "cuda_device_synchronize",
        "cuda_get_last_error", "cuda_peek_at_last_error", "cuda_mem_get_info", "cuda_set_device", "cuda_get_device",
        "cuda_get_device_count", "mb_event_create", "mb_event_record", "mb_event_sync", "mb_event_elapsed_ms",
        "mb_event_destroy", "mb_stream_sync", "mb_launch_count", "mb_fill_splitmix", "mb_host_alloc", "mb_host_free",
        "mb_memcpy_htod_async", "mb_memcpy_dtoh_async", "mb_prof_enable", "mb_prof_reset", "mb_prof_report", "gl_memset_zero",
        "cuda_get_device_name"]
_AGL_SIGNATURES = {
    "almost_goldilocks_cuda_init": (c_int, []),
    "agl_batch_add_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "agl_batch_sub_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "agl_batch_mul_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "agl_batch_inverse_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "aext2_batch_mul_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "aext2_batch_inverse_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "agl_sumcheck_round_message_ffi": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int]),
    "agl_sumcheck_fold_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_size_t, c_size_t]),
    "aext2_sumcheck_round_message_ffi": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int]),
    "aext2_sumcheck_fold_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t]),
    "aext2_sumcheck_fold_round_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t, c_void_p, c_int]),
    "aext2_sumcheck_fold_round_mixed_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_size_t, c_size_t, c_void_p, c_int]),
    "agl_eq_dp_all_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "aext2_eq_dp_all_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "ajtai_commit_dense_batched_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_int, c_void_p]),
    "ajtai_commit_dense_batched_at_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_int, c_u64, c_void_p]),
    "ajtai_commit_wide_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_int, c_void_p]),
    "ajtai_materialize_m_ffi": (c_int, [c_void_p, c_void_p, c_u64]),
    "ajtai_commit_s8_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_u64, c_void_p]),
    "ajtai_commit_s8_premat_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "ajtai_tc_matrix_bytes": (c_u64, [c_u64]),
    "ajtai_materialize_tc_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64]),
    "ajtai_commit_s8_tiled_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "ajtai_commit_s8_scalar_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_u64, c_void_p]),
    "ajtai_fold_witness_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "ajtai_fold_commitment_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "ajtai_multifold_commitment_ffi": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "ajtai_multifold_witness_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_u64, c_u64]),
    "ajtai_multifold_mixed_witness_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_u64, c_u64]),
    "ajtai_multifold_mixed_witness_tc_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_u64]),
    "ajtai_multifold_mixed_witness_tc_fused_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_u64]),
    "ajtai_multifold_mixed_witness_scalar_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_u64]),
    "ajtai_split_witness_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64]),
    "ajtai_commit_ternary_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "ajtai_commit_ternary_premat_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "ajtai_commit_sparse_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "aext2_wide_to_ternary_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int]),
    "agl_batch_div_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "aext2_batch_add_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "aext2_batch_sub_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "agl_batch_neg_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "agl_batch_square_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "agl_batch_double_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "aext2_batch_neg_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "aext2_batch_square_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "aext2_batch_frobenius_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "aext2_batch_conjugate_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "agl_to_aext2_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "aext2_to_agl_batch_ffi": (c_int, [c_void_p, c_void_p, c_int]),
    "agl_batch_mul_scalar_ffi": (c_int, [c_u64, c_void_p, c_void_p, c_int]),
    "aext2_batch_mul_scalar_ffi": (c_int, [c_u64, c_void_p, c_void_p, c_int]),
    "agl_batch_exp_ffi": (c_int, [c_void_p, c_u64, c_void_p, c_int]),
    "aext2_batch_exp_ffi": (c_int, [c_void_p, c_u64, c_void_p, c_int]),
    "aext2_scale_accumulate_ffi": (c_int, [c_u64, c_u64, c_void_p, c_void_p, c_int]),
    "agl_zero_buffer_ffi": (c_int, [c_void_p, c_size_t]),
    "agl_bit_permute_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "agl_cuda_error_string": (ctypes.c_char_p, [c_int]),
    "cuda_memset": (c_int, [c_void_p, c_int, c_size_t]),
    "cuda_sync_mine": (c_int, []),
    "cuda_stream_create": (c_int, [ctypes.POINTER(c_void_p)]),
    "cuda_stream_destroy": (c_int, [c_void_p]),
    "cuda_stream_synchronize": (c_int, [c_void_p]),
    "cuda_memcpy_dtod_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "cuda_memcpy_htod_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "cuda_memcpy_peer": (c_int, [c_void_p, c_int, c_void_p, c_int, c_size_t]),
    "cuda_enable_peer_access": (c_int, [c_int]),
    "cuda_pool_trim": (c_int, [c_size_t]),
    "agl_cached_bytes": (c_size_t, []),
    "agl_d2h_staged": (c_int, [c_void_p, c_void_p, c_size_t]),
    "agl_h2d_staged": (c_int, [c_void_p, c_void_p, c_size_t]),
    "aext2_sumcheck_batched_round_message_ffi": (c_int, [c_void_p, c_void_p, c_size_t, c_size_t, c_int, c_int]),
    "aext2_sumcheck_batched_fold_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_size_t, c_size_t, c_int]),
    "aext2_sumcheck_batched_round0_binary_msg_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_int, c_int, c_size_t]),
    "aext2_sumcheck_batched_round0_binary_fold_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_size_t, c_size_t, c_int, c_size_t]),
    "aext2_sharedeq_msg_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_int, c_int]),
    "aext2_fold_single_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_size_t, c_size_t, c_int]),
    "aext2_eq_suffix_dp_ffi": (c_int, [c_void_p, c_void_p, c_int, c_int, c_size_t]),
    "aext2_sharedeq_factored_msg_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_size_t, c_int, c_int]),
    "aext2_build_fu_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_size_t]),
    "aext2_build_fu_ternary_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_size_t]),
    "aext2_batched_lift_binary_ffi": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_size_t]),
    "aext2_lift_binary_contig_ffi": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_size_t]),
    "aext2_batched_lift_ternary_single_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_size_t]),
    "aext2_selective_add_batched_planes_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_size_t, c_int]),
    "aext2_eq_dp_all_stream_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(c_void_p), c_void_p]),
    "aext2_eq_dp_all_batched_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "agl_mpiop_sc_round": (c_int, [c_void_p, c_int, c_u64, c_int, c_void_p]),
    "agl_mpiop_sc_fold": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "agl_mpiop_sc_fold_round": (c_int, [c_void_p, c_void_p, c_int, c_u64, c_void_p, c_int, c_void_p]),
    "agl_mpiop_eq": (c_int, [c_void_p, c_int, c_void_p]),
    "agl_mpiop_eq_outer": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "agl_mpiop_axpy": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "agl_mpiop_lift": (c_int, [c_void_p, c_u64, c_void_p]),
    "agl_mpiop_pe": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "agl_mpiop_mle": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "agl_mpiop_gather": (c_int, [c_void_p, c_void_p, c_int, c_u64, c_void_p]),
    "agl_mpiop_sel_lookup": (c_int, [c_void_p, c_u64, c_int, c_u64, c_void_p, c_void_p]),
    "agl_mcommit_keygen": (c_int, [c_void_p, ctypes.c_uint32, c_int, c_u64, c_int, c_int, c_void_p]),
    "agl_mcommit_partial": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_u64, c_void_p, c_void_p]),
    "agl_mcommit_add": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int]),
    "agl_mcommit_finish": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "link_round_message_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64, c_u64, c_int, c_void_p, c_u64, c_void_p]),
    "link_round_message_sparse_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64,
                                              c_u64, c_int, c_void_p, c_u64, c_void_p]),
    "link_round0_bits_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64, c_void_p, c_u64, c_void_p]),
    "link_round0_bits_sparse_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64,
                                            c_void_p, c_u64, c_void_p]),
    "link_round_interleaved_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_u64, c_u64, c_u64, c_u64, ctypes.c_uint32, c_int, c_int, c_int, c_int, c_void_p, c_u64,
                                           c_void_p]),
    "link_fold_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_u64, c_u64, c_u64, c_u64]),
    "link_fold_sparse_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64, c_u64, c_u64]),
    "link_fold0_bits_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64, c_u64, c_u64]),
    "link_fold_w_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_u64, c_u64, c_u64, c_int, c_u64, c_u64]),
    "link_eq_expand_ffi": (c_int, [c_void_p, c_u64, c_u64, c_u64]),
    "link_omega_expand_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u64]),
    "link_expand_bits_ffi": (c_int, [c_void_p, c_void_p, c_u64]),
    "link_eq_gather_ffi": (c_int, [c_void_p, c_u64, c_void_p, c_void_p, c_u64]),
    "agl_bool_init_val_ffi": (c_int, [c_void_p, c_size_t]),
    "agl_bool_round_msg_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_int,
                                       c_void_p, c_size_t, c_void_p, c_void_p]),
    "agl_bool_fold_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_u64, c_u64, ctypes.c_uint32, c_int,
                                  c_void_p, c_void_p, c_void_p]),
    "agl_bool_finish_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_void_p]),
    "agl_monolith_permute_host": (c_int, [c_void_p]),
    "agl_monolith_round_constants": (c_int, [c_void_p]),
    "agl_transcript_create": (c_int, [ctypes.c_char_p, c_size_t, ctypes.POINTER(c_void_p)]),
    "agl_transcript_destroy": (c_int, [c_void_p]),
    "agl_transcript_fork": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, c_u64, ctypes.POINTER(c_void_p)]),
    "agl_transcript_append_scalar": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, c_u64]),
    "agl_transcript_append_u64": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, c_u64]),
    "agl_transcript_append_u64_slice": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, c_void_p, c_size_t]),
    "agl_transcript_append_ext2": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, c_u64, c_u64]),
    "agl_transcript_challenge_scalar": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, ctypes.POINTER(ctypes.c_uint64)]),
    "agl_transcript_challenge_vector": (c_int, [c_void_p, ctypes.c_char_p, c_size_t, c_void_p, c_size_t]),
    "agl_transcript_state": (c_int, [c_void_p, c_void_p]),
    "agl_same_point_prove_device_ffi": (c_int, [c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_void_p, c_void_p]),
    "aext2_sumcheck_batched_fold_message_ffi": (c_int, [c_void_p, c_void_p, c_u64, c_u64, c_size_t, c_size_t, c_int, c_int, c_void_p]),
    "aext2_sumcheck_batched_round0_binary_fold_message_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u64, c_size_t, c_size_t,
                                                                      c_int, c_int, c_size_t, c_void_p]),
    "agl_einsum_prove_device_ffi": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_void_p]),
    "agl_same_point_claims_device_ffi": (c_int, [c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "agl_same_point_verify_ffi": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, ctypes.POINTER(c_int)]),
    "agl_sumcheck_prove_device_ffi": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "agl_sumcheck_prove_host_ffi": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "agl_sumcheck_verify_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.POINTER(c_int)]),
    "agl_fused_permute_partial_eval_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "agl_partial_eval_ffi": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "agl_partial_eval_ext2_from_base_ffi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int]),
}


def load_agl():
    """The almost-Goldilocks library with argument types set. Raises LibraryMissing if it was not built."""
    global _AGL
    if _AGL is None:
        lib = _load("libalmost_goldilocks_cuda_wrapper.so")
        sigs = dict(_AGL_SIGNATURES)
        for name in _MEM:
            sigs[name] = _GL_SIGNATURES[name]
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _AGL = lib
    return _AGL


def agl_signatures():
    return dict(_AGL_SIGNATURES)


def gl_signatures():
    return dict(_GL_SIGNATURES)


class DeviceBuffer:
    """A caller-owned device allocation obtained from the library's cuda_malloc
    (the role of DeviceBuffer<u64> in goldilocks-cuda-rs/src/memory.rs)."""

    def __init__(self, lib, nbytes):
        self.lib = lib
        self.nbytes = int(nbytes)
        p = c_void_p()
        if self.nbytes > 0:
            rc = lib.cuda_malloc(ctypes.byref(p), self.nbytes)
            if rc != 0:
                raise MemoryError("cuda_malloc(%d) failed: %d" % (self.nbytes, rc))
        self.ptr = p.value or 0

    @classmethod
    def from_numpy(cls, lib, arr):
        import numpy as np
        arr = np.ascontiguousarray(arr)
        buf = cls(lib, arr.nbytes)
        if arr.nbytes:
            rc = lib.cuda_memcpy_htod(buf.ptr, arr.ctypes.data, arr.nbytes)
            if rc != 0:
                raise RuntimeError("cuda_memcpy_htod failed: %d" % rc)
        return buf

    def to_numpy(self, dtype="uint64", count=None, offset_bytes=0):
        import numpy as np
        dt = np.dtype(dtype)
        if count is None:
            count = (self.nbytes - offset_bytes) // dt.itemsize
        out = np.empty(count, dtype=dt)
        if out.nbytes:
            rc = self.lib.cuda_memcpy_dtoh(out.ctypes.data, self.ptr + offset_bytes, out.nbytes)
            if rc != 0:
                raise RuntimeError("cuda_memcpy_dtoh failed: %d" % rc)
        return out

    def free(self):
        if self.ptr:
            self.lib.cuda_free(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
