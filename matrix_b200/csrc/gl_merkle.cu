// C-ABI entry points for Poseidon2 hashing and Merkle trees (reference:
// goldilocks-cuda-rs/src/ffi.rs:287-300,549-561; definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:863-964,1604-1713).
#include "merkle_kernels.cuh"

using namespace mb;
using namespace mb::mk;

extern "C" {

// n width-8 states in, n permuted states out.
int poseidon2_hash_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n) {
    if (n < 0 || !d_input || !d_output) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL_ON("permute_batch", MB_STREAM);
        permute_batch_kernel<<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    }
    return finish_sync();
}

int poseidon2_compress_batch_ffi(const uint64_t* d_left, const uint64_t* d_right, uint64_t* d_output, int n) {
    if (n < 0 || !d_left || !d_right || !d_output) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL_ON("compress_pairs", MB_STREAM);
        compress_pairs_kernel<<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_left, d_right, d_output, (size_t)n);
    }
    return finish_sync();
}

// n output nodes from 2n input digests.
int poseidon2_merkle_layer_ffi(const uint64_t* d_input, uint64_t* d_output, int n) {
    if (n < 0 || !d_input || !d_output) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL_ON("compress_layer", MB_STREAM);
        compress_layer_kernel<<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    }
    return finish_sync();
}

// d_tree must hold (2 * num_leaves - 1) digests.
int poseidon2_merkle_tree_gl_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves) {
    if (num_leaves < 1) return MB_ERR_ARG;
    int rc = build_tree<false>(d_codeword, d_tree, (size_t)num_leaves, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

int poseidon2_merkle_tree_ext2_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves) {
    if (num_leaves < 1) return MB_ERR_ARG;
    int rc = build_tree<true>(d_codeword, d_tree, (size_t)num_leaves, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// Tuning hook: one Merkle layer with an explicit kernel choice
// (0 = one permutation per thread, 1 = eight lanes per permutation). No sync.
int mb_merkle_layer_variant(const uint64_t* d_input, uint64_t* d_output, int n, int variant) {
    if (n < 1 || !d_input || !d_output) return MB_ERR_ARG;
    if (variant == 1) {
        MB_KERNEL("compress_layer_coop");
        compress_layer_coop_kernel<<<grid_for((size_t)n * 8, 256, 8), 256, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    } else {
        MB_KERNEL("compress_layer");
        compress_layer_kernel<<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    }
    return finish_async();
}

}  // extern "C"
