// C-ABI entry points for Poseidon2 and Monolith hashing and Merkle trees
// (reference: goldilocks-cuda-rs/src/ffi.rs:287-300,549-582; definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:863-964,1604-1713,1889-2012).
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
        compress_layer_kernel<HashPoseidon2><<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    }
    return finish_sync();
}

// d_tree must hold (2 * num_leaves - 1) digests.
int poseidon2_merkle_tree_gl_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves) {
    if (num_leaves < 1) return MB_ERR_ARG;
    int rc = build_tree<HashPoseidon2, false>(d_codeword, d_tree, (size_t)num_leaves, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

int poseidon2_merkle_tree_ext2_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves) {
    if (num_leaves < 1) return MB_ERR_ARG;
    int rc = build_tree<HashPoseidon2, true>(d_codeword, d_tree, (size_t)num_leaves, MB_STREAM);
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
        compress_layer_kernel<HashPoseidon2><<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    }
    return finish_async();
}

// ---- Monolith (goldilocks-cuda-rs/src/ffi.rs:565-582; wrapper.cu:1889-2012) ------------

int monolith_merkle_tree_gl_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves) {
    if (num_leaves < 1) return MB_ERR_ARG;
    int rc = build_tree<HashMonolith, false>(d_codeword, d_tree, (size_t)num_leaves, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

int monolith_merkle_tree_ext2_ffi(const uint64_t* d_codeword, uint64_t* d_tree, int num_leaves) {
    if (num_leaves < 1) return MB_ERR_ARG;
    int rc = build_tree<HashMonolith, true>(d_codeword, d_tree, (size_t)num_leaves, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// n width-12 states on the device, permuted out of place (no reference twin; the
// reference only has the single-state test entry below).
int monolith_permute_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n) {
    if (n < 0 || !d_input || !d_output) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    {
        MB_KERNEL_ON("monolith_permute_batch", MB_STREAM);
        monolith_permute_batch_kernel<<<grid_for((size_t)n, BLOCK, 16), BLOCK, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    }
    return finish_sync();
}

// One permutation of a host state on the device (host pointers).
int monolith_permute_test_ffi(const uint64_t* h_input, uint64_t* h_output) {
    if (!h_input || !h_output) return MB_ERR_ARG;
    uint64_t* d = nullptr;
    if (pool_alloc((void**)&d, 2 * 12 * sizeof(uint64_t)) != cudaSuccess) return MB_ERR_CUDA;
    int rc = MB_OK;
    if (cudaMemcpyAsync(d, h_input, 12 * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
    if (rc == MB_OK) {
        MB_KERNEL_ON("monolith_permute_batch", MB_STREAM);
        monolith_permute_batch_kernel<<<1, 32, 0, MB_STREAM>>>(d, d + 12, 1);
    }
    if (rc == MB_OK && cudaMemcpyAsync(h_output, d + 12, 12 * sizeof(uint64_t), cudaMemcpyDeviceToHost, MB_STREAM) != cudaSuccess)
        rc = MB_ERR_CUDA;
    int rs = finish_sync();
    pool_free(d);
    return rc != MB_OK ? rc : rs;
}

}  // extern "C"
