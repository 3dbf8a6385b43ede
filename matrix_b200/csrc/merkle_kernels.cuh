// Merkle trees over Goldilocks codewords, hashed with Poseidon2 (width 8) or
// Monolith (width 12); the reference picks one at build time (cargo feature
// "monolith", goldilocks-cuda-rs/src/merkle.rs:44-47), here the hash is a
// template policy and both sets of entry points exist side by side.
//
// Tree buffer layout (goldilocks-cuda-rs/src/merkle.rs:266-280): the leaf
// digests, then every layer above them, the root last; 4 words per digest.
// Leaf k hashes the codeword pair k: permute([v0, v1, 0^6])[0..4] for base-field
// pairs, permute([a.c0, a.c1, b.c0, b.c1, 0^4])[0..4] for extension pairs; a node
// is permute(left || right)[0..4] (goldilocks-cuda-rs/src/cpu_poseidon2.rs:145-183,
// device twins goldilocks-cuda-rs/cuda/wrapper.cu:1604-1713). Monolith pads
// the same inputs with zeros to 12 words (goldilocks-cuda-rs/src/cpu_monolith.rs:150-211,
// wrapper.cu:1894-1987). Digests are written canonical.
//
// Hashing is bound by the integer pipes (about 520 modular multiplications for
// every 32-byte digest), not by HBM, so every layer is one fully parallel launch
// with one permutation per thread while the layer can fill the machine. Smaller
// layers are bound by the latency of one permutation: they spread each
// permutation over 8 lanes, and the last six are finished by a single block.
#pragma once
#include "common.cuh"
#include "gl_poseidon2.cuh"
#include "gl_monolith.cuh"

namespace mb {
namespace mk {

constexpr int BLOCK = 128;
constexpr int TAIL_NODES = 64;  // layers of at most this many nodes are finished by one block

// Hash policies. COOP: an 8-lanes-per-permutation variant exists for small layers.
struct HashPoseidon2 {
    static constexpr int WIDTH = 8;
    static constexpr bool COOP = true;
    static __device__ __forceinline__ void permute(uint64_t* s) { gl::poseidon2_permute(s); }
    static const char* leaves_name() { return "hash_leaves"; }
    static const char* layer_name() { return "compress_layer"; }
};
struct HashMonolith {
    static constexpr int WIDTH = 12;
    static constexpr bool COOP = false;
    static __device__ __forceinline__ void permute(uint64_t* s) { gl::monolith_permute(s); }
    static const char* leaves_name() { return "monolith_hash_leaves"; }
    static const char* layer_name() { return "monolith_compress_layer"; }
};

__device__ __forceinline__ void store_digest(uint64_t* out, const uint64_t* s) {
    *reinterpret_cast<ulonglong2*>(out) = make_ulonglong2(gl::canon(s[0]), gl::canon(s[1]));
    *reinterpret_cast<ulonglong2*>(out + 2) = make_ulonglong2(gl::canon(s[2]), gl::canon(s[3]));
}

template <class H, bool EXT2>
__global__ void __launch_bounds__(BLOCK)
hash_leaves_kernel(const uint64_t* __restrict__ cw, uint64_t* __restrict__ digests, size_t num_leaves) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < num_leaves; k += step) {
        uint64_t s[H::WIDTH];
        if (EXT2) {
            ulonglong2 a = *reinterpret_cast<const ulonglong2*>(cw + 4 * k);
            ulonglong2 b = *reinterpret_cast<const ulonglong2*>(cw + 4 * k + 2);
            s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y;
        } else {
            ulonglong2 a = *reinterpret_cast<const ulonglong2*>(cw + 2 * k);
            s[0] = a.x; s[1] = a.y; s[2] = 0; s[3] = 0;
        }
#pragma unroll
        for (int i = 4; i < H::WIDTH; i++) s[i] = 0;
        H::permute(s);
        store_digest(digests + 4 * k, s);
    }
}

template <class H>
__device__ __forceinline__ void compress_node(const uint64_t* in, uint64_t* out) {
    uint64_t s[H::WIDTH];
    const ulonglong2* p = reinterpret_cast<const ulonglong2*>(in);
    ulonglong2 a = p[0], b = p[1], c = p[2], d = p[3];
    s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y;
    s[4] = c.x; s[5] = c.y; s[6] = d.x; s[7] = d.y;
#pragma unroll
    for (int i = 8; i < H::WIDTH; i++) s[i] = 0;
    H::permute(s);
    store_digest(out, s);
}

// out[k] = compress(in[2k], in[2k+1]) for k < n
template <class H>
__global__ void __launch_bounds__(BLOCK)
compress_layer_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += step) compress_node<H>(in + 8 * k, out + 4 * k);
}

// Left and right children in separate arrays (poseidon2_compress_batch_ffi).
static __global__ void __launch_bounds__(BLOCK)
compress_pairs_kernel(const uint64_t* __restrict__ left, const uint64_t* __restrict__ right,
                      uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += step) {
        uint64_t s[8];
        ulonglong2 a = *reinterpret_cast<const ulonglong2*>(left + 4 * k);
        ulonglong2 b = *reinterpret_cast<const ulonglong2*>(left + 4 * k + 2);
        ulonglong2 c = *reinterpret_cast<const ulonglong2*>(right + 4 * k);
        ulonglong2 d = *reinterpret_cast<const ulonglong2*>(right + 4 * k + 2);
        s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y;
        s[4] = c.x; s[5] = c.y; s[6] = d.x; s[7] = d.y;
        gl::poseidon2_permute(s);
        store_digest(out + 4 * k, s);
    }
}

// One block finishes every layer above `layer` (of `size` <= TAIL_NODES nodes),
// one permutation per thread (hashes without an 8-lane variant).
template <class H>
__global__ void __launch_bounds__(TAIL_NODES / 2)
tree_tail_kernel(uint64_t* layer, size_t size, uint64_t* root_out, size_t stop) {
    while (size > stop) {
        uint64_t* next = layer + 4 * size;
        const size_t half = size / 2;
        if (threadIdx.x < half) compress_node<H>(layer + 8 * threadIdx.x, next + 4 * threadIdx.x);
        __syncthreads();
        layer = next;
        size = half;
    }
    if (root_out != nullptr && threadIdx.x < 4 * size) root_out[threadIdx.x] = layer[threadIdx.x];
}

// Full Monolith permutation of n width-12 states, canonical outputs.
static __global__ void __launch_bounds__(BLOCK)
monolith_permute_batch_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += step) {
        uint64_t s[12];
#pragma unroll
        for (int i = 0; i < 12; i++) s[i] = in[12 * k + i];
        gl::monolith_permute(s);
#pragma unroll
        for (int i = 0; i < 12; i++) out[12 * k + i] = gl::canon(s[i]);
    }
}

// ---- latency-oriented variants: 8 lanes per permutation ---------------------------
// Node k of the output layer is handled by 8 consecutive threads: thread l loads
// word l of the 64-byte input pair and threads 0..3 store the digest.
static __global__ void __launch_bounds__(256)
compress_layer_coop_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const int l = threadIdx.x & 7;
    const size_t groups = ((size_t)gridDim.x * blockDim.x) >> 3;
    const size_t rounds = (n + groups - 1) / groups;  // every lane of a warp runs the same trip count
    size_t k = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    for (size_t it = 0; it < rounds; it++, k += groups) {
        const bool live = k < n;
        uint64_t x = live ? in[8 * k + l] : 0;
        x = gl::poseidon2_permute_coop8(x, l);
        if (live && l < 4) out[4 * k + l] = gl::canon(x);
    }
}

template <bool EXT2>
__global__ void __launch_bounds__(256)
hash_leaves_coop_kernel(const uint64_t* __restrict__ cw, uint64_t* __restrict__ digests, size_t num_leaves) {
    constexpr int W = EXT2 ? 4 : 2;
    const int l = threadIdx.x & 7;
    const size_t groups = ((size_t)gridDim.x * blockDim.x) >> 3;
    const size_t rounds = (num_leaves + groups - 1) / groups;
    size_t k = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    for (size_t it = 0; it < rounds; it++, k += groups) {
        const bool live = k < num_leaves;
        uint64_t x = (live && l < W) ? cw[W * k + l] : 0;
        x = gl::poseidon2_permute_coop8(x, l);
        if (live && l < 4) digests[4 * k + l] = gl::canon(x);
    }
}

// One block (256 threads = 32 permutations at a time) walks every remaining
// layer above `layer` (of `size` <= 64 nodes) up to the layer of `stop` nodes (1: the root). root_out (may be null)
// receives a copy of that last layer: pinned host memory there saves the caller a copy command per tree.
static __global__ void __launch_bounds__(256)
tree_tail_coop_kernel(uint64_t* layer, size_t size, uint64_t* root_out, size_t stop) {
    __shared__ uint64_t node[64 * 4];    // the current layer, kept on chip between levels (also written to the tree)
    const int l = threadIdx.x & 7;
    const size_t g = threadIdx.x >> 3;   // 32 groups: a layer of at most 64 nodes is one pass
    if (threadIdx.x < 4 * size) node[threadIdx.x] = layer[threadIdx.x];
    __syncthreads();
    while (size > stop) {
        uint64_t* next = layer + 4 * size;
        const size_t half = size / 2;
        const bool live = g < half;
        uint64_t x = live ? node[8 * g + l] : 0;
        if (g < ((half + 3) & ~(size_t)3)) {   // only warps with a live group spend issue slots (four groups per warp)
            x = gl::poseidon2_permute_coop8(x, l);
            x = gl::canon(x);
        }
        __syncthreads();
        if (live && l < 4) {
            node[4 * g + l] = x;
            next[4 * g + l] = x;
        }
        __syncthreads();
        layer = next;
        size = half;
    }
    if (root_out != nullptr && threadIdx.x < 4 * size) root_out[threadIdx.x] = node[threadIdx.x];
}

// Up to five levels in one launch: block b takes nodes [2^levels b, 2^levels (b + 1)) of `layer` (size nodes, a
// multiple of 2^levels) and writes its 2^(levels-1), ..., 1 nodes of the layers above, so that the layer `levels`
// up (size >> levels nodes) is complete when the grid ends; last_out (may be null; device or pinned host memory)
// also receives that layer, one digest per block. What a small layer costs is not the dependent chain of a
// permutation but issue slots: eight warps of 8-lane permutations on one SM take about 8 us per level, one warp
// per scheduler about half of that. So a block holds at most 16 permutations (one warp per scheduler) and a layer
// of 4096 nodes is spread over 128 SMs; the old form (one launch per layer of 256-thread blocks, then one block for
// the last six levels) cost 136 us for the twelve top levels of every tree, this one about half. Blocks are whole
// warps (the 8-lane permutation shuffles with the full mask): threads beyond the block's groups compute on zeros
// and store nothing.
static __global__ void __launch_bounds__(128)
tree_up_coop_kernel(uint64_t* layer, size_t size, int levels, uint64_t* last_out) {
    __shared__ uint64_t node[32 * 4];    // this block's nodes of the current layer (also written to the tree)
    const int l = threadIdx.x & 7;
    const size_t g = threadIdx.x >> 3;   // up to 16 groups of 8 lanes
    size_t in_nodes = (size_t)1 << levels;   // nodes of this block in the current layer
    if (threadIdx.x < 4 * in_nodes) node[threadIdx.x] = layer[4 * ((size_t)blockIdx.x * in_nodes) + threadIdx.x];
    __syncthreads();
    size_t layer_size = size;
    uint64_t* cur = layer;
#pragma unroll 1
    for (int t = 0; t < levels; t++) {
        uint64_t* next = cur + 4 * layer_size;
        const size_t half = in_nodes / 2;
        uint64_t* dst = next + 4 * ((size_t)blockIdx.x * half);
        const bool live = g < half;      // whole warps drop out as the layers shrink
        uint64_t x = live ? node[8 * g + l] : 0;
        if (g < ((half + 3) & ~(size_t)3)) {   // warps with a live group (warp-uniform: four groups per warp)
            x = gl::poseidon2_permute_coop8(x, l);
            x = gl::canon(x);
        }
        __syncthreads();                 // every group has read its pair before the nodes are overwritten
        if (live && l < 4) {
            node[4 * g + l] = x;
            dst[4 * g + l] = x;
        }
        __syncthreads();
        cur = next;
        layer_size /= 2;
        in_nodes = half;
    }
    if (last_out != nullptr && threadIdx.x < 4) last_out[4 * (size_t)blockIdx.x + threadIdx.x] = node[threadIdx.x];
}

// Full permutation of n width-8 states (poseidon2_hash_batch_ffi).
static __global__ void __launch_bounds__(BLOCK)
permute_batch_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += step) {
        uint64_t s[8];
        const ulonglong2* p = reinterpret_cast<const ulonglong2*>(in + 8 * k);
        ulonglong2 a = p[0], b = p[1], c = p[2], d = p[3];
        s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y;
        s[4] = c.x; s[5] = c.y; s[6] = d.x; s[7] = d.y;
        gl::poseidon2_permute(s);
        store_digest(out + 8 * k, s);
        store_digest(out + 8 * k + 4, s + 4);
    }
}

// Measured on B200: a layer of up to 2^12 nodes takes 16.6 us with 8 lanes per
// permutation and 22.7 us with one permutation per thread (both are the latency
// of a single permutation); from 2^13 nodes up the per-thread kernel wins.
constexpr size_t COOP_NODES = (size_t)1 << 12;

template <class H>
inline void launch_compress_layer(const uint64_t* in, uint64_t* out, size_t n, cudaStream_t st) {
    if constexpr (H::COOP) {
        if (n <= COOP_NODES) {
            MB_KERNEL_ON("compress_layer_coop", st);
            compress_layer_coop_kernel<<<grid_for(n * 8, 256, 8), 256, 0, st>>>(in, out, n);
            return;
        }
    }
    MB_KERNEL_ON(H::layer_name(), st);
    compress_layer_kernel<H><<<grid_for(n, BLOCK, 16), BLOCK, 0, st>>>(in, out, n);
}

template <class H, bool EXT2>
inline void launch_hash_leaves(const uint64_t* cw, uint64_t* digests, size_t n, cudaStream_t st) {
    if constexpr (H::COOP) {
        if (n <= COOP_NODES) {
            MB_KERNEL_ON("hash_leaves_coop", st);
            hash_leaves_coop_kernel<EXT2><<<grid_for(n * 8, 256, 8), 256, 0, st>>>(cw, digests, n);
            return;
        }
    }
    MB_KERNEL_ON(H::leaves_name(), st);
    hash_leaves_kernel<H, EXT2><<<grid_for(n, BLOCK, 16), BLOCK, 0, st>>>(cw, digests, n);
}

template <class H>
inline void launch_tree_tail(uint64_t* layer, size_t size, cudaStream_t st, uint64_t* root_out = nullptr, size_t stop = 1) {
    MB_KERNEL_ON("tree_tail", st);
    if constexpr (H::COOP) tree_tail_coop_kernel<<<1, 256, 0, st>>>(layer, size, root_out, stop);
    else tree_tail_kernel<H><<<1, TAIL_NODES / 2, 0, st>>>(layer, size, root_out, stop);
}

// Every layer above `layer` (`size` nodes) up to the layer of `stop` nodes (1: the root; a power of two up to 32
// otherwise, for a caller that hashes the last levels on the host: a level there is bound by the latency of one
// permutation, which a host core beats). root_out (may be null; device or pinned host memory) receives that last
// layer: min(size, stop) digests. Layers of more than COOP_NODES nodes take one launch each; with an 8-lane
// permutation the rest goes five levels per launch, then one block for what is left.
template <class H>
inline void finish_layers(uint64_t* layer, size_t size, cudaStream_t st, uint64_t* root_out = nullptr, size_t stop = 1) {
    if constexpr (H::COOP) {
        while (size > COOP_NODES) {
            size_t half = size / 2;
            launch_compress_layer<H>(layer, layer + 4 * size, half, st);
            layer += 4 * size;
            size = half;
        }
        // five levels per launch (fewer in the last one), down to the layer of `stop` nodes, which the last launch
        // also copies to root_out
        while (size > stop) {
            int levels = 0;
            while (levels < 5 && (size >> levels) > stop) levels++;
            const size_t out_nodes = size >> levels;
            const unsigned threads = (unsigned)(4u << levels) < 32u ? 32u : (unsigned)(4u << levels);
            {
                MB_KERNEL_ON("tree_up", st);
                tree_up_coop_kernel<<<(unsigned)out_nodes, threads, 0, st>>>(layer, size, levels, out_nodes == stop ? root_out : nullptr);
            }
            layer += 4 * (2 * size - 2 * out_nodes);   // size + size/2 + ... + 2 out_nodes nodes
            size = out_nodes;
            if (size == stop) return;
        }
    }
    while (size > (size_t)TAIL_NODES) {
        size_t half = size / 2;
        launch_compress_layer<H>(layer, layer + 4 * size, half, st);
        layer += 4 * size;
        size = half;
    }
    if (size > 1 || stop > 1) launch_tree_tail<H>(layer, size, st, root_out, stop);
    else if (root_out != nullptr) cudaMemcpyAsync(root_out, layer, 32, cudaMemcpyDefault, st);   // a single leaf
}

// Layers above the digests already present in tree[0 .. 4*num_leaves). root_out (may be null; device or pinned
// host memory) receives a copy of the root.
template <class H>
inline int build_layers(uint64_t* d_tree, size_t num_leaves, cudaStream_t st, uint64_t* root_out = nullptr, size_t stop = 1) {
    finish_layers<H>(d_tree, num_leaves, st, root_out, stop);
    return finish_async();
}

// stop > 1: the layers above the one of `stop` nodes are left to the caller (finish_layers).
template <class H, bool EXT2>
inline int build_tree(const uint64_t* d_codeword, uint64_t* d_tree, size_t num_leaves, cudaStream_t st,
                      uint64_t* root_out = nullptr, size_t stop = 1) {
    if (!d_codeword || !d_tree || num_leaves < 1 || (num_leaves & (num_leaves - 1))) return MB_ERR_ARG;
    launch_hash_leaves<H, EXT2>(d_codeword, d_tree, num_leaves, st);
    return build_layers<H>(d_tree, num_leaves, st, root_out, stop);
}

// dst[c * words + i] = src[i] for c = 1 .. copies-1 (dst = src: in-place replication of a prefix).
static __global__ void replicate_kernel(uint64_t* base, size_t words, size_t copies) {
    const size_t pairs = words / 2, total = pairs * (copies - 1);
    const size_t step = (size_t)gridDim.x * blockDim.x;
    ulonglong2* b = reinterpret_cast<ulonglong2*>(base);
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
        size_t c = t / pairs + 1, i = t % pairs;
        b[c * pairs + i] = b[i];
    }
}

// Tree over a base-field codeword that consists of `copies` equal blocks (what
// the foldable-code encoder produces: goldilocks-cuda-rs/cuda/wrapper.cu:1277-1312
// repeats every coefficient 2^log_rate times and its butterflies never mix the
// copies, so after the bit reversal block c equals block 0). Every layer of the
// tree is then periodic too: only the first size/copies nodes of each layer are
// hashed, the rest are copied. The buffer ends up identical to build_tree's.
template <class H>
inline int build_tree_periodic(const uint64_t* d_codeword, uint64_t* d_tree, size_t num_leaves, size_t copies,
                               cudaStream_t st) {
    if (!d_codeword || !d_tree || num_leaves < 1 || (num_leaves & (num_leaves - 1))) return MB_ERR_ARG;
    if (copies < 2 || num_leaves / copies < 2 * (size_t)TAIL_NODES) return build_tree<H, false>(d_codeword, d_tree, num_leaves, st);
    size_t uniq = num_leaves / copies;
    {
        MB_KERNEL_ON(H::leaves_name(), st);
        hash_leaves_kernel<H, false><<<grid_for(uniq, BLOCK, 16), BLOCK, 0, st>>>(d_codeword, d_tree, uniq);
    }
    {
        MB_KERNEL_ON("replicate", st);
        replicate_kernel<<<grid_for(uniq * 2 * (copies - 1), 256, 8), 256, 0, st>>>(d_tree, 4 * uniq, copies);
    }
    uint64_t* layer = d_tree;
    size_t size = num_leaves;
    while (size > TAIL_NODES && size / copies >= 2) {
        size_t half = size / 2, u = half / copies;
        uint64_t* next = layer + 4 * size;
        launch_compress_layer<H>(layer, next, u, st);
        {
            MB_KERNEL_ON("replicate", st);
            replicate_kernel<<<grid_for(u * 2 * (copies - 1), 256, 8), 256, 0, st>>>(next, 4 * u, copies);
        }
        layer = next;
        size = half;
    }
    // the remaining layers are small: ordinary path on the fully populated layer
    finish_layers<H>(layer, size, st);
    return finish_async();
}

}  // namespace mk
}  // namespace mb
