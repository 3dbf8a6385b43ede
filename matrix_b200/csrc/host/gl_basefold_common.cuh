// Shared by the single-GPU and the sharded Basefold host layers: device buffers, the kernels of the
// opening's inner sumcheck and query phase, the folding table and the commitment object.
//
//   BasefoldTable        goldilocks-cuda-rs/src/basefold.rs:267-362
//   DeviceMerkleTree     goldilocks-cuda-rs/src/merkle.rs:20-160
//   BasefoldCommitment   goldilocks-cuda-rs/src/basefold.rs:368-414 (commit_device)
#pragma once
#include <cstring>
#include <memory>
#include <atomic>
#include <vector>
#include "../basefold_kernels.cuh"
#include "../eq_kernels.cuh"
#include "../merkle_kernels.cuh"
#include "host_tree_top.hpp"
#include "gl_transcript.hpp"

namespace mb {
namespace bf {
int interpolate_async(const uint64_t*, uint64_t*, uint64_t*, int, cudaStream_t);
int encode_async(const uint64_t*, uint64_t*, uint64_t*, int, int, cudaStream_t);
}  // namespace bf
}  // namespace mb

using namespace mb;

namespace mbhost {

// ---- small RAII device buffer ----------------------------------------------------
struct DevBuf {
    uint64_t* p = nullptr;
    size_t words = 0;
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    ~DevBuf() { release(); }
    int alloc(size_t w) {
        release();
        words = w;
        if (w == 0) return MB_OK;
        return pool_alloc(reinterpret_cast<void**>(&p), w * sizeof(uint64_t)) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    }
    void release() {
        pool_free(p);
        p = nullptr;
        words = 0;
    }
};

// ---- kernels private to the host layer ---------------------------------------------

// weights[k] = 1 / weights[k] for the (point, weight) table.
static __global__ void table_invert_kernel(uint64_t* table, size_t entries) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < entries; k += step)
        table[2 * k + 1] = gl::canon(gl::inv(table[2 * k + 1]));
}

// Oracle of the opening's inner sumcheck from tables in value form:
// with e = (eq[2j], eq[2j+1] - eq[2j]) and b likewise,
// c0 = sum e0 b0, c1 = sum (e0 b1 + e1 b0), c2 = sum e1 b1
// (the coefficients cuda/basefold.cuh:334-383 computes after its in-place
// interp step). BH_BASE: bh holds base-field values.
template <bool BH_BASE>
__device__ __forceinline__ void oracle_accumulate(gl::E2 q0, gl::E2 q1, gl::E2 b0, gl::E2 b1, gl::E2& a0, gl::E2& a1,
                                                  gl::E2& a2) {
    gl::E2 qd = gl::e2_sub(q1, q0), bd = gl::e2_sub(b1, b0);
    if (BH_BASE) {
        a0 = gl::e2_add(a0, gl::e2_mul_base(q0, b0.c0));
        a1 = gl::e2_add(a1, gl::e2_add(gl::e2_mul_base(q0, bd.c0), gl::e2_mul_base(qd, b0.c0)));
        a2 = gl::e2_add(a2, gl::e2_mul_base(qd, bd.c0));
    } else {
        a0 = gl::e2_add(a0, gl::e2_mul(q0, b0));
        a1 = gl::e2_add(a1, gl::e2_add(gl::e2_mul(q0, bd), gl::e2_mul(qd, b0)));
        a2 = gl::e2_add(a2, gl::e2_mul(qd, bd));
    }
}

// Block partials, then the last block to finish adds them up into final_out[6].
__device__ __forceinline__ void oracle_finish(gl::E2 a0, gl::E2 a1, gl::E2 a2, uint64_t* partial, unsigned int* counter,
                                              uint64_t* final_out) {
    uint64_t v[6] = {a0.c0, a0.c1, a1.c0, a1.c1, a2.c0, a2.c1};
    sc::block_sum_store<6>(v, partial + 6 * (size_t)blockIdx.x, sc::GlAdd(), sc::GlCanon());
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll
    for (int k = 0; k < 6; k++) v[k] = 0;
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x)
#pragma unroll
        for (int k = 0; k < 6; k++) v[k] = gl::add(v[k], __ldcg(partial + 6 * (size_t)b + k));
    sc::block_sum_store<6>(v, final_out, sc::GlAdd(), sc::GlCanon());
    if (threadIdx.x == 0) *counter = 0;
}

// First oracle: eq (extension) x bh (base), both of length 2 * pairs.
static __global__ void __launch_bounds__(256)
oracle0_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ bh, size_t pairs, uint64_t* partial,
               unsigned int* counter, uint64_t* final_out) {
    gl::E2 a0{0, 0}, a1{0, 0}, a2{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < pairs; j += step) {
        gl::E2 q0 = gl::e2_load(eq + 4 * j), q1 = gl::e2_load(eq + 4 * j + 2);
        ulonglong2 b = *reinterpret_cast<const ulonglong2*>(bh + 2 * j);
        oracle_accumulate<true>(q0, q1, gl::E2{b.x, 0}, gl::E2{b.y, 0}, a0, a1, a2);
    }
    oracle_finish(a0, a1, a2, partial, counter, final_out);
}

// One round: fold eq and bh on r (four inputs -> two outputs each) and
// accumulate the oracle of the folded tables. BH_BASE: bh_in is base field
// (round 0); outputs are always extension elements.
template <bool BH_BASE>
__global__ void __launch_bounds__(256)
open_round_kernel(const uint64_t* __restrict__ eq_in, const uint64_t* __restrict__ bh_in, gl::E2 r,
                  uint64_t* __restrict__ eq_out, uint64_t* __restrict__ bh_out, size_t quarter, uint64_t* partial,
                  unsigned int* counter, uint64_t* final_out) {
    gl::E2 a0{0, 0}, a1{0, 0}, a2{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t y = (size_t)blockIdx.x * blockDim.x + threadIdx.x; y < quarter; y += step) {
        const uint64_t* pe = eq_in + 8 * y;
        gl::E2 e0 = gl::e2_load(pe), e1 = gl::e2_load(pe + 2), e2 = gl::e2_load(pe + 4), e3 = gl::e2_load(pe + 6);
        gl::E2 q0 = gl::e2_add(e0, gl::e2_mul(r, gl::e2_sub(e1, e0)));
        gl::E2 q1 = gl::e2_add(e2, gl::e2_mul(r, gl::e2_sub(e3, e2)));
        gl::E2 b0, b1;
        if (BH_BASE) {
            ulonglong2 u = *reinterpret_cast<const ulonglong2*>(bh_in + 4 * y);
            ulonglong2 w = *reinterpret_cast<const ulonglong2*>(bh_in + 4 * y + 2);
            uint64_t d0 = gl::sub(u.y, u.x), d1 = gl::sub(w.y, w.x);
            b0 = gl::E2{gl::add(u.x, gl::mul(r.c0, d0)), gl::mul(r.c1, d0)};
            b1 = gl::E2{gl::add(w.x, gl::mul(r.c0, d1)), gl::mul(r.c1, d1)};
        } else {
            const uint64_t* pb = bh_in + 8 * y;
            gl::E2 f0 = gl::e2_load(pb), f1 = gl::e2_load(pb + 2), f2 = gl::e2_load(pb + 4), f3 = gl::e2_load(pb + 6);
            b0 = gl::e2_add(f0, gl::e2_mul(r, gl::e2_sub(f1, f0)));
            b1 = gl::e2_add(f2, gl::e2_mul(r, gl::e2_sub(f3, f2)));
        }
        q0 = gl::e2_canon(q0); q1 = gl::e2_canon(q1); b0 = gl::e2_canon(b0); b1 = gl::e2_canon(b1);
        gl::e2_store(eq_out + 4 * y, q0);
        gl::e2_store(eq_out + 4 * y + 2, q1);
        gl::e2_store(bh_out + 4 * y, b0);
        gl::e2_store(bh_out + 4 * y + 2, b1);
        oracle_accumulate<false>(q0, q1, b0, b1, a0, a1, a2);
    }
    oracle_finish(a0, a1, a2, partial, counter, final_out);
}

// Query phase: every value pair and authentication path of every query in
// one launch. Block q handles query q; out is the per-query part of the proof.
struct QueryLevels {
    int nv, lr;
    const uint64_t* commit_cw;    // base-field codeword
    const uint64_t* commit_tree;  // its tree
    const uint64_t* fcw[40];      // folded codewords (extension)
    const uint64_t* ftree[40];    // their trees
};

__device__ __forceinline__ void copy_path(const uint64_t* tree, size_t num_leaves, size_t leaf, uint64_t* out) {
    // layer l starts at 4 * (2 * num_leaves - (num_leaves >> (l - 1))) for l >= 1
    int depth = 0;
    for (size_t s = num_leaves; s > 1; s >>= 1) depth++;
    for (int t = threadIdx.x; t < depth * 4; t += blockDim.x) {
        int l = t >> 2, w = t & 3;
        size_t off = 2 * num_leaves - ((2 * num_leaves) >> l);  // digests before layer l
        size_t sib = (leaf >> l) ^ 1;
        out[t] = tree[4 * (off + sib) + w];
    }
}

static __global__ void query_gather_kernel(QueryLevels lv, const uint64_t* __restrict__ leaf_idx, uint64_t* __restrict__ out,
                                    size_t qwords) {
    const int nv = lv.nv, lr = lv.lr;
    uint64_t* pq = out + (size_t)blockIdx.x * qwords;
    const size_t leaf = (size_t)leaf_idx[blockIdx.x];
    uint64_t* vals = pq + 1;
    if (threadIdx.x == 0) {
        pq[0] = leaf;
        vals[0] = lv.commit_cw[2 * leaf];
        vals[1] = 0;
        vals[2] = lv.commit_cw[2 * leaf + 1];
        vals[3] = 0;
    }
    for (int t = threadIdx.x; t < (nv - 1) * 4; t += blockDim.x) {
        int i = t >> 2, w = t & 3;
        size_t idx = leaf >> (i + 1);
        vals[4 * (i + 1) + w] = lv.fcw[i][4 * idx + w];
    }
    uint64_t* pp = vals + 4 * nv;
    size_t leaves = (size_t)1 << (nv + lr - 1);
    copy_path(lv.commit_tree, leaves, leaf, pp);
    pp += 4 * (nv + lr - 1);
    for (int i = 0; i <= nv - 2; i++) {
        size_t fl = (size_t)1 << (nv + lr - 2 - i);
        copy_path(lv.ftree[i], fl, leaf >> (i + 1), pp);
        pp += 4 * (nv + lr - 2 - i);
    }
}

// ---- BasefoldTable ------------------------------------------------------------------
class BasefoldTable {
public:
    // basefold.rs:281-321: xorshift64 (13, 7, 17) mod p; x1 redrawn while equal
    // to x0; weight = 1 / (x1 - x0). The stream is sequential and runs on the
    // host; the inversions run on the device.
    int generate(int nv, int lr, int num_rounds, uint64_t seed) {
        if (nv < 1 || lr < 0 || num_rounds < 1 || num_rounds > nv || nv + lr > 34) return MB_ERR_ARG;
        num_vars = nv; log_rate = lr; rounds = num_rounds;
        level_offsets.clear(); level_sizes.clear();
        size_t total = 0;
        for (int i = 0; i < num_rounds; i++) {
            level_offsets.push_back(total);
            level_sizes.push_back((size_t)1 << (nv + lr - i - 1));
            total += level_sizes.back();
        }
        entries = total;
        uint64_t* h = nullptr;
        MB_CUDA(cudaMallocHost(&h, total * 2 * sizeof(uint64_t)));
        uint64_t s = seed;
        auto next = [&s]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s % gl::P; };
        for (size_t k = 0; k < total; k++) {
            uint64_t x0 = next(), x1 = next();
            while (x1 == x0) x1 = next();
            h[2 * k] = x0;
            h[2 * k + 1] = x1 >= x0 ? x1 - x0 : x1 + (gl::P - x0);
        }
        int rc = d_entries.alloc(total * 2);
        if (rc == MB_OK && cudaMemcpyAsync(d_entries.p, h, total * 2 * sizeof(uint64_t), cudaMemcpyHostToDevice,
                                           MB_STREAM) != cudaSuccess)
            rc = MB_ERR_CUDA;
        if (rc == MB_OK) {
            {
                MB_KERNEL_ON("table_invert", MB_STREAM);
                table_invert_kernel<<<grid_for(total, 256, 8), 256, 0, MB_STREAM>>>(d_entries.p, total);
            }
            rc = finish_sync();
        }
        cudaFreeHost(h);
        return rc;
    }
    const uint64_t* device_level_ptr(int level) const { return d_entries.p + 2 * level_offsets[level]; }

    int num_vars = 0, log_rate = 0, rounds = 0;
    size_t entries = 0;
    std::vector<size_t> level_offsets, level_sizes;
    DevBuf d_entries;
};

// Merkle hash of commitments made from now on: 0 = Poseidon2, 1 = Monolith. The
// reference fixes this at build time (cargo feature "monolith", default on:
// goldilocks-cuda-rs/src/basefold.rs:11-14); a commitment remembers the hash it
// was built with and its openings use the same one.
inline std::atomic<int> g_merkle_hash{0};

// ---- BasefoldCommitment -----------------------------------------------------------------
class BasefoldCommitment {
public:
    // commit_device (basefold.rs:382-414): interpolate, encode, Merkle tree.
    int commit_device(const uint64_t* d_evals, int nv, int lr) {
        if (nv < 1 || lr < 0 || nv + lr > 32 || !d_evals) return MB_ERR_ARG;
        num_vars = nv; log_rate = lr;
        hash = g_merkle_hash.load();
        size_t n = (size_t)1 << nv, cw_len = (size_t)1 << (nv + lr);
        DevBuf coeffs;
        int rc = coeffs.alloc(n);
        if (rc == MB_OK) rc = d_bh_evals.alloc(n);
        if (rc == MB_OK) rc = d_codeword.alloc(cw_len);
        if (rc == MB_OK) rc = d_tree.alloc(4 * (cw_len - 1));
        if (rc != MB_OK) return rc;
        rc = bf::interpolate_async(d_evals, coeffs.p, d_bh_evals.p, nv, MB_STREAM);
        if (rc == MB_OK) rc = bf::encode_async(coeffs.p, coeffs.p, d_codeword.p, nv, lr, MB_STREAM);
        if (rc == MB_OK)
            rc = hash ? mk::build_tree_periodic<mk::HashMonolith>(d_codeword.p, d_tree.p, cw_len / 2, (size_t)1 << lr, MB_STREAM)
                      : mk::build_tree_periodic<mk::HashPoseidon2>(d_codeword.p, d_tree.p, cw_len / 2, (size_t)1 << lr, MB_STREAM);
        if (rc != MB_OK) return rc;
        MB_CUDA(cudaMemcpyAsync(root, d_tree.p + 4 * (cw_len - 2), 32, cudaMemcpyDeviceToHost, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        return MB_OK;
    }
    uint64_t root[4] = {0, 0, 0, 0};
    int num_vars = 0, log_rate = 0, hash = 0;
    DevBuf d_codeword, d_bh_evals, d_tree;
};

// ---- host hashing of tree tops: host_tree_top.hpp -------------------------------------------
// nodes: the layer of `count` digests (a power of two, at most HOST_TOP) the device left; upper: pinned staging for
// count - 1 digests that stays untouched until the stream has run the upload; d_tree: the tree of num_leaves
// leaves (2 num_leaves - 1 digests, layers back to back). root receives the root.
inline int host_finish_top(int hash, const uint64_t* nodes, size_t count, uint64_t* upper, uint64_t* d_tree, size_t num_leaves,
                           uint64_t* root, cudaStream_t st) {
    host_hash_top(hash, nodes, count, upper, root);
    if (count > 1)
        MB_CUDA(cudaMemcpyAsync(d_tree + 4 * (2 * num_leaves - count), upper, 32 * (count - 1), cudaMemcpyHostToDevice, st));
    return MB_OK;
}

// Pinned staging of the calling thread, grown on demand (contents are not kept across a growth).
inline uint64_t* pinned_arena(size_t words) {
    struct Holder {
        uint64_t* p = nullptr;
        size_t cap = 0;
        ~Holder() { if (p) cudaFreeHost(p); }
    };
    static thread_local Holder h;
    if (h.cap < words) {
        if (h.p) cudaFreeHost(h.p);
        h.p = nullptr;
        h.cap = 0;
        if (cudaMallocHost(&h.p, words * sizeof(uint64_t)) != cudaSuccess) { h.p = nullptr; return nullptr; }
        h.cap = words;
    }
    return h.p;
}

inline size_t query_words(int nv, int lr) {
    size_t w = 1 + (size_t)nv * 4 + 4 * (size_t)(nv + lr - 1);
    for (int i = 0; i <= nv - 2; i++) w += 4 * (size_t)(nv + lr - 2 - i);
    return w;
}
inline size_t proof_words(int nv, int lr, int nq) {
    return 2 + (size_t)nv * 6 + (size_t)(nv - 1) * 4 + ((size_t)2 << lr) + (size_t)nq * query_words(nv, lr);
}

}  // namespace mbhost
