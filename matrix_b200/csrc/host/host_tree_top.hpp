// Host hashing of the top of a Merkle tree (Poseidon2 or Monolith over Goldilocks, as the device trees).
//
// The last levels of a tree are bound by the latency of one permutation per level on the device (about 10 us with
// the 8-lane Poseidon2, a whole single-thread permutation with Monolith); a host core runs a permutation in about
// 1 us. So a round's tree stops on the device at a layer of HOST_TOP digests (mk::build_tree's `stop`), which the
// kernel leaves in pinned memory, and the host hashes the three levels above: seven permutations, then one small
// upload puts them into the device tree for the query phase (host_finish_top, gl_basefold_common.cuh).
#pragma once
#include <cstdint>
#include <cstring>
#include "gl_monolith_host.hpp"
#include "gl_poseidon2_host.hpp"

namespace mbhost {

struct Digest {
    uint64_t w[4];
};
// compress(l, r): the first four words of the permutation of (l, r, 0 ...), canonical. hash: 0 Poseidon2, 1 Monolith.
inline Digest host_compress(int hash, const uint64_t* l, const uint64_t* r) {
    uint64_t s[12] = {l[0], l[1], l[2], l[3], r[0], r[1], r[2], r[3], 0, 0, 0, 0};
    if (hash) monohost::permute(s);
    else p2host::permute(s);
    Digest d;
    for (int i = 0; i < 4; i++) d.w[i] = s[i];   // both host forms return canonical words
    return d;
}
inline Digest host_compress(int hash, const Digest& l, const Digest& r) { return host_compress(hash, l.w, r.w); }

constexpr size_t HOST_TOP = 8;

// nodes: a layer of `count` digests (a power of two). upper receives the count - 1 digests of the layers above it,
// layer by layer as the tree stores them (count / 2, count / 4, ..., 1); root receives the last one.
inline void host_hash_top(int hash, const uint64_t* nodes, size_t count, uint64_t* upper, uint64_t* root) {
    const uint64_t* cur = nodes;
    uint64_t* out = upper;
    for (size_t size = count; size > 1; size /= 2) {
        for (size_t j = 0; j < size / 2; j++) {
            const Digest d = host_compress(hash, cur + 8 * j, cur + 8 * j + 4);
            std::memcpy(out + 4 * j, d.w, 32);
        }
        cur = out;
        out += 4 * (size / 2);
    }
    std::memcpy(root, cur, 32);
}

}  // namespace mbhost
