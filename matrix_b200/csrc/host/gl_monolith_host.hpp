// Monolith-64 over Goldilocks for the host (the permutation of gl_monolith.cuh; same function, same constants):
// the tops of Merkle trees are hashed by a host core between two kernel launches of a round, so the permutation is
// written for one (128-bit products, branch-free reductions, the MDS layer as a split cyclic convolution on 32-bit
// halves) rather than shared with the device's 32-bit limb forms.
#pragma once
#include <cstdint>
#include "../gl_monolith.cuh"
#include "host_field.hpp"

namespace mbhost {
namespace monohost {

using hf::u128;

// s <- MDS s + rc (rc may be null), loose words out: L + 2^32 H + rc is below 162 * 2^64.
static inline void concrete(uint64_t* s, const uint64_t* rc) {
    int64_t lo[12], hi[12], L[12], H[12];
    for (int j = 0; j < 12; j++) { lo[j] = (int64_t)(s[j] & 0xFFFFFFFFULL); hi[j] = (int64_t)(s[j] >> 32); }
    hf::circulant12(lo, L);
    hf::circulant12(hi, H);
    for (int i = 0; i < 12; i++) s[i] = hf::gl_red(((u128)(uint64_t)H[i] << 32) + (uint64_t)L[i] + (rc ? rc[i] : 0));
}

// In place; any 64-bit words in, canonical residues out.
static inline void permute(uint64_t* s) {
    concrete(s, nullptr);
    for (int r = 1; r <= gl::MONO_ROUNDS; r++) {
        for (int i = 0; i < 4; i++) s[i] = gl::mono_bar(hf::gl_canon(s[i]));   // bars act on the canonical word
        // bricks: s_i += s_{i-1}^2 on the values before the layer ((2^64 - 1)^2 + 2^64 - 1 < 2^128)
        uint64_t t[12];
        for (int i = 1; i < 12; i++) t[i] = hf::gl_red((u128)s[i - 1] * s[i - 1] + s[i]);
        for (int i = 1; i < 12; i++) s[i] = t[i];
        concrete(s, r < gl::MONO_ROUNDS ? gl::h_mono_rc[r] : nullptr);
    }
    for (int i = 0; i < 12; i++) s[i] = hf::gl_canon(s[i]);
}

}  // namespace monohost
}  // namespace mbhost
