// Poseidon2 width 8 over Goldilocks for the host (the permutation of gl_poseidon2.cuh; same function, same tables).
//
// The device form counts 32-bit instructions; a host core has a 64 x 64 -> 128 multiplier, 128-bit adds in two
// instructions and out-of-order issue, so this form multiplies through unsigned __int128, keeps the linear layers
// as 128-bit sums with one reduction per output, and lets the S-box chain of an internal round overlap the other
// lanes' products. A round loop's host side (transcript, tree tops) is a chain of these permutations between two
// kernel launches, so their latency is on every proof's critical path.
#pragma once
#include <cstdint>
#include "../gl_poseidon2.cuh"
#include "host_field.hpp"

namespace mbhost {
namespace p2host {

using hf::u128;
constexpr uint64_t EPS = hf::GL_EPS;
static inline uint64_t red(u128 x) { return hf::gl_red(x); }   // any 128-bit value, loose result
static inline uint64_t mul(uint64_t a, uint64_t b) { return red((u128)a * b); }
static inline uint64_t sbox7(uint64_t x) {
    const uint64_t x2 = mul(x, x), x4 = mul(x2, x2), x3 = mul(x2, x);
    return mul(x4, x3);
}

// y = M4 x for M4 = [2 3 1 1; 1 2 3 1; 1 1 2 3; 3 1 1 2], as 128-bit sums (inputs below 2^64: outputs below 7 2^64).
static inline void mat4(const uint64_t* x, u128* y) {
    const u128 t01 = (u128)x[0] + x[1], t23 = (u128)x[2] + x[3];
    const u128 t0123 = t01 + t23;
    const u128 t01123 = t0123 + x[1], t01233 = t0123 + x[3];
    y[3] = t01233 + ((u128)x[0] << 1);
    y[1] = t01123 + ((u128)x[2] << 1);
    y[0] = t01123 + t01;
    y[2] = t01233 + t23;
}

// s <- [[2 M4, M4], [M4, 2 M4]] s + rc (rc may be null): sums stay below 22 2^64.
static inline void external_linear(uint64_t* s, const uint64_t* rc) {
    u128 a[4], b[4];
    mat4(s, a);
    mat4(s + 4, b);
    for (int i = 0; i < 4; i++) {
        const u128 sum = a[i] + b[i];
        s[i] = red(a[i] + sum + (rc ? rc[i] : 0));
        s[i + 4] = red(b[i] + sum + (rc ? rc[i + 4] : 0));
    }
}

// In place; any 64-bit words in, canonical residues out.
static inline void permute(uint64_t* s) {
    const uint64_t(*rc_ext)[8] = gl::h_p2_rc_ext;
    const uint64_t* rc_int = gl::h_p2_rc_int;
    const uint64_t* diag = gl::h_p2_diag;
    for (int i = 0; i < 8; i++) s[i] = red((u128)s[i] + rc_ext[0][i]);
    for (int r = 0; r < 4; r++) {
        for (int i = 0; i < 8; i++) s[i] = sbox7(s[i]);
        external_linear(s, r < 3 ? rc_ext[r + 1] : nullptr);
    }
    // Internal rounds: s_0 <- sbox(s_0 + rc), then s_i <- d_i s_i + sum_j s_j. The chain that matters is lane 0's:
    // with rest = the other lanes' sum (reduced beside the S-box), the new lane 0 is s0 (d_0 + 1) + rest + the next
    // round's constant in one 128-bit sum ((2^64 - 1) p + 2 (2^64 - 1) < 2^128), so a round costs the S-box and one
    // multiply-reduce on the chain.
    s[0] = red((u128)s[0] + rc_int[0]);
    const uint64_t d0p1 = diag[0] + 1;
    for (int r = 0; r < 22; r++) {
        u128 rest128 = 0;
        for (int i = 1; i < 8; i++) rest128 += s[i];
        const uint64_t rest = red(rest128);
        u128 prod[8];
        for (int i = 1; i < 8; i++) prod[i] = (u128)s[i] * diag[i] + rest;
        const uint64_t s0 = sbox7(s[0]);
        s[0] = red((u128)s0 * d0p1 + rest + (r < 21 ? rc_int[r + 1] : 0));
        for (int i = 1; i < 8; i++) s[i] = red(prod[i] + s0);
    }
    for (int i = 0; i < 8; i++) s[i] = red((u128)s[i] + rc_ext[4][i]);
    for (int r = 4; r < 8; r++) {
        for (int i = 0; i < 8; i++) s[i] = sbox7(s[i]);
        external_linear(s, r < 7 ? rc_ext[r + 1] : nullptr);
    }
    for (int i = 0; i < 8; i++) s[i] = s[i] >= gl::P ? s[i] - gl::P : s[i];
}

}  // namespace p2host
}  // namespace mbhost
