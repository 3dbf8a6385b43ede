// Field arithmetic for host code on a round loop's critical path (transcript permutations, tree tops, the last
// rounds of a sumcheck): Goldilocks p = 2^64 - 2^32 + 1 and almost-Goldilocks q = 2^64 - 2^32 - 31 through the host
// core's 64 x 64 -> 128 multiplier, with no data-dependent branches (the carries are coin flips). The device forms
// in gl_field.cuh / agl_field.cuh count 32-bit instructions instead and run three to four times slower here.
// Same residues as those forms; the tests compare the two on canonical, loose and extreme words.
#pragma once
#include <cstdint>

namespace mbhost {
namespace hf {

typedef unsigned __int128 u128;

// ---- Goldilocks --------------------------------------------------------------------
constexpr uint64_t GL_P = 0xFFFFFFFF00000001ULL;
constexpr uint64_t GL_EPS = 0xFFFFFFFFULL;   // 2^64 mod p

// x mod p as a loose 64-bit residue, for any 128-bit x: with 2^64 = 2^32 - 1 and 2^96 = -1 (mod p),
// x = lo - hi_hi + hi_lo (2^32 - 1). A borrow is repaired by - EPS (the wrapped value is above 2^64 - 2^32), a
// carry by + EPS (the wrapped value is below hi_lo EPS < 2^64 - 2^33).
static inline uint64_t gl_red(u128 x) {
    const uint64_t lo = (uint64_t)x, hi = (uint64_t)(x >> 64);
    const uint64_t hh = hi >> 32, hl = hi & GL_EPS, t1 = (hl << 32) - hl;
    uint64_t t0 = lo - hh;
    t0 -= (0 - (uint64_t)(lo < hh)) & GL_EPS;
    uint64_t r = t0 + t1;
    r += (0 - (uint64_t)(r < t1)) & GL_EPS;
    return r;
}
static inline uint64_t gl_canon(uint64_t x) { return x >= GL_P ? x - GL_P : x; }
// canonical in, canonical out
static inline uint64_t gl_add(uint64_t a, uint64_t b) {
    const uint64_t s = a + b, w = s - GL_P;
    return ((s < a) | (s >= GL_P)) ? w : s;
}
static inline uint64_t gl_sub(uint64_t a, uint64_t b) {
    const uint64_t d = a - b;
    return a < b ? d + GL_P : d;
}
static inline uint64_t gl_mul(uint64_t a, uint64_t b) { return gl_canon(gl_red((u128)a * b)); }

// ---- almost-Goldilocks ---------------------------------------------------------------
constexpr uint64_t AGL_P = 0xFFFFFFFEFFFFFFE1ULL;
constexpr uint64_t AGL_C = 0x000000010000001FULL;   // 2^64 mod q

// lo + hi c for a high word below 2^31, loose result: one carry repair (the wrapped sum is below hi c).
static inline uint64_t agl_red_small(u128 x) {
    const uint64_t lo = (uint64_t)x, t = (uint64_t)(x >> 64) * AGL_C;
    uint64_t r = lo + t;
    r += (0 - (uint64_t)(r < t)) & AGL_C;
    return r;
}
// Any 128-bit value: two folds of the high word (2^64 = c) bring it below 2^34 and then below 8.
static inline uint64_t agl_red(u128 x) {
    x = (u128)(uint64_t)(x >> 64) * AGL_C + (uint64_t)x;
    x = (u128)(uint64_t)(x >> 64) * AGL_C + (uint64_t)x;
    return agl_red_small(x);
}
static inline uint64_t agl_canon(uint64_t x) { return x >= AGL_P ? x - AGL_P : x; }
static inline uint64_t agl_add(uint64_t a, uint64_t b) {
    const uint64_t s = a + b, w = s - AGL_P;
    return ((s < a) | (s >= AGL_P)) ? w : s;
}
static inline uint64_t agl_sub(uint64_t a, uint64_t b) {
    const uint64_t d = a - b;
    return a < b ? d + AGL_P : d;
}

// ---- quadratic extensions, canonical words in and out ----------------------------------
// (a0 + a1 X)(b0 + b1 X) with X^2 = W: products of canonical words stay below 2^128 - 2^97, so a reduced word
// (times W) can be added to a product without overflow.
struct GlE2Ops {
    static constexpr uint64_t W = 7;
    static uint64_t add(uint64_t a, uint64_t b) { return gl_add(a, b); }
    static uint64_t sub(uint64_t a, uint64_t b) { return gl_sub(a, b); }
    static uint64_t red(u128 x) { return gl_red(x); }
    static uint64_t canon(uint64_t x) { return gl_canon(x); }
};
struct AglE2Ops {
    static constexpr uint64_t W = 3;
    static uint64_t add(uint64_t a, uint64_t b) { return agl_add(a, b); }
    static uint64_t sub(uint64_t a, uint64_t b) { return agl_sub(a, b); }
    static uint64_t red(u128 x) { return agl_red(x); }
    static uint64_t canon(uint64_t x) { return agl_canon(x); }
};
template <class F>
static inline void e2_mul(uint64_t a0, uint64_t a1, uint64_t b0, uint64_t b1, uint64_t& c0, uint64_t& c1) {
    const uint64_t t11 = F::red((u128)a1 * b1), t10 = F::red((u128)a1 * b0);
    c0 = F::canon(F::red((u128)a0 * b0 + (u128)t11 * F::W));
    c1 = F::canon(F::red((u128)a0 * b1 + t10));
}

}  // namespace hf
}  // namespace mbhost
