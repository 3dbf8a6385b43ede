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

// ---- the circulant MDS layer of Monolith, width 12 --------------------------------------
// The MDS layer of both Monolith instances (Goldilocks and almost-Goldilocks, width 12) is the circulant with first row C = 7 23 8 26 13 10 9 7 6 22 21 8: out_i = sum_j C[(j - i) mod 12] s_j,
// a cyclic convolution of s with c'_k = C[-k mod 12]. On 32-bit halves of the state words the sums are exact
// integers below 161 * 2^32, and the convolution splits by x^12 - 1 = (x^6 - 1)(x^6 + 1) and x^6 - 1 =
// (x^3 - 1)(x^3 + 1): sums and differences of the halves, a cyclic and a negacyclic product of length 3 (9 + 9
// multiply-adds), a negacyclic product of length 6 (36) and two exact halvings, 54 multiply-adds by small
// constants instead of 144.
namespace mds {
constexpr int C[12] = {7, 23, 8, 26, 13, 10, 9, 7, 6, 22, 21, 8};
constexpr int cp(int k) { return C[(12 - k) % 12]; }     // out = cp (*) s, cyclic of length 12
constexpr int cpq(int k) { return cp(k) + cp(k + 6); }         // mod x^6 - 1
constexpr int cmq(int k) { return cp(k) - cp(k + 6); }         // mod x^6 + 1
constexpr int cpp(int k) { return cpq(k) + cpq(k + 3); }       // mod x^3 - 1
constexpr int cpm(int k) { return cpq(k) - cpq(k + 3); }       // mod x^3 + 1
}  // namespace mds

// out_i = sum_j C[(j - i) mod 12] x_j for twelve values below 2^32, as exact integers.
inline void circulant12(const int64_t* x, int64_t* out) {
    using namespace mds;
    int64_t sp[6], sm[6], spp[3], spm[3];
    for (int k = 0; k < 6; k++) { sp[k] = x[k] + x[k + 6]; sm[k] = x[k] - x[k + 6]; }
    for (int k = 0; k < 3; k++) { spp[k] = sp[k] + sp[k + 3]; spm[k] = sp[k] - sp[k + 3]; }
    const int64_t opp0 = cpp(0) * spp[0] + cpp(2) * spp[1] + cpp(1) * spp[2];
    const int64_t opp1 = cpp(1) * spp[0] + cpp(0) * spp[1] + cpp(2) * spp[2];
    const int64_t opp2 = cpp(2) * spp[0] + cpp(1) * spp[1] + cpp(0) * spp[2];
    const int64_t opm0 = cpm(0) * spm[0] - cpm(2) * spm[1] - cpm(1) * spm[2];
    const int64_t opm1 = cpm(1) * spm[0] + cpm(0) * spm[1] - cpm(2) * spm[2];
    const int64_t opm2 = cpm(2) * spm[0] + cpm(1) * spm[1] + cpm(0) * spm[2];
    const int64_t op[6] = {(opp0 + opm0) >> 1, (opp1 + opm1) >> 1, (opp2 + opm2) >> 1,
                           (opp0 - opm0) >> 1, (opp1 - opm1) >> 1, (opp2 - opm2) >> 1};
    int64_t om[6];
    om[0] = cmq(0) * sm[0] - cmq(5) * sm[1] - cmq(4) * sm[2] - cmq(3) * sm[3] - cmq(2) * sm[4] - cmq(1) * sm[5];
    om[1] = cmq(1) * sm[0] + cmq(0) * sm[1] - cmq(5) * sm[2] - cmq(4) * sm[3] - cmq(3) * sm[4] - cmq(2) * sm[5];
    om[2] = cmq(2) * sm[0] + cmq(1) * sm[1] + cmq(0) * sm[2] - cmq(5) * sm[3] - cmq(4) * sm[4] - cmq(3) * sm[5];
    om[3] = cmq(3) * sm[0] + cmq(2) * sm[1] + cmq(1) * sm[2] + cmq(0) * sm[3] - cmq(5) * sm[4] - cmq(4) * sm[5];
    om[4] = cmq(4) * sm[0] + cmq(3) * sm[1] + cmq(2) * sm[2] + cmq(1) * sm[3] + cmq(0) * sm[4] - cmq(5) * sm[5];
    om[5] = cmq(5) * sm[0] + cmq(4) * sm[1] + cmq(3) * sm[2] + cmq(2) * sm[3] + cmq(1) * sm[4] + cmq(0) * sm[5];
    for (int k = 0; k < 6; k++) { out[k] = (op[k] + om[k]) >> 1; out[k + 6] = (op[k] - om[k]) >> 1; }
}

}  // namespace hf
}  // namespace mbhost
