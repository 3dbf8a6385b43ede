// Monolith-64 permutation over Goldilocks: width 12, 4 bars, 6 rounds, 8-bit
// lookups (goldilocks-cuda-rs/src/cpu_monolith.rs:18-144, device twin
// cuda/monolith.cuh). Host and device.
//
//   permute = concrete_0 ; for r = 1..6: bars ; bricks ; concrete_r
//   bars     byte S-box on words 0..3 of the canonical state
//   bricks   s_i += s_{i-1}^2 for i = 11 down to 1
//   concrete circulant MDS (first row 7 23 8 26 13 10 9 7 6 22 21 8) + constants
//
// The concrete layer is formed on 32-bit halves: every output is
// sum_j m_j lo(s_j) + 2^32 sum_j m_j hi(s_j) with integer weights (row sum 160,
// so with the constant's halves both sums stay below 161 * 2^32 < 2^40), one
// mad.wide.u32 per term and one reduction per output instead of twelve modular
// multiply-adds. Values are loose in [0, 2^64) between layers; words 0..3 are
// made canonical before the bars (the S-box acts on the canonical bit pattern),
// and the caller canonicalises what it stores.
#pragma once
#include "gl_field.cuh"

namespace gl {

#define GLMONO_RC_INIT                                                                                                  \
    {{0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0},                                                                               \
     {13596126580325903823ULL, 5676126986831820406ULL, 11349149288412960427ULL, 3368797843020733411ULL,                 \
      16240671731749717664ULL, 9273190757374900239ULL, 14446552112110239438ULL, 4033077683985131644ULL,                 \
      4291229347329361293ULL, 13231607645683636062ULL, 1383651072186713277ULL, 8898815177417587567ULL},                 \
     {2383619671172821638ULL, 6065528368924797662ULL, 16737578966352303081ULL, 2661700069680749654ULL,                  \
      7414030722730336790ULL, 18124970299993404776ULL, 9169923000283400738ULL, 15832813151034110977ULL,                 \
      16245117847613094506ULL, 11056181639108379773ULL, 10546400734398052938ULL, 8443860941261719174ULL},               \
     {15799082741422909885ULL, 13421235861052008152ULL, 15448208253823605561ULL, 2540286744040770964ULL,                \
      2895626806801935918ULL, 8644593510196221619ULL, 17722491003064835823ULL, 5166255496419771636ULL,                  \
      1015740739405252346ULL, 4400043467547597488ULL, 5176473243271652644ULL, 4517904634837939508ULL},                  \
     {18341030605319882173ULL, 13366339881666916534ULL, 6291492342503367536ULL, 10004214885638819819ULL,                \
      4748655089269860551ULL, 1520762444865670308ULL, 8393589389936386108ULL, 11025183333304586284ULL,                  \
      5993305003203422738ULL, 458912836931247573ULL, 5947003897778655410ULL, 17184667486285295106ULL},                  \
     {15710528677110011358ULL, 8929476121507374707ULL, 2351989866172789037ULL, 11264145846854799752ULL,                 \
      14924075362538455764ULL, 10107004551857451916ULL, 18325221206052792232ULL, 16751515052585522105ULL,               \
      15305034267720085905ULL, 15639149412312342017ULL, 14624541102106656564ULL, 3542311898554959098ULL},               \
     {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}}

constexpr int MONO_W = 12;
constexpr int MONO_ROUNDS = 6;

#ifdef __CUDACC__
static __constant__ uint64_t c_mono_rc[MONO_ROUNDS + 1][MONO_W] = GLMONO_RC_INIT;
#endif
static const uint64_t h_mono_rc[MONO_ROUNDS + 1][MONO_W] = GLMONO_RC_INIT;

GLF uint64_t mono_rc(int round, int i) {
#ifdef __CUDA_ARCH__
    return c_mono_rc[round][i];
#else
    return h_mono_rc[round][i];
#endif
}

// The byte S-box on four bytes at once: y = rotl8(x ^ (rotl8(~x,1) & rotl8(x,2) & rotl8(x,3)), 1).
GLF uint32_t mono_bar32(uint32_t x) {
    uint32_t nx = ~x;
    uint32_t l1 = ((nx & 0x80808080u) >> 7) | ((nx & 0x7F7F7F7Fu) << 1);
    uint32_t l2 = ((x & 0xC0C0C0C0u) >> 6) | ((x & 0x3F3F3F3Fu) << 2);
    uint32_t l3 = ((x & 0xE0E0E0E0u) >> 5) | ((x & 0x1F1F1F1Fu) << 3);
    uint32_t t = x ^ (l1 & l2 & l3);
    return ((t & 0x80808080u) >> 7) | ((t & 0x7F7F7F7Fu) << 1);
}
GLF uint64_t mono_bar(uint64_t x) { return pack64(mono_bar32(lo32(x)), mono_bar32(hi32(x))); }

// MDS times state plus the constants of `round` (`HAS_RC` false: zero constants).
template <bool HAS_RC>
GLF void mono_concrete(uint64_t* s, int round) {
    constexpr uint32_t C[MONO_W] = {7, 23, 8, 26, 13, 10, 9, 7, 6, 22, 21, 8};
    uint32_t lo[MONO_W], hi[MONO_W];
#pragma unroll
    for (int j = 0; j < MONO_W; j++) {
        lo[j] = lo32(s[j]);
        hi[j] = hi32(s[j]);
    }
#pragma unroll
    for (int i = 0; i < MONO_W; i++) {
        uint64_t L = 0, H = 0;
        if (HAS_RC) {
            uint64_t rc = mono_rc(round, i);
            L = lo32(rc);
            H = hi32(rc);
        }
#pragma unroll
        for (int j = 0; j < MONO_W; j++) {
            const uint32_t m = C[(j - i + MONO_W) % MONO_W];
            L = madwide(lo[j], m, L);
            H = madwide(hi[j], m, H);
        }
        s[i] = reduce_limb_sums(L, H);
    }
}

// In place; loose in, loose out.
GLF void monolith_permute(uint64_t* s) {
    mono_concrete<false>(s, 0);
#ifdef __CUDA_ARCH__
#pragma unroll 1
#endif
    for (int r = 1; r <= MONO_ROUNDS; r++) {
#pragma unroll
        for (int i = 0; i < 4; i++) s[i] = mono_bar(canon(s[i]));
#pragma unroll
        for (int i = MONO_W - 1; i >= 1; i--) s[i] = mul_add(s[i - 1], s[i - 1], s[i]);
        if (r < MONO_ROUNDS) mono_concrete<true>(s, r);
        else mono_concrete<false>(s, r);
    }
}

}  // namespace gl
