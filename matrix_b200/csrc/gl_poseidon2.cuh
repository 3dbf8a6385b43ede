// Poseidon2 permutation, width 8 over Goldilocks (4 + 22 + 4 rounds, x^7),
// plus the leaf / node hash forms used by the Merkle trees.
//
// Same function as the reference's poseidon2_permute_8 (cuda/poseidon2.cuh:322-358,
// CPU twin goldilocks-cuda-rs/src/cpu_poseidon2.rs:120-141) with the same round
// constants (cuda/poseidon2.cuh:50-94). State words are loose residues in
// [0, 2^64); callers canonicalise what they write out.
#pragma once
#include "gl_field.cuh"

namespace gl {

#define GLP2_RC_EXT_INIT                                                                              \
    {                                                                                                 \
        {0xdd5743e7f2a5a5d9ULL, 0xcb3a864e58ada44bULL, 0xd5a3726889dedc0dULL, 0x79365a7f967583c1ULL,  \
         0xb7820c177b0a3c30ULL, 0x68a60479943b7240ULL, 0x0a22eeab67b97c41ULL, 0xbee9d90e037fa7d4ULL}, \
        {0xf1dda5b9259dfcb4ULL, 0x27515210be112d59ULL, 0x654a4db8f15f6c3aULL, 0x5a9bfff8c29db0c4ULL,  \
         0xb72f2628c95a885bULL, 0xffcb54fc166beaddULL, 0xe32f91d59c463772ULL, 0x9e0ff2a9bbea79dbULL}, \
        {0xce57d6245ddca6b2ULL, 0xb1fc8d402bba1eb1ULL, 0x64df974fb666d528ULL, 0x59e4e5b237e52e78ULL,  \
         0x5e255e2742caa8fcULL, 0xc4a17304e330ef9aULL, 0x60e3a513cdd9f0b1ULL, 0xbf29a6a5a0c9c8baULL}, \
        {0xcea721cce82fb11bULL, 0xe5b55eb8098ece81ULL, 0x4ec66bfb89f7c380ULL, 0xc33be12b6ef7e4faULL,  \
         0xa41b5f5b84c57d7dULL, 0xb526206b2138a936ULL, 0x9f7a5ac62f16eb4eULL, 0x7de77f405f683aa5ULL}, \
        {0x014ef1197d341346ULL, 0x9725e20825d07394ULL, 0xc8ff2a22516f3604ULL, 0xde1b51f7cf493493ULL,  \
         0xa7e3af1a53eadb78ULL, 0x9b7b7ee0ddf9f229ULL, 0xf0a460f2dc649e7dULL, 0xdc4448d02c2cb823ULL}, \
        {0xaa62c88e0b294011ULL, 0x058eb9d810ce9f74ULL, 0x4e3d7a5403566d24ULL, 0xe8ae66da2f8b7a63ULL,  \
         0x3fdad3b08dae2e0bULL, 0xec81e61303dd409bULL, 0x3cbaa1cd35d31fc4ULL, 0x847f7806eec88ffaULL}, \
        {0x98ae09a325893803ULL, 0xf8a6475077968838ULL, 0xdf55b7419443de5bULL, 0xdbe15699e696ca70ULL,  \
         0x8e54a27d8db00424ULL, 0x7679a45cd9d1e12aULL, 0x2844f52be73e0e2fULL, 0xd41f8eb31ada34f8ULL}, \
        {0xe9dd318bae1f3961ULL, 0xf7462137299efe1aULL, 0x6dbbe06779e1d573ULL, 0xfe35b05cbe707632ULL,  \
         0x5d8896b12654fd8cULL, 0x6f96ef47c32d4ae2ULL, 0xb0caa221dbbfc0daULL, 0x0bc2a5bf1f238d3fULL}, \
    }
#define GLP2_RC_INT_INIT                                                                             \
    {                                                                                                \
        0x488897d85ff51f56ULL, 0x1140737ccb162218ULL, 0xa7eeb9215866ed35ULL, 0x9bd2976fee49fcc9ULL,  \
        0xc0c8f0de580a3fccULL, 0x4fb2dae6ee8fc793ULL, 0x343a89f35f37395bULL, 0x223b525a77ca72c8ULL,  \
        0x56ccb62574aaa918ULL, 0xc4d507d8027af9edULL, 0xa080673cf0b7e95cULL, 0xf0184884eb70dcf8ULL,  \
        0x044f10b0cb3d5c69ULL, 0xe9e3f7993938f186ULL, 0x1b761c80e772f459ULL, 0x606cec607a1b5facULL,  \
        0x14a0c2e1d45f03cdULL, 0x4eace8855398574fULL, 0xf905ca7103eff3e6ULL, 0xf8c8f8d20862c059ULL,  \
        0xb524fe8bdd678e5aULL, 0xfbb7865901a1ec41ULL,                                                \
    }
#define GLP2_DIAG_INIT                                                                               \
    {                                                                                                \
        0xa98811a1fed4e3a5ULL, 0x1cc48b54f377e2a0ULL, 0xe40cd4f6c5609a26ULL, 0x11de79ebca97a4a3ULL,  \
        0x9177c73d8b7e929cULL, 0x2a6fe8085797e791ULL, 0x3de6e93329f8d5adULL, 0x3f7af9125da962feULL,  \
    }

// All table entries are below p. Statically initialised __constant__ data is
// loaded with the module on every device that runs it; no init call is needed.
static const uint64_t h_p2_rc_ext[8][8] = GLP2_RC_EXT_INIT;
static const uint64_t h_p2_rc_int[22] = GLP2_RC_INT_INIT;
static const uint64_t h_p2_diag[8] = GLP2_DIAG_INIT;
#ifdef __CUDACC__
static __constant__ uint64_t d_p2_rc_ext[8][8] = GLP2_RC_EXT_INIT;
static __constant__ uint64_t d_p2_rc_int[22] = GLP2_RC_INT_INIT;
static __constant__ uint64_t d_p2_diag[8] = GLP2_DIAG_INIT;
#endif

GLF uint64_t p2_rc_ext(int r, int i) {
#ifdef __CUDA_ARCH__
    return d_p2_rc_ext[r][i];
#else
    return h_p2_rc_ext[r][i];
#endif
}
GLF uint64_t p2_rc_int(int r) {
#ifdef __CUDA_ARCH__
    return d_p2_rc_int[r];
#else
    return h_p2_rc_int[r];
#endif
}
GLF uint64_t p2_diag(int i) {
#ifdef __CUDA_ARCH__
    return d_p2_diag[i];
#else
    return h_p2_diag[i];
#endif
}

GLF uint64_t sbox7(uint64_t x) {
    uint64_t x2 = sqr(x), x4 = sqr(x2), x3 = mul(x2, x);
    return mul(x4, x3);
}

// External linear layer: y = M x with M = [[2 M4, M4], [M4, 2 M4]],
// M4 = [2 3 1 1; 1 2 3 1; 1 1 2 3; 3 1 1 2] (the 4x4 map on each half followed
// by the cross-half sums of mds_light_8 in the reference), plus the next
// round's constants. Instead of a chain of modular additions, the low and high
// 32-bit halves of the eight inputs are accumulated separately with their small
// integer weights (row sum 21, so both sums stay below 2^37) and each output is
// reduced once.
template <bool HAS_RC>
GLF void p2_external_linear(uint64_t* s, int next_round) {
    constexpr uint32_t M[8][8] = {{4, 6, 2, 2, 2, 3, 1, 1}, {2, 4, 6, 2, 1, 2, 3, 1}, {2, 2, 4, 6, 1, 1, 2, 3},
                                  {6, 2, 2, 4, 3, 1, 1, 2}, {2, 3, 1, 1, 4, 6, 2, 2}, {1, 2, 3, 1, 2, 4, 6, 2},
                                  {1, 1, 2, 3, 2, 2, 4, 6}, {3, 1, 1, 2, 6, 2, 2, 4}};
    uint64_t y[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint64_t L = 0, H = 0;
        if (HAS_RC) {
            uint64_t rc = p2_rc_ext(next_round, i);
            L = lo32(rc);
            H = hi32(rc);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            L = madwide(lo32(s[j]), M[i][j], L);
            H = madwide(hi32(s[j]), M[i][j], H);
        }
        y[i] = reduce_limb_sums(L, H);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) s[i] = y[i];
}

// Internal linear layer: s_i = d_i s_i + sum(s); `rc0` (the next round's
// constant for lane 0, or 0) rides along in lane 0's sum.
GLF void p2_internal_linear(uint64_t* s, uint64_t rc0) {
    uint64_t SL = 0, SH = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        SL = madwide(lo32(s[i]), 1u, SL);
        SH = madwide(hi32(s[i]), 1u, SH);
    }
    uint64_t sum = reduce_limb_sums(SL, SH);
    s[0] = mul_add(s[0], p2_diag(0), add_c(sum, rc0));
#pragma unroll
    for (int i = 1; i < 8; i++) s[i] = mul_add(s[i], p2_diag(i), sum);
}

// In place; loose in, loose out. Round constants are added by the linear layer
// that precedes the S-boxes using them, so only the first external and the
// first internal / terminal constants need explicit additions.
GLF void poseidon2_permute(uint64_t* s) {
#pragma unroll
    for (int i = 0; i < 8; i++) s[i] = add_c(s[i], p2_rc_ext(0, i));
#pragma unroll 1
    for (int r = 0; r < 4; r++) {
#pragma unroll
        for (int i = 0; i < 8; i++) s[i] = sbox7(s[i]);
        if (r < 3) {
            p2_external_linear<true>(s, r + 1);
        } else {
            p2_external_linear<false>(s, 0);
            s[0] = add_c(s[0], p2_rc_int(0));
        }
    }
#pragma unroll 1
    for (int r = 0; r < 22; r++) {
        s[0] = sbox7(s[0]);
        p2_internal_linear(s, r < 21 ? p2_rc_int(r + 1) : 0);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) s[i] = add_c(s[i], p2_rc_ext(4, i));
#pragma unroll 1
    for (int r = 4; r < 8; r++) {
#pragma unroll
        for (int i = 0; i < 8; i++) s[i] = sbox7(s[i]);
        if (r < 7) p2_external_linear<true>(s, r + 1);
        else p2_external_linear<false>(s, 0);
    }
}

#ifdef __CUDACC__
// ---- one permutation spread over 8 lanes ----------------------------------------
// Layers near the top of a Merkle tree (and a transcript) have too few
// permutations to fill the machine; what matters there is the latency of one
// permutation. Eight consecutive lanes of a warp hold one state word each: the
// S-boxes of an external round run in parallel, the linear layers exchange
// halves with warp shuffles, and in the internal rounds lane 0 runs the S-box
// while the sum is formed by a three-step butterfly. Per-lane constants come
// from global copies of the tables (a divergent index into __constant__ memory
// would serialise). All 32 lanes of the warp must call; `lane8` = lane & 7.
static __device__ const uint64_t g_p2_rc_ext[8][8] = GLP2_RC_EXT_INIT;
static __device__ const uint64_t g_p2_diag[8] = GLP2_DIAG_INIT;

__device__ __forceinline__ uint64_t p2_coop_external(uint64_t x, const uint32_t (&w)[8], uint64_t rc) {
    uint64_t L = lo32(rc), H = hi32(rc);
    const uint32_t xl = lo32(x), xh = hi32(x);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        L = madwide(__shfl_sync(0xffffffffu, xl, j, 8), w[j], L);
        H = madwide(__shfl_sync(0xffffffffu, xh, j, 8), w[j], H);
    }
    return reduce_limb_sums(L, H);
}

__device__ __forceinline__ uint64_t poseidon2_permute_coop8(uint64_t x, int lane8) {
    // row lane8 of M = [[2 M4, M4], [M4, 2 M4]]
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int d = ((j & 3) - (lane8 & 3)) & 3;  // M4 is circulant: first row 2 3 1 1
        uint32_t m4 = d == 0 ? 2u : (d == 1 ? 3u : 1u);
        w[j] = ((j >> 2) == (lane8 >> 2)) ? 2u * m4 : m4;
    }
    const uint64_t diag = g_p2_diag[lane8];
    x = add_c(x, g_p2_rc_ext[0][lane8]);
#pragma unroll 1
    for (int r = 0; r < 4; r++) {
        x = sbox7(x);
        x = p2_coop_external(x, w, r < 3 ? g_p2_rc_ext[r + 1][lane8] : (lane8 == 0 ? p2_rc_int(0) : 0));
    }
    // Internal rounds: x_0 <- sbox(x_0), then x_i <- diag_i x_i + sum_j x_j. What matters here is the length of
    // the dependent chain, so everything that does not need the S-box output runs beside it: the products
    // diag_i x_i of the other lanes and the sum of their x_i (a three-step butterfly) are formed from the round's
    // inputs while the S-box chain (three multiplications deep) is in flight; afterwards lane 0's value is
    // broadcast, added to the partial sum, and one 128-bit add and reduction finish every lane. All lanes execute
    // the S-box arithmetic (only lane 0 keeps it), which keeps the warp converged so that the two chains interleave.
    const bool lane0 = lane8 == 0;
#pragma unroll 1
    for (int r = 0; r < 22; r++) {
        const uint64_t t = sbox7(x);
        // beside the S-box: the other lanes' products and their partial sum
        uint64_t ylo = x * diag, yhi = umulhi(x, diag);
        uint64_t UL = lane0 ? 0 : lo32(x), UH = lane0 ? 0 : hi32(x);
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) {
            UL += __shfl_xor_sync(0xffffffffu, UL, off, 8);
            UH += __shfl_xor_sync(0xffffffffu, UH, off, 8);
        }
        // after the S-box: its output to every lane, the full sum, lane 0's own product
        const uint32_t tl = __shfl_sync(0xffffffffu, lo32(t), 0, 8), th = __shfl_sync(0xffffffffu, hi32(t), 0, 8);
        // lane 0's own product needs the S-box output; formed on every lane (no branch) beside the sum
        const uint64_t zlo = t * diag, zhi = umulhi(t, diag);
        uint64_t sum = reduce_limb_sums(UL + tl, UH + th);
        sum = add_c(sum, (lane0 && r < 21) ? p2_rc_int(r + 1) : 0);
        ylo = lane0 ? zlo : ylo;
        yhi = lane0 ? zhi : yhi;
        uint32_t carry;
        const uint64_t l2 = add_carry(ylo, sum, carry);
        x = reduce128(l2, yhi + carry);
    }
    x = add_c(x, g_p2_rc_ext[4][lane8]);
#pragma unroll 1
    for (int r = 4; r < 8; r++) {
        x = sbox7(x);
        x = p2_coop_external(x, w, r < 7 ? g_p2_rc_ext[r + 1][lane8] : 0);
    }
    return x;
}
#endif

}  // namespace gl
