/*
 * CPU oracle (test infrastructure, not the product): Goldilocks helpers,
 * Poseidon2 width 8, the duplex transcript and the Merkle hash functions.
 * See gl.h for the reference lines each part follows.
 */
#include "gl.h"
#include <string.h>

uint64_t gl_pow(uint64_t a, uint64_t e) {
    uint64_t r = 1;
    while (e) {
        if (e & 1) r = gl_mul(r, a);
        a = gl_mul(a, a);
        e >>= 1;
    }
    return r;
}

/* Fermat inverse a^(p-2); gl_inv(0) = 0 like any power of zero. */
uint64_t gl_inv(uint64_t a) { return gl_pow(a, GL_P - 2); }

/* 1/(c0 + c1 X) = (c0 - c1 X) / (c0^2 - 7 c1^2) */
ext2_t e2_inv(ext2_t a) {
    uint64_t n = gl_sub(gl_mul(a.c0, a.c0), gl_mul(7, gl_mul(a.c1, a.c1)));
    uint64_t ni = gl_inv(n);
    return e2(gl_mul(a.c0, ni), gl_mul(gl_neg(a.c1), ni));
}

/* Constants: goldilocks-cuda-rs/src/cpu_poseidon2.rs:16-52 (identical tables in
 * cuda/poseidon2.cuh:50-94 and zk-torch-3/src/transcript.rs:14-56). */
static const uint64_t RC_EXT[8][8] = {
    {0xdd5743e7f2a5a5d9ULL, 0xcb3a864e58ada44bULL, 0xd5a3726889dedc0dULL, 0x79365a7f967583c1ULL,
     0xb7820c177b0a3c30ULL, 0x68a60479943b7240ULL, 0x0a22eeab67b97c41ULL, 0xbee9d90e037fa7d4ULL},
    {0xf1dda5b9259dfcb4ULL, 0x27515210be112d59ULL, 0x654a4db8f15f6c3aULL, 0x5a9bfff8c29db0c4ULL,
     0xb72f2628c95a885bULL, 0xffcb54fc166beaddULL, 0xe32f91d59c463772ULL, 0x9e0ff2a9bbea79dbULL},
    {0xce57d6245ddca6b2ULL, 0xb1fc8d402bba1eb1ULL, 0x64df974fb666d528ULL, 0x59e4e5b237e52e78ULL,
     0x5e255e2742caa8fcULL, 0xc4a17304e330ef9aULL, 0x60e3a513cdd9f0b1ULL, 0xbf29a6a5a0c9c8baULL},
    {0xcea721cce82fb11bULL, 0xe5b55eb8098ece81ULL, 0x4ec66bfb89f7c380ULL, 0xc33be12b6ef7e4faULL,
     0xa41b5f5b84c57d7dULL, 0xb526206b2138a936ULL, 0x9f7a5ac62f16eb4eULL, 0x7de77f405f683aa5ULL},
    {0x014ef1197d341346ULL, 0x9725e20825d07394ULL, 0xc8ff2a22516f3604ULL, 0xde1b51f7cf493493ULL,
     0xa7e3af1a53eadb78ULL, 0x9b7b7ee0ddf9f229ULL, 0xf0a460f2dc649e7dULL, 0xdc4448d02c2cb823ULL},
    {0xaa62c88e0b294011ULL, 0x058eb9d810ce9f74ULL, 0x4e3d7a5403566d24ULL, 0xe8ae66da2f8b7a63ULL,
     0x3fdad3b08dae2e0bULL, 0xec81e61303dd409bULL, 0x3cbaa1cd35d31fc4ULL, 0x847f7806eec88ffaULL},
    {0x98ae09a325893803ULL, 0xf8a6475077968838ULL, 0xdf55b7419443de5bULL, 0xdbe15699e696ca70ULL,
     0x8e54a27d8db00424ULL, 0x7679a45cd9d1e12aULL, 0x2844f52be73e0e2fULL, 0xd41f8eb31ada34f8ULL},
    {0xe9dd318bae1f3961ULL, 0xf7462137299efe1aULL, 0x6dbbe06779e1d573ULL, 0xfe35b05cbe707632ULL,
     0x5d8896b12654fd8cULL, 0x6f96ef47c32d4ae2ULL, 0xb0caa221dbbfc0daULL, 0x0bc2a5bf1f238d3fULL},
};
static const uint64_t RC_INT[22] = {
    0x488897d85ff51f56ULL, 0x1140737ccb162218ULL, 0xa7eeb9215866ed35ULL,
    0x9bd2976fee49fcc9ULL, 0xc0c8f0de580a3fccULL, 0x4fb2dae6ee8fc793ULL,
    0x343a89f35f37395bULL, 0x223b525a77ca72c8ULL, 0x56ccb62574aaa918ULL,
    0xc4d507d8027af9edULL, 0xa080673cf0b7e95cULL, 0xf0184884eb70dcf8ULL,
    0x044f10b0cb3d5c69ULL, 0xe9e3f7993938f186ULL, 0x1b761c80e772f459ULL,
    0x606cec607a1b5facULL, 0x14a0c2e1d45f03cdULL, 0x4eace8855398574fULL,
    0xf905ca7103eff3e6ULL, 0xf8c8f8d20862c059ULL, 0xb524fe8bdd678e5aULL,
    0xfbb7865901a1ec41ULL,
};
static const uint64_t DIAG_8[8] = {
    0xa98811a1fed4e3a5ULL, 0x1cc48b54f377e2a0ULL, 0xe40cd4f6c5609a26ULL,
    0x11de79ebca97a4a3ULL, 0x9177c73d8b7e929cULL, 0x2a6fe8085797e791ULL,
    0x3de6e93329f8d5adULL, 0x3f7af9125da962feULL,
};

/* cpu_poseidon2.rs:64-69 */
static inline uint64_t sbox7(uint64_t x) {
    uint64_t x2 = gl_mul(x, x), x4 = gl_mul(x2, x2), x3 = gl_mul(x2, x);
    return gl_mul(x4, x3);
}

/* cpu_poseidon2.rs:72-86 */
static inline void mds4(uint64_t *s) {
    uint64_t t01 = gl_add(s[0], s[1]), t23 = gl_add(s[2], s[3]);
    uint64_t t0123 = gl_add(t01, t23);
    uint64_t t01123 = gl_add(t0123, s[1]), t01233 = gl_add(t0123, s[3]);
    uint64_t n0 = gl_add(t01123, t01);
    uint64_t n1 = gl_add(t01123, gl_add(s[2], s[2]));
    uint64_t n2 = gl_add(t01233, t23);
    uint64_t n3 = gl_add(t01233, gl_add(s[0], s[0]));
    s[0] = n0; s[1] = n1; s[2] = n2; s[3] = n3;
}

/* cpu_poseidon2.rs:89-105 */
static inline void mds_light_8(uint64_t *s) {
    mds4(s);
    mds4(s + 4);
    for (int i = 0; i < 4; i++) {
        uint64_t sum = gl_add(s[i], s[i + 4]);
        s[i] = gl_add(s[i], sum);
        s[i + 4] = gl_add(s[i + 4], sum);
    }
}

/* cpu_poseidon2.rs:108-117 */
static inline void diffusion_8(uint64_t *s) {
    uint64_t sum = s[0];
    for (int i = 1; i < 8; i++) sum = gl_add(sum, s[i]);
    for (int i = 0; i < 8; i++) s[i] = gl_add(gl_mul(s[i], gl_canon(DIAG_8[i])), sum);
}

/* cpu_poseidon2.rs:120-141. The tabulated constants are used as field
 * elements; those at or above p are reduced first (same residue). */
void gl_poseidon2_permute(uint64_t s[8]) {
    for (int r = 0; r < 4; r++) {
        for (int i = 0; i < 8; i++) s[i] = sbox7(gl_add(s[i], gl_canon(RC_EXT[r][i])));
        mds_light_8(s);
    }
    for (int r = 0; r < 22; r++) {
        s[0] = sbox7(gl_add(s[0], gl_canon(RC_INT[r])));
        diffusion_8(s);
    }
    for (int r = 0; r < 4; r++) {
        for (int i = 0; i < 8; i++) s[i] = sbox7(gl_add(s[i], gl_canon(RC_EXT[4 + r][i])));
        mds_light_8(s);
    }
}

/* ------------------------------------------------------------------ */
/* Transcript: zk-torch-3/src/transcript.rs:183-317                    */
/* ------------------------------------------------------------------ */

static void duplexing(gl_transcript_t *t) {
    for (int i = 0; i < t->in_count; i++) t->sponge[i] = t->in_buf[i];
    for (int i = t->in_count; i < 4; i++) t->sponge[i] = 0;
    t->in_count = 0;
    gl_poseidon2_permute(t->sponge);
    t->permutations++;
    for (int i = 0; i < 4; i++) t->out_buf[3 - i] = t->sponge[i];
    t->out_count = 4;
}

void gl_transcript_absorb(gl_transcript_t *t, uint64_t v) {
    t->out_count = 0;
    t->in_buf[t->in_count++] = v;
    if (t->in_count == 4) duplexing(t);
}

uint64_t gl_transcript_squeeze(gl_transcript_t *t) {
    if (t->out_count == 0) duplexing(t);
    t->out_count--;
    return t->out_buf[t->out_count];
}

void gl_transcript_new(gl_transcript_t *t, const uint8_t *label, size_t n) {
    memset(t, 0, sizeof(*t));
    for (size_t i = 0; i < n; i++) gl_transcript_absorb(t, label[i]);
}

/* transcript.rs:201-209: length, then bytes; empty labels are skipped. */
static void absorb_label(gl_transcript_t *t, const char *label) {
    size_t n = label ? strlen(label) : 0;
    if (n == 0) return;
    gl_transcript_absorb(t, (uint64_t)n);
    for (size_t i = 0; i < n; i++) gl_transcript_absorb(t, (uint8_t)label[i]);
}

void gl_transcript_append_u64(gl_transcript_t *t, const char *label, uint64_t v) {
    absorb_label(t, label);
    gl_transcript_absorb(t, v);
}
void gl_transcript_append_scalar(gl_transcript_t *t, const char *label, uint64_t v) {
    absorb_label(t, label);
    gl_transcript_absorb(t, v);
}
void gl_transcript_append_ext2(gl_transcript_t *t, const char *label, ext2_t v) {
    absorb_label(t, label);
    gl_transcript_absorb(t, v.c0);
    gl_transcript_absorb(t, v.c1);
}
uint64_t gl_transcript_challenge_scalar(gl_transcript_t *t, const char *label) {
    absorb_label(t, label);
    return gl_transcript_squeeze(t);
}
ext2_t gl_transcript_challenge_ext2(gl_transcript_t *t, const char *label) {
    absorb_label(t, label);
    uint64_t c0 = gl_transcript_squeeze(t);
    uint64_t c1 = gl_transcript_squeeze(t);
    return e2(c0, c1);
}

/* ------------------------------------------------------------------ */
/* Merkle hashing: cpu_poseidon2.rs:145-183                            */
/* ------------------------------------------------------------------ */

/* The reference chooses the Merkle hash at build time (cargo feature
 * "monolith", goldilocks-cuda-rs/src/merkle.rs:44-47, basefold.rs:11-14); the
 * oracle chooses at run time: 0 = Poseidon2, 1 = Monolith. Set before use, not
 * while another thread hashes. */
static int g_merkle_hash = 0;
void oracle_set_merkle_hash(int h) { g_merkle_hash = h; }
int oracle_get_merkle_hash(void) { return g_merkle_hash; }

void gl_hash_gl_leaf(uint64_t a, uint64_t b, uint64_t out[4]) {
    if (g_merkle_hash) { gl_monolith_hash_gl_leaf(a, b, out); return; }
    uint64_t s[8] = { a, b, 0, 0, 0, 0, 0, 0 };
    gl_poseidon2_permute(s);
    memcpy(out, s, 32);
}
void gl_hash_ext2_leaf(ext2_t a, ext2_t b, uint64_t out[4]) {
    if (g_merkle_hash) { gl_monolith_hash_ext2_leaf(a, b, out); return; }
    uint64_t s[8] = { a.c0, a.c1, b.c0, b.c1, 0, 0, 0, 0 };
    gl_poseidon2_permute(s);
    memcpy(out, s, 32);
}
void gl_compress(const uint64_t l[4], const uint64_t r[4], uint64_t out[4]) {
    if (g_merkle_hash) { gl_monolith_compress(l, r, out); return; }
    uint64_t s[8];
    memcpy(s, l, 32);
    memcpy(s + 4, r, 32);
    gl_poseidon2_permute(s);
    memcpy(out, s, 32);
}

/* flat wrappers for tests */
void oracle_gl_e2_inv(const uint64_t *a, uint64_t *out) { ext2_t r = e2_inv(e2(a[0], a[1])); out[0] = r.c0; out[1] = r.c1; }

/* ---- Degree-5 extension F_p[X]/(X^5 - 3): cuda/extension.cuh:27-28 (W = 3,
 * DTH_ROOT = W^((p-1)/5)), :388-456 (product, wrapped terms times W), :516-530
 * (Frobenius: coefficient i times DTH_ROOT^i), :574-611 (inverse through the four
 * conjugates and the norm), :625-638 (square-and-multiply, low bit first).
 * Elements are five canonical words; inputs are canonicalised first. ---- */
#define E5_DTH 1041288259238279555ULL

static void e5_mul_o(const uint64_t *a, const uint64_t *b, uint64_t *r) {
    uint64_t t[9] = {0};
    for (int i = 0; i < 5; i++)
        for (int j = 0; j < 5; j++) t[i + j] = gl_add(t[i + j], gl_mul(a[i], b[j]));
    for (int k = 0; k < 5; k++) r[k] = k < 4 ? gl_add(t[k], gl_mul(3, t[k + 5])) : t[k];
}
static void e5_frob_o(const uint64_t *a, uint64_t *r) {
    uint64_t d = 1;
    for (int i = 0; i < 5; i++) { r[i] = gl_mul(a[i], d); d = gl_mul(d, E5_DTH); }
}
void oracle_gl_e5_mul(const uint64_t *a, const uint64_t *b, uint64_t *out) {
    uint64_t x[5], y[5];
    for (int i = 0; i < 5; i++) { x[i] = a[i] % GL_P; y[i] = b[i] % GL_P; }
    e5_mul_o(x, y, out);
}
void oracle_gl_e5_frobenius(const uint64_t *a, uint64_t *out) {
    uint64_t x[5];
    for (int i = 0; i < 5; i++) x[i] = a[i] % GL_P;
    e5_frob_o(x, out);
}
void oracle_gl_e5_inv(const uint64_t *a, uint64_t *out) {
    uint64_t x[5], f[5], conj[5], t[5], norm[5];
    for (int i = 0; i < 5; i++) x[i] = a[i] % GL_P;
    e5_frob_o(x, f);                 /* a^p */
    memcpy(conj, f, sizeof conj);
    for (int k = 0; k < 3; k++) {    /* times a^(p^2), a^(p^3), a^(p^4) */
        e5_frob_o(f, t); memcpy(f, t, sizeof f);
        e5_mul_o(conj, f, t); memcpy(conj, t, sizeof conj);
    }
    e5_mul_o(x, conj, norm);         /* in the base field */
    uint64_t ni = gl_inv(norm[0]);
    for (int i = 0; i < 5; i++) out[i] = gl_mul(conj[i], ni);
}
void oracle_gl_e5_pow(const uint64_t *a, uint64_t e, uint64_t *out) {
    uint64_t r[5] = {1, 0, 0, 0, 0}, b[5], t[5];
    for (int i = 0; i < 5; i++) b[i] = a[i] % GL_P;
    while (e) {
        if (e & 1) { e5_mul_o(r, b, t); memcpy(r, t, sizeof r); }
        e5_mul_o(b, b, t); memcpy(b, t, sizeof b);
        e >>= 1;
    }
    memcpy(out, r, sizeof r);
}

/* Thread count of the OpenMP regions of this library (a launcher may have set OMP_NUM_THREADS=1 in the
 * environment; the timed CPU arm wants every host core). */
#include <omp.h>
void oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int oracle_max_threads(void) { return omp_get_max_threads(); }
