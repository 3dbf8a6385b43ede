/*
 * CPU oracle (test infrastructure, not the product): the Monolith permutation
 * (width 12, 4 bars, 6 rounds, 8-bit lookups) over Goldilocks and over
 * almost-Goldilocks, the Merkle hash functions built on the Goldilocks one and
 * the almost-Goldilocks duplex transcript built on the other.
 *
 *   Goldilocks Monolith   goldilocks-cuda-rs/src/cpu_monolith.rs:18-211
 *   AGL Monolith          zk-torch-4/src/crypto/monolith.rs:66-200
 *   AGL transcript        zk-torch-4/src/transcript.rs:34-260
 *
 * Pinned by the reference's known-answer tests: cpu_monolith.rs:237-254
 * (permutation of 0..11), crypto/monolith.rs:379-392 (the same for AGL),
 * :403-408 (round constants 1,0..3) and transcript.rs:358-371 (golden squeeze).
 *
 * The AGL round constants come from SHA-256 (the reference uses the sha2 crate,
 * version 0.10.8 in zk-torch-4/Cargo.lock); SHA-256 is restated here from
 * FIPS 180-4.
 */
#include "gl.h"
#include "agl.h"
#include <string.h>
#include <stdlib.h>

#define MW 12
#define MROUNDS 6

/* first row of the circulant MDS matrix (cpu_monolith.rs:46-59): row i is row 0 rotated right by i */
static const uint64_t MDS_ROW[MW] = { 7, 23, 8, 26, 13, 10, 9, 7, 6, 22, 21, 8 };

/* cpu_monolith.rs:22-44 */
static const uint64_t GL_RC[MROUNDS + 1][MW] = {
    { 0 },
    { 13596126580325903823ULL, 5676126986831820406ULL, 11349149288412960427ULL, 3368797843020733411ULL,
      16240671731749717664ULL, 9273190757374900239ULL, 14446552112110239438ULL, 4033077683985131644ULL,
      4291229347329361293ULL, 13231607645683636062ULL, 1383651072186713277ULL, 8898815177417587567ULL },
    { 2383619671172821638ULL, 6065528368924797662ULL, 16737578966352303081ULL, 2661700069680749654ULL,
      7414030722730336790ULL, 18124970299993404776ULL, 9169923000283400738ULL, 15832813151034110977ULL,
      16245117847613094506ULL, 11056181639108379773ULL, 10546400734398052938ULL, 8443860941261719174ULL },
    { 15799082741422909885ULL, 13421235861052008152ULL, 15448208253823605561ULL, 2540286744040770964ULL,
      2895626806801935918ULL, 8644593510196221619ULL, 17722491003064835823ULL, 5166255496419771636ULL,
      1015740739405252346ULL, 4400043467547597488ULL, 5176473243271652644ULL, 4517904634837939508ULL },
    { 18341030605319882173ULL, 13366339881666916534ULL, 6291492342503367536ULL, 10004214885638819819ULL,
      4748655089269860551ULL, 1520762444865670308ULL, 8393589389936386108ULL, 11025183333304586284ULL,
      5993305003203422738ULL, 458912836931247573ULL, 5947003897778655410ULL, 17184667486285295106ULL },
    { 15710528677110011358ULL, 8929476121507374707ULL, 2351989866172789037ULL, 11264145846854799752ULL,
      14924075362538455764ULL, 10107004551857451916ULL, 18325221206052792232ULL, 16751515052585522105ULL,
      15305034267720085905ULL, 15639149412312342017ULL, 14624541102106656564ULL, 3542311898554959098ULL },
    { 0 },
};

/* The byte S-box applied to all eight bytes at once (cpu_monolith.rs:97-103):
 * y = rotl8(x ^ (rotl8(~x, 1) & rotl8(x, 2) & rotl8(x, 3)), 1) per byte. */
static inline uint64_t bar_64(uint64_t x) {
    uint64_t l1 = ((~x & 0x8080808080808080ULL) >> 7) | ((~x & 0x7F7F7F7F7F7F7F7FULL) << 1);
    uint64_t l2 = ((x & 0xC0C0C0C0C0C0C0C0ULL) >> 6) | ((x & 0x3F3F3F3F3F3F3F3FULL) << 2);
    uint64_t l3 = ((x & 0xE0E0E0E0E0E0E0E0ULL) >> 5) | ((x & 0x1F1F1F1F1F1F1F1FULL) << 3);
    uint64_t t = x ^ (l1 & l2 & l3);
    return ((t & 0x8080808080808080ULL) >> 7) | ((t & 0x7F7F7F7F7F7F7F7FULL) << 1);
}

/* cpu_monolith.rs:120-131: MDS times state plus round constants, reduced from 128 bits */
static void gl_concrete(uint64_t *s, int round) {
    uint64_t out[MW];
    for (int row = 0; row < MW; row++) {
        u128 acc = GL_RC[round][row];
        for (int col = 0; col < MW; col++) acc += (u128)s[col] * MDS_ROW[(col - row + MW) % MW];
        out[row] = (uint64_t)(acc % GL_P);
    }
    memcpy(s, out, sizeof(out));
}

/* cpu_monolith.rs:137-144. The bars act on the canonical words the preceding
 * concrete layer left; their outputs may exceed p and are reduced by the
 * arithmetic that follows (:111-117 bricks, top index first). */
void gl_monolith_permute(uint64_t s[MW]) {
    gl_concrete(s, 0);
    for (int r = 1; r <= MROUNDS; r++) {
        for (int i = 0; i < 4; i++) s[i] = bar_64(s[i]);
        for (int i = MW - 1; i >= 1; i--) {
            uint64_t prev = s[i - 1] % GL_P;
            s[i] = gl_add(s[i] % GL_P, gl_mul(prev, prev));
        }
        gl_concrete(s, r);
    }
}

void oracle_gl_monolith_permute(uint64_t *s) { gl_monolith_permute(s); }

/* cpu_monolith.rs:150-211: leaf and node hashes, digest = first four words */
void gl_monolith_hash_gl_leaf(uint64_t a, uint64_t b, uint64_t out[4]) {
    uint64_t s[MW] = { a, b };
    gl_monolith_permute(s);
    memcpy(out, s, 32);
}
void gl_monolith_hash_ext2_leaf(ext2_t a, ext2_t b, uint64_t out[4]) {
    uint64_t s[MW] = { a.c0, a.c1, b.c0, b.c1 };
    gl_monolith_permute(s);
    memcpy(out, s, 32);
}
void gl_monolith_compress(const uint64_t l[4], const uint64_t r[4], uint64_t out[4]) {
    uint64_t s[MW] = { 0 };
    memcpy(s, l, 32);
    memcpy(s + 4, r, 32);
    gl_monolith_permute(s);
    memcpy(out, s, 32);
}

/* ------------------------------------------------------------------ */
/* SHA-256 (FIPS 180-4), single-shot, short messages                   */
/* ------------------------------------------------------------------ */
static const uint32_t SHA_K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2,
};
static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

void oracle_sha256(const uint8_t *msg, size_t len, uint8_t out[32]) {
    uint32_t h[8] = { 0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19 };
    size_t total = ((len + 9 + 63) / 64) * 64;
    for (size_t off = 0; off < total; off += 64) {
        uint8_t blk[64];
        for (int i = 0; i < 64; i++) {
            size_t p = off + i;
            if (p < len) blk[i] = msg[p];
            else if (p == len) blk[i] = 0x80;
            else if (p >= total - 8) blk[i] = (uint8_t)(((uint64_t)len * 8) >> (8 * (total - 1 - p)));
            else blk[i] = 0;
        }
        uint32_t w[64];
        for (int i = 0; i < 16; i++)
            w[i] = ((uint32_t)blk[4 * i] << 24) | ((uint32_t)blk[4 * i + 1] << 16) | ((uint32_t)blk[4 * i + 2] << 8) | blk[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
            uint32_t ch = (e & f) ^ (~e & g);
            uint32_t t1 = hh + S1 + ch + SHA_K[i] + w[i];
            uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
            uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
            uint32_t t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    for (int i = 0; i < 8; i++)
        for (int j = 0; j < 4; j++) out[4 * i + j] = (uint8_t)(h[i] >> (24 - 8 * j));
}

/* ------------------------------------------------------------------ */
/* AGL Monolith                                                        */
/* ------------------------------------------------------------------ */
static uint64_t AGL_RC[MROUNDS + 1][MW];
static int agl_rc_ready;

/* crypto/monolith.rs:66-107: SHA-256("AGL-Monolith-RC-v1" || round || pos || salt as
 * little-endian u32), first 8 bytes little-endian, salt incremented until below q;
 * rounds 1..5 only, rounds 0 and 6 stay zero. */
static void agl_rc_init(void) {
    if (agl_rc_ready) return;
    static const char TAG[] = "AGL-Monolith-RC-v1";
    for (uint32_t r = 1; r < MROUNDS; r++) {
        for (uint32_t i = 0; i < MW; i++) {
            for (uint32_t salt = 0;; salt++) {
                uint8_t msg[18 + 12], dg[32];
                memcpy(msg, TAG, 18);
                uint32_t f[3] = { r, i, salt };
                for (int k = 0; k < 3; k++)
                    for (int b = 0; b < 4; b++) msg[18 + 4 * k + b] = (uint8_t)(f[k] >> (8 * b));
                oracle_sha256(msg, sizeof(msg), dg);
                uint64_t v = 0;
                for (int b = 7; b >= 0; b--) v = (v << 8) | dg[b];
                if (v < AGL_Q) { AGL_RC[r][i] = v; break; }
            }
        }
    }
    agl_rc_ready = 1;
}

void oracle_agl_monolith_rc(uint64_t *out) {
    agl_rc_init();
    memcpy(out, AGL_RC, sizeof(AGL_RC));
}

/* crypto/monolith.rs:177-193 */
static void agl_concrete(uint64_t *s, int round) {
    uint64_t out[MW];
    for (int row = 0; row < MW; row++) {
        agl_u128 acc = AGL_RC[round][row];
        for (int col = 0; col < MW; col++) acc += (agl_u128)(s[col] % AGL_Q) * MDS_ROW[(col - row + MW) % MW];
        out[row] = (uint64_t)(acc % AGL_Q);
    }
    memcpy(s, out, sizeof(out));
}

/* crypto/monolith.rs:201-208 */
void agl_monolith_permute(uint64_t s[MW]) {
    agl_rc_init();
    agl_concrete(s, 0);
    for (int r = 1; r <= MROUNDS; r++) {
        for (int i = 0; i < 4; i++) s[i] = bar_64(s[i]);
        for (int i = MW - 1; i >= 1; i--) {
            uint64_t prev = s[i - 1] % AGL_Q;
            s[i] = agl_add(s[i] % AGL_Q, agl_mul(prev, prev));
        }
        agl_concrete(s, r);
    }
}
void oracle_agl_monolith_permute(uint64_t *s) { agl_monolith_permute(s); }

/* ------------------------------------------------------------------ */
/* AGL transcript: width 12, rate 8, overwrite mode, LIFO outputs       */
/* ------------------------------------------------------------------ */
typedef struct {
    uint64_t sponge[MW];
    uint64_t in_buf[8];
    uint64_t out_buf[8];
    int in_count, out_count;
} agl_transcript_t;

/* transcript.rs:209-222 */
static void agl_duplexing(agl_transcript_t *t) {
    for (int i = 0; i < t->in_count; i++) t->sponge[i] = t->in_buf[i];
    for (int i = t->in_count; i < 8; i++) t->sponge[i] = 0;
    t->in_count = 0;
    agl_monolith_permute(t->sponge);
    for (int i = 0; i < 8; i++) t->out_buf[7 - i] = t->sponge[i];
    t->out_count = 8;
}
/* transcript.rs:224-235 */
static void agl_absorb(agl_transcript_t *t, uint64_t v) {
    t->out_count = 0;
    t->in_buf[t->in_count++] = v;
    if (t->in_count == 8) agl_duplexing(t);
}
/* transcript.rs:237-243 */
static uint64_t agl_squeeze(agl_transcript_t *t) {
    if (t->out_count == 0) agl_duplexing(t);
    return t->out_buf[--t->out_count];
}
/* transcript.rs:60-68 */
static void agl_absorb_label(agl_transcript_t *t, const uint8_t *label, size_t n) {
    if (n == 0) return;
    agl_absorb(t, (uint64_t)n);
    for (size_t i = 0; i < n; i++) agl_absorb(t, label[i]);
}

/* A scripted run for the tests: ops[i] = kind (0 append one word, 1 challenge
 * scalar, 2 fork with branch id = value), label i = labels + label_off[i] with
 * length label_len[i]; appended values are reduced mod q (transcript.rs:70-113),
 * challenges are written to out in order. A fork (transcript.rs:168-173)
 * continues on the forked copy. Returns the number of challenges. */
size_t oracle_agl_transcript_run(const uint8_t *init_label, size_t init_len, size_t n_ops, const int *ops,
                                 const uint8_t *labels, const size_t *label_off, const size_t *label_len,
                                 const uint64_t *values, uint64_t *out, uint64_t *state_out) {
    agl_transcript_t t;
    memset(&t, 0, sizeof(t));
    for (size_t i = 0; i < init_len; i++) agl_absorb(&t, init_label[i]); /* transcript.rs:34-47 */
    size_t n_out = 0;
    for (size_t i = 0; i < n_ops; i++) {
        agl_absorb_label(&t, labels + label_off[i], label_len[i]);
        if (ops[i] == 0) agl_absorb(&t, values[i] % AGL_Q);
        else if (ops[i] == 1) out[n_out++] = agl_squeeze(&t);
        else agl_absorb(&t, values[i]);
    }
    if (state_out) memcpy(state_out, t.sponge, sizeof(t.sponge));
    return n_out;
}

/* ------------------------------------------------------------------ */
/* Linear sumcheck over the almost-Goldilocks extension with this       */
/* transcript (zk-torch-4)                                              */
/* ------------------------------------------------------------------ */
static void agl_append_u64(agl_transcript_t *t, const char *label, uint64_t v) { /* transcript.rs:83-88 */
    agl_absorb_label(t, (const uint8_t *)label, strlen(label));
    agl_absorb(t, v % AGL_Q);
}
static void agl_append_ext2(agl_transcript_t *t, const char *label, aext2_t v) { /* transcript.rs:102-106 */
    agl_absorb_label(t, (const uint8_t *)label, strlen(label));
    agl_absorb(t, v.c0 % AGL_Q);
    agl_absorb(t, v.c1 % AGL_Q);
}
static aext2_t agl_challenge_ext2(agl_transcript_t *t, const char *label) { /* transcript.rs:120-125 */
    agl_absorb_label(t, (const uint8_t *)label, strlen(label));
    uint64_t c0 = agl_squeeze(t), c1 = agl_squeeze(t);
    return ae2(c0, c1);
}
static void agl_transcript_init(agl_transcript_t *t, const uint8_t *label, size_t n) { /* transcript.rs:34-47 */
    memset(t, 0, sizeof(*t));
    for (size_t i = 0; i < n; i++) agl_absorb(t, label[i]);
}

/* CpuLinearSumcheckProverExt2::new + prove (zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:23-100),
 * the loop GpuLinearSumcheckProver runs with the same labels (gpu_prover.rs:26-112).
 * polys: d tables of 2^num_var extension elements, poly-major, (c0, c1) words (a base-field
 * table is lifted first: from_base). The transcript starts as Transcript::new(label).
 * Outputs: round_msgs[num_var][d+1][2], challenges[num_var][2], final_evals[d][2],
 * final_eval[2], state12 (sponge words after the proof; may be NULL). */
int oracle_agl_sumcheck_prove(const uint64_t *polys_in, int d, int num_var, int base_field, const uint8_t *label,
                              size_t label_len, uint64_t *round_msgs, uint64_t *challenges, uint64_t *final_evals,
                              uint64_t *final_eval, uint64_t *state12) {
    size_t n = (size_t)1 << num_var;
    aext2_t *p = malloc(sizeof(aext2_t) * n * (size_t)d);
    if (!p) return -1;
    for (size_t i = 0; i < n * (size_t)d; i++)
        p[i] = base_field ? ae2(polys_in[i] % AGL_Q, 0) : ae2(polys_in[2 * i] % AGL_Q, polys_in[2 * i + 1] % AGL_Q);
    agl_transcript_t t;
    agl_transcript_init(&t, label, label_len);
    agl_append_u64(&t, "num_var", (uint64_t)num_var);
    agl_append_u64(&t, "num_poly", (uint64_t)d);
    size_t len = n;
    for (int round = 0; round < num_var; round++) {
        size_t half = len / 2;
        for (int e = 0; e <= d; e++) {
            aext2_t c = ae2((uint64_t)e, 0), sum = ae2(0, 0);
            for (size_t j = 0; j < half; j++) {
                aext2_t prod = ae2(1, 0);
                for (int i = 0; i < d; i++) {
                    aext2_t a = p[(size_t)i * n + 2 * j], b = p[(size_t)i * n + 2 * j + 1];
                    prod = ae2_mul(prod, ae2_add(a, ae2_mul(c, ae2_sub(b, a))));
                }
                sum = ae2_add(sum, prod);
            }
            round_msgs[((size_t)round * (d + 1) + e) * 2] = sum.c0;
            round_msgs[((size_t)round * (d + 1) + e) * 2 + 1] = sum.c1;
        }
        for (int e = 0; e <= d; e++) {
            const uint64_t *w = round_msgs + ((size_t)round * (d + 1) + e) * 2;
            agl_append_ext2(&t, "round_message", ae2(w[0], w[1]));
        }
        aext2_t r = agl_challenge_ext2(&t, "challenge");
        challenges[2 * round] = r.c0;
        challenges[2 * round + 1] = r.c1;
        r = ae2(r.c0 % AGL_Q, r.c1 % AGL_Q);
        for (int i = 0; i < d; i++)
            for (size_t j = 0; j < half; j++) {
                aext2_t a = p[(size_t)i * n + 2 * j], b = p[(size_t)i * n + 2 * j + 1];
                p[(size_t)i * n + j] = ae2_add(a, ae2_mul(r, ae2_sub(b, a)));
            }
        len = half;
    }
    aext2_t prod = ae2(1, 0);
    for (int i = 0; i < d; i++) {
        final_evals[2 * i] = p[(size_t)i * n].c0;
        final_evals[2 * i + 1] = p[(size_t)i * n].c1;
        prod = ae2_mul(prod, p[(size_t)i * n]);
    }
    final_eval[0] = prod.c0;
    final_eval[1] = prod.c1;
    if (state12) memcpy(state12, t.sponge, sizeof(t.sponge));
    free(p);
    return 0;
}

/* verifier.rs:91-113 */
static aext2_t agl_interpolate(const aext2_t *evals, int n, aext2_t x) {
    aext2_t result = ae2(0, 0);
    for (int i = 0; i < n; i++) {
        aext2_t basis = ae2(1, 0);
        for (int j = 0; j < n; j++) {
            if (j == i) continue;
            aext2_t num = ae2_sub(x, ae2((uint64_t)j, 0)), den = ae2_sub(ae2((uint64_t)i, 0), ae2((uint64_t)j, 0));
            basis = ae2_mul(basis, ae2_mul(num, ae2_inv(den)));
        }
        result = ae2_add(result, ae2_mul(basis, evals[i]));
    }
    return result;
}
/* SumcheckVerifier::verify (verifier.rs:14-88): 1 = accepted; challenges written as far as checked. */
int oracle_agl_sumcheck_verify(const uint64_t *round_msgs, const uint64_t *final_eval, const uint64_t *claimed_sum, int d,
                               int num_var, const uint8_t *label, size_t label_len, uint64_t *challenges) {
    agl_transcript_t t;
    agl_transcript_init(&t, label, label_len);
    agl_append_u64(&t, "num_var", (uint64_t)num_var);
    agl_append_u64(&t, "num_poly", (uint64_t)d);
    aext2_t current = ae2(claimed_sum[0] % AGL_Q, claimed_sum[1] % AGL_Q);
    for (int round = 0; round < num_var; round++) {
        aext2_t msg[16];
        for (int e = 0; e <= d; e++) {
            const uint64_t *w = round_msgs + ((size_t)round * (d + 1) + e) * 2;
            msg[e] = ae2(w[0] % AGL_Q, w[1] % AGL_Q);
        }
        aext2_t s = ae2_add(msg[0], msg[1]);
        if (s.c0 != current.c0 || s.c1 != current.c1) return 0;
        for (int e = 0; e <= d; e++) agl_append_ext2(&t, "round_message", msg[e]);
        aext2_t r = agl_challenge_ext2(&t, "challenge");
        challenges[2 * round] = r.c0;
        challenges[2 * round + 1] = r.c1;
        current = agl_interpolate(msg, d + 1, ae2(r.c0 % AGL_Q, r.c1 % AGL_Q));
    }
    return current.c0 == final_eval[0] % AGL_Q && current.c1 == final_eval[1] % AGL_Q;
}

/* ------------------------------------------------------------------ */
/* Same-point sumcheck over the almost-Goldilocks extension             */
/* (zk-torch-4/src/fold/same_point_sumcheck.rs)                         */
/* ------------------------------------------------------------------ */
/* Witness kinds of an instance (FoldData, zk-torch-4/src/fold/mod.rs:107-160):
 *   0  binary, packed: bit j of word j / 64 is f[j]
 *   1  ternary, one chunk: `words` words of +1 masks, then `words` words of -1 masks (words = max(1, 2^(arity-6)))
 *   2  dense base-field table of 2^arity words
 * The dense CPU prover lifts every kind to an extension table first (same_point_sumcheck.rs:924-1030); the
 * small-alphabet round-0 paths of the reference compute the same field elements. */
static void sp_lift(int kind, const uint64_t *w, int arity, aext2_t *out) {
    size_t n = (size_t)1 << arity, words = arity >= 6 ? n >> 6 : 1;
    for (size_t j = 0; j < n; j++) {
        if (kind == 0) out[j] = ae2((w[j >> 6] >> (j & 63)) & 1, 0);
        else if (kind == 1) {
            uint64_t p = (w[j >> 6] >> (j & 63)) & 1, m = (w[words + (j >> 6)] >> (j & 63)) & 1;
            out[j] = ae2(agl_sub(p, m), 0);
        } else out[j] = ae2(w[j] % AGL_Q, 0);
    }
}
static void sp_eq_table(const uint64_t *pt, int arity, aext2_t *out) { /* poly/mod.rs:86-120: variable 0 = bit 0 */
    out[0] = ae2(1, 0);
    for (int i = 0; i < arity; i++) {
        aext2_t ri = ae2(pt[2 * i] % AGL_Q, pt[2 * i + 1] % AGL_Q);
        size_t half = (size_t)1 << i;
        for (size_t j = 0; j < half; j++) {
            aext2_t a = out[j], ar = ae2_mul(a, ri);
            out[j] = ae2_sub(a, ar);
            out[j + half] = ar;
        }
    }
}
/* FoldData::evaluate_at_ext2 (fold/mod.rs:107-110): the multilinear extension of the witness at `pt`. */
void oracle_agl_witness_eval(int kind, const uint64_t *w, int arity, const uint64_t *pt, uint64_t *out2) {
    size_t n = (size_t)1 << arity;
    aext2_t *eq = malloc(sizeof(aext2_t) * n), *f = malloc(sizeof(aext2_t) * n);
    sp_eq_table(pt, arity, eq);
    sp_lift(kind, w, arity, f);
    aext2_t acc = ae2(0, 0);
    for (size_t j = 0; j < n; j++) acc = ae2_add(acc, ae2_mul(eq[j], f[j]));
    out2[0] = acc.c0; out2[1] = acc.c1;
    free(eq); free(f);
}
static aext2_t sp_eq_eval(const uint64_t *a, const aext2_t *b, int n) { /* same_point_sumcheck.rs:907-921 */
    aext2_t acc = ae2(1, 0), one = ae2(1, 0);
    for (int i = 0; i < n; i++) {
        aext2_t ai = ae2(a[2 * i] % AGL_Q, a[2 * i + 1] % AGL_Q);
        acc = ae2_mul(acc, ae2_add(ae2_mul(ai, b[i]), ae2_mul(ae2_sub(one, ai), ae2_sub(one, b[i]))));
    }
    return acc;
}
static void sp_header(agl_transcript_t *t, int M, int N, const int *arity, const uint64_t *pts, const size_t *pt_off,
                      const uint64_t *vals) { /* same_point_sumcheck.rs:78-87 */
    agl_append_u64(t, "sp_num_var", (uint64_t)N);
    agl_append_u64(t, "sp_num_inst", (uint64_t)M);
    for (int i = 0; i < M; i++) {
        agl_append_u64(t, "sp_arity_i", (uint64_t)arity[i]);
        for (int k = 0; k < arity[i]; k++) agl_append_ext2(t, "sp_r_i", ae2(pts[pt_off[i] + 2 * k], pts[pt_off[i] + 2 * k + 1]));
        agl_append_ext2(t, "sp_y_i", ae2(vals[2 * i], vals[2 * i + 1]));
    }
}

/* prove_same_point (same_point_sumcheck.rs:58-157) with the dense per-instance state (:270-470) and
 * compute_round_message (:826-883). M instances; instance i has arity[i] <= N variables (>= 1), claim point
 * pts[pt_off[i] ..] (arity[i] pairs), claim value vals[2 i ..], witness kind[i] at wit + wit_off[i] (words).
 * The transcript starts as Transcript::new(label). Outputs: round_msgs[N][3][2], challenges[N][2], f_evals[M][2],
 * final_eval[2], state12 (sponge after the proof; may be NULL). */
int oracle_agl_same_point_prove(int M, int N, const int *arity, const uint64_t *pts, const size_t *pt_off, const uint64_t *vals,
                                const int *kind, const uint64_t *wit, const size_t *wit_off, const uint8_t *label,
                                size_t label_len, uint64_t *round_msgs, uint64_t *challenges, uint64_t *f_evals,
                                uint64_t *final_eval, uint64_t *state12) {
    if (M < 1 || N < 1) return -2;
    for (int i = 0; i < M; i++) if (arity[i] < 1 || arity[i] > N) return -2;
    agl_transcript_t t;
    agl_transcript_init(&t, label, label_len);
    sp_header(&t, M, N, arity, pts, pt_off, vals);
    aext2_t alpha = agl_challenge_ext2(&t, "sp_alpha");
    aext2_t *alphas = malloc(sizeof(aext2_t) * M), **eq = malloc(sizeof(void *) * M), **f = malloc(sizeof(void *) * M);
    aext2_t *constant = malloc(sizeof(aext2_t) * M), *R = malloc(sizeof(aext2_t) * N);
    size_t *len = malloc(sizeof(size_t) * M);
    aext2_t *contrib = malloc(sizeof(aext2_t) * 3 * M);
    aext2_t pw = ae2(1, 0);
    for (int i = 0; i < M; i++) {
        alphas[i] = pw;
        pw = ae2_mul(pw, alpha);
        len[i] = (size_t)1 << arity[i];
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < M; i++) {
        eq[i] = malloc(sizeof(aext2_t) * len[i]);
        f[i] = malloc(sizeof(aext2_t) * len[i]);
        sp_eq_table(pts + pt_off[i], arity[i], eq[i]);
        sp_lift(kind[i], wit + wit_off[i], arity[i], f[i]);
    }
    const aext2_t two = ae2(2, 0);
    for (int round = 0; round < N; round++) {
        aext2_t msg[3] = { ae2(0, 0), ae2(0, 0), ae2(0, 0) };
        const aext2_t pow_remaining = ae2((uint64_t)1 << (N - round - 1), 0);
        /* instances in parallel (the reference uses rayon over leaves); field sums do not depend on the order */
#pragma omp parallel for schedule(dynamic, 1)
        for (int i = 0; i < M; i++) {
            aext2_t *out = contrib + 3 * (size_t)i;
            if (round >= arity[i]) { /* constant mode: alpha^i 2^(N - round - 1) eq_i(R) f_i(R) at all three points */
                aext2_t w = ae2_mul(alphas[i], ae2_mul(pow_remaining, constant[i]));
                out[0] = out[1] = out[2] = w;
                continue;
            }
            size_t half = len[i] / 2;
            aext2_t s0 = ae2(0, 0), s1 = ae2(0, 0), s2 = ae2(0, 0);
            for (size_t j = 0; j < half; j++) {
                aext2_t e0 = eq[i][2 * j], e1 = eq[i][2 * j + 1], f0 = f[i][2 * j], f1 = f[i][2 * j + 1];
                aext2_t e2v = ae2_sub(ae2_mul(two, e1), e0), f2v = ae2_sub(ae2_mul(two, f1), f0);
                s0 = ae2_add(s0, ae2_mul(e0, f0));
                s1 = ae2_add(s1, ae2_mul(e1, f1));
                s2 = ae2_add(s2, ae2_mul(e2v, f2v));
            }
            aext2_t scale = ae2_mul(alphas[i], ae2((uint64_t)1 << (N - arity[i]), 0));
            out[0] = ae2_mul(scale, s0);
            out[1] = ae2_mul(scale, s1);
            out[2] = ae2_mul(scale, s2);
        }
        for (int i = 0; i < M; i++)
            for (int c = 0; c < 3; c++) msg[c] = ae2_add(msg[c], contrib[3 * (size_t)i + c]);
        for (int c = 0; c < 3; c++) {
            agl_append_ext2(&t, "sp_round_msg", msg[c]);
            round_msgs[((size_t)round * 3 + c) * 2] = msg[c].c0;
            round_msgs[((size_t)round * 3 + c) * 2 + 1] = msg[c].c1;
        }
        aext2_t r = agl_challenge_ext2(&t, "sp_round_challenge");
        challenges[2 * round] = r.c0;
        challenges[2 * round + 1] = r.c1;
        R[round] = r;
#pragma omp parallel for schedule(dynamic, 1)
        for (int i = 0; i < M; i++) {
            if (round >= arity[i]) continue;
            size_t half = len[i] / 2;
            for (size_t j = 0; j < half; j++) {
                aext2_t a = eq[i][2 * j], b = eq[i][2 * j + 1];
                eq[i][j] = ae2_add(a, ae2_mul(r, ae2_sub(b, a)));
                a = f[i][2 * j]; b = f[i][2 * j + 1];
                f[i][j] = ae2_add(a, ae2_mul(r, ae2_sub(b, a)));
            }
            len[i] = half;
            if (round + 1 == arity[i]) constant[i] = ae2_mul(eq[i][0], f[i][0]);
        }
    }
    aext2_t fin = ae2(0, 0);
    for (int i = 0; i < M; i++) {
        f_evals[2 * i] = f[i][0].c0;
        f_evals[2 * i + 1] = f[i][0].c1;
        agl_append_ext2(&t, "sp_f_eval", f[i][0]);
    }
    for (int i = 0; i < M; i++) {
        aext2_t eq_i = sp_eq_eval(pts + pt_off[i], R, arity[i]);
        fin = ae2_add(fin, ae2_mul(alphas[i], ae2_mul(eq_i, f[i][0])));
    }
    final_eval[0] = fin.c0;
    final_eval[1] = fin.c1;
    if (state12) memcpy(state12, t.sponge, sizeof(t.sponge));
    for (int i = 0; i < M; i++) { free(eq[i]); free(f[i]); }
    free(alphas); free(eq); free(f); free(constant); free(R); free(len); free(contrib);
    return 0;
}

/* verify_same_point (same_point_sumcheck.rs:161-219). Returns 1 and writes the challenges when the proof is
 * accepted, 0 otherwise. */
int oracle_agl_same_point_verify(int M, int N, const int *arity, const uint64_t *pts, const size_t *pt_off, const uint64_t *vals,
                                 const uint64_t *round_msgs, const uint64_t *f_evals, const uint64_t *final_eval,
                                 const uint8_t *label, size_t label_len, uint64_t *challenges) {
    if (M < 1) return 0;
    agl_transcript_t t;
    agl_transcript_init(&t, label, label_len);
    sp_header(&t, M, N, arity, pts, pt_off, vals);
    aext2_t alpha = agl_challenge_ext2(&t, "sp_alpha");
    aext2_t *alphas = malloc(sizeof(aext2_t) * M), *R = malloc(sizeof(aext2_t) * N);
    aext2_t pw = ae2(1, 0), current = ae2(0, 0);
    for (int i = 0; i < M; i++) {
        alphas[i] = pw;
        pw = ae2_mul(pw, alpha);
        aext2_t y = ae2(vals[2 * i] % AGL_Q, vals[2 * i + 1] % AGL_Q);
        current = ae2_add(current, ae2_mul(alphas[i], ae2_mul(y, ae2((uint64_t)1 << (N - arity[i]), 0))));
    }
    int ok = 1;
    for (int round = 0; round < N && ok; round++) {
        aext2_t m[3];
        for (int c = 0; c < 3; c++) m[c] = ae2(round_msgs[((size_t)round * 3 + c) * 2] % AGL_Q, round_msgs[((size_t)round * 3 + c) * 2 + 1] % AGL_Q);
        aext2_t sum = ae2_add(m[0], m[1]);
        if (sum.c0 != current.c0 || sum.c1 != current.c1) { ok = 0; break; }
        for (int c = 0; c < 3; c++) agl_append_ext2(&t, "sp_round_msg", m[c]);
        aext2_t r = agl_challenge_ext2(&t, "sp_round_challenge");
        R[round] = r;
        if (challenges) { challenges[2 * round] = r.c0; challenges[2 * round + 1] = r.c1; }
        current = agl_interpolate(m, 3, r);
    }
    if (ok) {
        aext2_t expected = ae2(0, 0);
        for (int i = 0; i < M; i++) agl_append_ext2(&t, "sp_f_eval", ae2(f_evals[2 * i], f_evals[2 * i + 1]));
        for (int i = 0; i < M; i++) {
            aext2_t fe = ae2(f_evals[2 * i] % AGL_Q, f_evals[2 * i + 1] % AGL_Q);
            expected = ae2_add(expected, ae2_mul(alphas[i], ae2_mul(sp_eq_eval(pts + pt_off[i], R, arity[i]), fe)));
        }
        if (current.c0 != expected.c0 || current.c1 != expected.c1) ok = 0;
        if (final_eval[0] % AGL_Q != expected.c0 || final_eval[1] % AGL_Q != expected.c1) ok = 0;
    }
    free(alphas); free(R);
    return ok;
}
