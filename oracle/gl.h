/*
 * CPU oracle (test infrastructure, not the product): Goldilocks field, its
 * quadratic extension, Poseidon2 width 8 and the duplex transcript.
 *
 * Every function restates the reference's CPU arithmetic and cites the file
 * and lines it follows. All values are canonical residues in [0, p).
 *
 * Only tests, the smoke check and the benchmark's cpu_baseline leg may link
 * or load this code. The CUDA library never does.
 */
#ifndef ORACLE_GL_H
#define ORACLE_GL_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GL_P 0xFFFFFFFF00000001ULL

typedef unsigned __int128 u128;

/* goldilocks-cuda-rs/src/field.rs:34-40 (reduce), :55-66 (add), :70-79 (sub),
 * :83-106 (mul). Inputs here are always canonical, so one conditional
 * subtraction suffices where the reference uses the same. */
static inline uint64_t gl_canon(uint64_t v) { return v >= GL_P ? v - GL_P : v; }

static inline uint64_t gl_add(uint64_t a, uint64_t b) {
    u128 s = (u128)a + b;
    if (s >= GL_P) s -= GL_P;
    return (uint64_t)s;
}
static inline uint64_t gl_sub(uint64_t a, uint64_t b) {
    return a >= b ? a - b : a + (GL_P - b);
}
static inline uint64_t gl_neg(uint64_t a) { return a ? GL_P - a : 0; }

static inline uint64_t gl_mul(uint64_t a, uint64_t b) {
    u128 full = (u128)a * b;
    uint64_t lo = (uint64_t)full, hi = (uint64_t)(full >> 64);
    /* 2^64 = 2^32 - 1 (mod p), 2^96 = -1 (mod p) */
    uint64_t hh = hi >> 32, hl = hi & 0xFFFFFFFFULL;
    uint64_t t = lo;
    if (t < hh) t += GL_P;       /* lo - hh with borrow folded in (wraps mod 2^64) */
    t -= hh;
    uint64_t m = hl * 0xFFFFFFFFULL; /* < 2^64 */
    u128 r = (u128)t + m;
    if (r >= GL_P) r -= GL_P;
    if (r >= GL_P) r -= GL_P;
    return (uint64_t)r;
}

uint64_t gl_pow(uint64_t a, uint64_t e);
uint64_t gl_inv(uint64_t a);

/* Quadratic extension F_p[X]/(X^2 - 7): goldilocks-cuda-rs/src/extension.rs:10-125 */
typedef struct { uint64_t c0, c1; } ext2_t;

static inline ext2_t e2(uint64_t c0, uint64_t c1) { ext2_t r = { c0, c1 }; return r; }
static inline ext2_t e2_add(ext2_t a, ext2_t b) { return e2(gl_add(a.c0, b.c0), gl_add(a.c1, b.c1)); }
static inline ext2_t e2_sub(ext2_t a, ext2_t b) { return e2(gl_sub(a.c0, b.c0), gl_sub(a.c1, b.c1)); }
static inline ext2_t e2_mul(ext2_t a, ext2_t b) {
    uint64_t m0 = gl_mul(a.c0, b.c0), m1 = gl_mul(a.c1, b.c1);
    uint64_t cross = gl_add(gl_mul(a.c0, b.c1), gl_mul(a.c1, b.c0));
    return e2(gl_add(m0, gl_mul(7, m1)), cross);
}
static inline ext2_t e2_mul_base(ext2_t a, uint64_t b) { return e2(gl_mul(a.c0, b), gl_mul(a.c1, b)); }
ext2_t e2_inv(ext2_t a);

/* Poseidon2 width 8: goldilocks-cuda-rs/src/cpu_poseidon2.rs:16-141 */
void gl_poseidon2_permute(uint64_t state[8]);

/* Duplex transcript, width 8, rate 4: zk-torch-3/src/transcript.rs:174-350 */
typedef struct {
    uint64_t sponge[8];
    uint64_t in_buf[4];
    uint64_t out_buf[4];
    int in_count;
    int out_count;
    uint64_t permutations; /* bookkeeping only: number of duplexings so far */
} gl_transcript_t;

void gl_transcript_new(gl_transcript_t *t, const uint8_t *label, size_t label_len);
void gl_transcript_absorb(gl_transcript_t *t, uint64_t v);
uint64_t gl_transcript_squeeze(gl_transcript_t *t);
void gl_transcript_append_u64(gl_transcript_t *t, const char *label, uint64_t v);
void gl_transcript_append_scalar(gl_transcript_t *t, const char *label, uint64_t v);
void gl_transcript_append_ext2(gl_transcript_t *t, const char *label, ext2_t v);
uint64_t gl_transcript_challenge_scalar(gl_transcript_t *t, const char *label);
ext2_t gl_transcript_challenge_ext2(gl_transcript_t *t, const char *label);

/* Merkle hashing: goldilocks-cuda-rs/src/cpu_poseidon2.rs:145-183 */
void gl_hash_gl_leaf(uint64_t a, uint64_t b, uint64_t out[4]);
void gl_hash_ext2_leaf(ext2_t a, ext2_t b, uint64_t out[4]);
void gl_compress(const uint64_t l[4], const uint64_t r[4], uint64_t out[4]);
/* 0 = Poseidon2 (default), 1 = Monolith for the three functions above */
void oracle_set_merkle_hash(int h);
int oracle_get_merkle_hash(void);

/* Monolith width 12: goldilocks-cuda-rs/src/cpu_monolith.rs:18-211 */
void gl_monolith_permute(uint64_t state[12]);
void gl_monolith_hash_gl_leaf(uint64_t a, uint64_t b, uint64_t out[4]);
void gl_monolith_hash_ext2_leaf(ext2_t a, ext2_t b, uint64_t out[4]);
void gl_monolith_compress(const uint64_t l[4], const uint64_t r[4], uint64_t out[4]);

#ifdef __cplusplus
}
#endif
#endif
