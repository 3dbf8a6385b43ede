/*
 * CPU oracle (test infrastructure, not the product): almost-Goldilocks field
 * q = 2^64 - 2^32 - 31 and its quadratic extension X^2 = 3, canonical residues.
 * Follows almost-goldilocks-cuda-rs/src/field.rs:34-119 (host ops canonicalise)
 * and cuda_almost_goldilocks/almost_extension.cuh:99-110 (extension product).
 */
#ifndef ORACLE_AGL_H
#define ORACLE_AGL_H
#include <stdint.h>
#include <stddef.h>
typedef unsigned __int128 agl_u128;
#define AGL_Q 0xFFFFFFFEFFFFFFE1ULL

static inline uint64_t agl_canon(uint64_t v) { return v >= AGL_Q ? v - AGL_Q : v; }
static inline uint64_t agl_add(uint64_t a, uint64_t b) { agl_u128 s = (agl_u128)a + b; if (s >= AGL_Q) s -= AGL_Q; return (uint64_t)s; }
static inline uint64_t agl_sub(uint64_t a, uint64_t b) { return a >= b ? a - b : a + (AGL_Q - b); }
static inline uint64_t agl_mul(uint64_t a, uint64_t b) { return (uint64_t)(((agl_u128)a * b) % AGL_Q); }
static inline uint64_t agl_pow(uint64_t a, uint64_t e) { uint64_t r = 1; while (e) { if (e & 1) r = agl_mul(r, a); a = agl_mul(a, a); e >>= 1; } return r; }
static inline uint64_t agl_inv(uint64_t a) { return agl_pow(a, AGL_Q - 2); }

typedef struct { uint64_t c0, c1; } aext2_t;
static inline aext2_t ae2(uint64_t c0, uint64_t c1) { aext2_t r = { c0, c1 }; return r; }
static inline aext2_t ae2_add(aext2_t a, aext2_t b) { return ae2(agl_add(a.c0, b.c0), agl_add(a.c1, b.c1)); }
static inline aext2_t ae2_sub(aext2_t a, aext2_t b) { return ae2(agl_sub(a.c0, b.c0), agl_sub(a.c1, b.c1)); }
static inline aext2_t ae2_mul(aext2_t a, aext2_t b) {
    uint64_t m0 = agl_mul(a.c0, b.c0), m1 = agl_mul(a.c1, b.c1);
    return ae2(agl_add(m0, agl_mul(3, m1)), agl_add(agl_mul(a.c0, b.c1), agl_mul(a.c1, b.c0)));
}
/* 1 / (c0 + c1 X) = (c0 - c1 X) / (c0^2 - 3 c1^2); the inverse of zero is zero */
static inline aext2_t ae2_inv(aext2_t a) {
    uint64_t n = agl_sub(agl_mul(a.c0, a.c0), agl_mul(3, agl_mul(a.c1, a.c1)));
    uint64_t ni = agl_inv(n);
    return ae2(agl_mul(a.c0, ni), agl_mul(agl_sub(0, a.c1), ni));
}
#endif
