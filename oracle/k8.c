/*
 * CPU oracle (test infrastructure, not the product): the field
 * K = F_q[Theta]/(Theta^8 - 3) over almost-Goldilocks and the product sumcheck
 * over tables of K elements.
 *
 *   field      zk-torch-4/src/morpheus/field8.rs:56-121 (add, sub, mul_ref)
 *   eq table   zk-torch-4/src/morpheus/field8.rs:160-182
 *   round sums zk-torch-4/src/morpheus/piop/mod.rs:797-812
 *   fold       zk-torch-4/src/morpheus/piop/mod.rs:831-835
 *
 * The reference pins no K8 value (its tests are ring identities, field8.rs:193-256);
 * the tests here check the same identities and an independent big-integer product.
 */
#include "agl.h"
#include <string.h>
#include <stdlib.h>

typedef struct { uint64_t c[8]; } k8_t;

static k8_t k8_add(k8_t a, k8_t b) { k8_t r; for (int i = 0; i < 8; i++) r.c[i] = agl_add(a.c[i] % AGL_Q, b.c[i] % AGL_Q); return r; }
static k8_t k8_sub(k8_t a, k8_t b) { k8_t r; for (int i = 0; i < 8; i++) r.c[i] = agl_sub(a.c[i] % AGL_Q, b.c[i] % AGL_Q); return r; }

/* field8.rs:104-121: every product reduced, the wrapped half scaled by 3 */
static k8_t k8_mul(k8_t a, k8_t b) {
    agl_u128 lo[8] = { 0 }, hi[8] = { 0 };
    for (int i = 0; i < 8; i++)
        for (int j = 0; j < 8; j++) {
            agl_u128 p = agl_mul(a.c[i] % AGL_Q, b.c[j] % AGL_Q);
            if (i + j < 8) lo[i + j] += p; else hi[i + j - 8] += p;
        }
    k8_t r;
    for (int k = 0; k < 8; k++) r.c[k] = (uint64_t)((lo[k] + 3 * (agl_u128)(uint64_t)(hi[k] % AGL_Q)) % AGL_Q);
    return r;
}

void oracle_k8_add(const uint64_t *a, const uint64_t *b, uint64_t *o) { k8_t x, y; memcpy(&x, a, 64); memcpy(&y, b, 64); x = k8_add(x, y); memcpy(o, &x, 64); }
void oracle_k8_sub(const uint64_t *a, const uint64_t *b, uint64_t *o) { k8_t x, y; memcpy(&x, a, 64); memcpy(&y, b, 64); x = k8_sub(x, y); memcpy(o, &x, 64); }
void oracle_k8_mul(const uint64_t *a, const uint64_t *b, uint64_t *o) { k8_t x, y; memcpy(&x, a, 64); memcpy(&y, b, 64); x = k8_mul(x, y); memcpy(o, &x, 64); }

/* field8.rs:160-182: bit j of the index matches point[j] */
void oracle_k8_eq_table(const uint64_t *point, int n, uint64_t *out) {
    k8_t *t = (k8_t *)out;
    size_t size = (size_t)1 << n;
    memset(t, 0, size * 64);
    t[0].c[0] = 1;
    k8_t one = { { 1, 0, 0, 0, 0, 0, 0, 0 } };
    for (int i = 0; i < n; i++) {
        size_t half = (size_t)1 << i;
        k8_t ri, omr;
        memcpy(&ri, point + 8 * i, 64);
        omr = k8_sub(one, ri);
        for (size_t j = half; j-- > 0;) {
            t[j | half] = k8_mul(t[j], ri);
            t[j] = k8_mul(t[j], omr);
        }
    }
}

/* piop/mod.rs:797-812: s[t] = sum_k prod_j (T_j[2k] + t (T_j[2k+1] - T_j[2k])), t = 0..d */
void oracle_k8_sc_round(const uint64_t *const *tabs, int ntab, size_t len, int d, uint64_t *out) {
    k8_t acc[8];
    memset(acc, 0, sizeof(acc));
    for (size_t k = 0; k < len / 2; k++) {
        k8_t vals[8], diffs[8];
        for (int j = 0; j < ntab; j++) {
            const k8_t *t = (const k8_t *)tabs[j];
            vals[j] = k8_add(t[2 * k], (k8_t){ { 0 } });
            diffs[j] = k8_sub(t[2 * k + 1], t[2 * k]);
        }
        for (int tt = 0; tt <= d; tt++) {
            if (tt > 0) for (int j = 0; j < ntab; j++) vals[j] = k8_add(vals[j], diffs[j]);
            k8_t p = vals[0];
            for (int j = 1; j < ntab; j++) p = k8_mul(p, vals[j]);
            acc[tt] = k8_add(acc[tt], p);
        }
    }
    memcpy(out, acc, (size_t)(d + 1) * 64);
}

/* piop/mod.rs:831-835: out[k] = t[2k] + r (t[2k+1] - t[2k]) */
void oracle_k8_sc_fold(const uint64_t *in, size_t len, const uint64_t *r, uint64_t *out) {
    const k8_t *t = (const k8_t *)in;
    k8_t rr;
    memcpy(&rr, r, 64);
    k8_t *o = (k8_t *)out;
    for (size_t k = 0; k < len / 2; k++) o[k] = k8_add(t[2 * k], k8_mul(rr, k8_sub(t[2 * k + 1], t[2 * k])));
}

/* out[x] += c * in[x] */
void oracle_k8_axpy(uint64_t *out, const uint64_t *in, size_t n, const uint64_t *c) {
    k8_t cc;
    memcpy(&cc, c, 64);
    k8_t *o = (k8_t *)out;
    const k8_t *t = (const k8_t *)in;
    for (size_t x = 0; x < n; x++) o[x] = k8_add(o[x], k8_mul(t[x], cc));
}
