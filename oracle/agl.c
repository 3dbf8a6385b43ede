/*
 * CPU oracle (test infrastructure, not the product): almost-Goldilocks sumcheck
 * round message / fold, eq tables and partial evaluation, base field and
 * extension. Same algorithms as the Goldilocks oracle (sumcheck.c) over the
 * other field: zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100 (message, fold),
 * cuda_almost_goldilocks/almost_eq_lagrange.cuh:25-60 (eq step),
 * cuda_almost_goldilocks/almost_partial_eval.cuh:22-83 (partial evaluation).
 */
#include "agl.h"
#include <string.h>
#define MAX_D 8

uint64_t oracle_agl_mul(uint64_t a, uint64_t b) { return agl_mul(agl_canon(a), agl_canon(b)); }
uint64_t oracle_agl_inv(uint64_t a) { return agl_inv(agl_canon(a)); }
void oracle_aext2_mul(const uint64_t *a, const uint64_t *b, uint64_t *o) {
    aext2_t r = ae2_mul(ae2(agl_canon(a[0]), agl_canon(a[1])), ae2(agl_canon(b[0]), agl_canon(b[1])));
    o[0] = r.c0; o[1] = r.c1;
}

void oracle_agl_round_message(const uint64_t *polys, int d, size_t stride, size_t half, uint64_t *out) {
    uint64_t acc[MAX_D + 1] = { 0 };
    for (size_t y = 0; y < half; y++) {
        uint64_t val[MAX_D], diff[MAX_D];
        for (int i = 0; i < d; i++) {
            uint64_t a = agl_canon(polys[i * stride + 2 * y]), b = agl_canon(polys[i * stride + 2 * y + 1]);
            val[i] = a; diff[i] = agl_sub(b, a);
        }
        for (int c = 0; c <= d; c++) {
            uint64_t prod = 1;
            for (int i = 0; i < d; i++) { prod = agl_mul(prod, val[i]); val[i] = agl_add(val[i], diff[i]); }
            acc[c] = agl_add(acc[c], prod);
        }
    }
    memcpy(out, acc, sizeof(uint64_t) * (d + 1));
}
void oracle_agl_fold(const uint64_t *in, uint64_t *out, uint64_t r, int d, size_t stride, size_t half) {
    r = agl_canon(r);
    for (int i = 0; i < d; i++)
        for (size_t y = 0; y < half; y++) {
            uint64_t a = agl_canon(in[i * stride + 2 * y]), b = agl_canon(in[i * stride + 2 * y + 1]);
            out[i * stride + y] = agl_add(a, agl_mul(r, agl_sub(b, a)));
        }
}
void oracle_aext2_round_message(const uint64_t *polys, int d, size_t stride, size_t half, uint64_t *out) {
    aext2_t acc[MAX_D + 1];
    for (int c = 0; c <= d; c++) acc[c] = ae2(0, 0);
    for (size_t y = 0; y < half; y++) {
        aext2_t val[MAX_D], diff[MAX_D];
        for (int i = 0; i < d; i++) {
            const uint64_t *p = polys + (i * stride + 2 * y) * 2;
            aext2_t a = ae2(agl_canon(p[0]), agl_canon(p[1])), b = ae2(agl_canon(p[2]), agl_canon(p[3]));
            val[i] = a; diff[i] = ae2_sub(b, a);
        }
        for (int c = 0; c <= d; c++) {
            aext2_t prod = ae2(1, 0);
            for (int i = 0; i < d; i++) { prod = ae2_mul(prod, val[i]); val[i] = ae2_add(val[i], diff[i]); }
            acc[c] = ae2_add(acc[c], prod);
        }
    }
    for (int c = 0; c <= d; c++) { out[2 * c] = acc[c].c0; out[2 * c + 1] = acc[c].c1; }
}
void oracle_aext2_fold(const uint64_t *in, uint64_t *out, uint64_t r0, uint64_t r1, int d, size_t stride, size_t half) {
    aext2_t r = ae2(agl_canon(r0), agl_canon(r1));
    for (int i = 0; i < d; i++)
        for (size_t y = 0; y < half; y++) {
            const uint64_t *p = in + (i * stride + 2 * y) * 2;
            aext2_t a = ae2(agl_canon(p[0]), agl_canon(p[1])), b = ae2(agl_canon(p[2]), agl_canon(p[3]));
            aext2_t v = ae2_add(a, ae2_mul(r, ae2_sub(b, a)));
            out[(i * stride + y) * 2] = v.c0; out[(i * stride + y) * 2 + 1] = v.c1;
        }
}
/* base tables in, extension challenge, extension tables out (stride_out in extension elements) */
void oracle_aext2_fold_mixed(const uint64_t *in, uint64_t *out, uint64_t r0, uint64_t r1, int d, size_t stride_in,
                             size_t stride_out, size_t half) {
    aext2_t r = ae2(agl_canon(r0), agl_canon(r1));
    for (int i = 0; i < d; i++)
        for (size_t y = 0; y < half; y++) {
            uint64_t a = agl_canon(in[i * stride_in + 2 * y]), b = agl_canon(in[i * stride_in + 2 * y + 1]);
            aext2_t v = ae2_add(ae2(a, 0), ae2_mul(r, ae2(agl_sub(b, a), 0)));
            out[(i * stride_out + y) * 2] = v.c0; out[(i * stride_out + y) * 2 + 1] = v.c1;
        }
}
void oracle_agl_eq_base(const uint64_t *point, int nv, uint64_t *out) {
    size_t n = (size_t)1 << nv;
    memset(out, 0, sizeof(uint64_t) * n);
    out[0] = 1;
    for (int i = 0; i < nv; i++) {
        uint64_t ri = agl_canon(point[i]);
        size_t half = (size_t)1 << i;
        for (size_t j = 0; j < half; j++) { uint64_t a = out[j], ar = agl_mul(a, ri); out[j] = agl_sub(a, ar); out[j + half] = ar; }
    }
}
void oracle_agl_eq_ext2(const uint64_t *point, int nv, uint64_t *out) {
    size_t n = (size_t)1 << nv;
    memset(out, 0, sizeof(uint64_t) * 2 * n);
    out[0] = 1;
    for (int i = 0; i < nv; i++) {
        aext2_t ri = ae2(agl_canon(point[2 * i]), agl_canon(point[2 * i + 1]));
        size_t half = (size_t)1 << i;
        for (size_t j = 0; j < half; j++) {
            aext2_t a = ae2(out[2 * j], out[2 * j + 1]), ar = ae2_mul(a, ri), lo = ae2_sub(a, ar);
            out[2 * j] = lo.c0; out[2 * j + 1] = lo.c1;
            out[2 * (j + half)] = ar.c0; out[2 * (j + half) + 1] = ar.c1;
        }
    }
}
/* fix the m low variables; base field in place semantics: out has 2^(log_n-m) */
void oracle_agl_partial_eval(const uint64_t *in, uint64_t *out, const uint64_t *r, int log_n, int m) {
    size_t n = (size_t)1 << log_n;
    uint64_t *cur = (uint64_t *)__builtin_malloc(sizeof(uint64_t) * n);
    for (size_t i = 0; i < n; i++) cur[i] = agl_canon(in[i]);
    for (int i = 0; i < m; i++) {
        n /= 2;
        uint64_t ri = agl_canon(r[i]);
        for (size_t y = 0; y < n; y++) cur[y] = agl_add(cur[2 * y], agl_mul(ri, agl_sub(cur[2 * y + 1], cur[2 * y])));
    }
    memcpy(out, cur, sizeof(uint64_t) * n);
    __builtin_free(cur);
}
void oracle_agl_partial_eval_ext2_from_base(const uint64_t *in, uint64_t *out, const uint64_t *r, int log_n, int m) {
    size_t n = (size_t)1 << log_n;
    aext2_t *cur = (aext2_t *)__builtin_malloc(sizeof(aext2_t) * n);
    for (size_t i = 0; i < n; i++) cur[i] = ae2(agl_canon(in[i]), 0);
    for (int i = 0; i < m; i++) {
        n /= 2;
        aext2_t ri = ae2(agl_canon(r[2 * i]), agl_canon(r[2 * i + 1]));
        for (size_t y = 0; y < n; y++) cur[y] = ae2_add(cur[2 * y], ae2_mul(ri, ae2_sub(cur[2 * y + 1], cur[2 * y])));
    }
    for (size_t y = 0; y < n; y++) { out[2 * y] = cur[y].c0; out[2 * y + 1] = cur[y].c1; }
    __builtin_free(cur);
}
