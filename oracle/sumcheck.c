/*
 * CPU oracle (test infrastructure, not the product): the linear sumcheck
 * prover over Goldilocks and its quadratic extension.
 *
 * Follows zk-torch-3/src/sumcheck/cpu_ext2_prover.rs:21-113 (protocol and
 * transcript order) and the host checks in
 * goldilocks-cuda-rs/src/sumcheck_prover.rs:447-481 (base-field message and
 * fold). Loops are parallelised with OpenMP; sums of canonical residues do not
 * depend on the order of addition.
 */
#include "gl.h"
#include <stdlib.h>
#include <string.h>

#define MAX_D 8

/* Round message over the base field: P(c) = sum_y prod_i (a_i + c (b_i - a_i)),
 * c = 0..d, with a_i = poly_i[2y], b_i = poly_i[2y+1]. Tables are poly-major
 * with stride `stride` elements. */
void oracle_gl_round_message(const uint64_t *polys, int d, size_t stride, size_t half,
                             uint64_t *out /* d+1 */) {
    uint64_t acc[MAX_D + 1] = { 0 };
#pragma omp parallel
    {
        uint64_t loc[MAX_D + 1] = { 0 };
#pragma omp for schedule(static) nowait
        for (size_t y = 0; y < half; y++) {
            uint64_t val[MAX_D], diff[MAX_D];
            for (int i = 0; i < d; i++) {
                uint64_t a = polys[i * stride + 2 * y], b = polys[i * stride + 2 * y + 1];
                val[i] = a;
                diff[i] = gl_sub(b, a);
            }
            for (int c = 0; c <= d; c++) {
                uint64_t prod = 1;
                for (int i = 0; i < d; i++) {
                    prod = gl_mul(prod, val[i]);
                    val[i] = gl_add(val[i], diff[i]);
                }
                loc[c] = gl_add(loc[c], prod);
            }
        }
#pragma omp critical
        for (int c = 0; c <= d; c++) acc[c] = gl_add(acc[c], loc[c]);
    }
    memcpy(out, acc, sizeof(uint64_t) * (d + 1));
}

/* out[i*stride + y] = a + r (b - a) */
void oracle_gl_fold(const uint64_t *in, uint64_t *out, uint64_t r, int d, size_t stride, size_t half) {
    for (int i = 0; i < d; i++) {
#pragma omp parallel for schedule(static)
        for (size_t y = 0; y < half; y++) {
            uint64_t a = in[i * stride + 2 * y], b = in[i * stride + 2 * y + 1];
            out[i * stride + y] = gl_add(a, gl_mul(r, gl_sub(b, a)));
        }
    }
}

/* Extension-field twins. Tables hold interleaved (c0, c1); stride counts
 * extension elements. */
void oracle_gl_round_message_ext2(const uint64_t *polys, int d, size_t stride, size_t half,
                                  uint64_t *out /* (d+1)*2 */) {
    ext2_t acc[MAX_D + 1];
    for (int c = 0; c <= d; c++) acc[c] = e2(0, 0);
#pragma omp parallel
    {
        ext2_t loc[MAX_D + 1];
        for (int c = 0; c <= d; c++) loc[c] = e2(0, 0);
#pragma omp for schedule(static) nowait
        for (size_t y = 0; y < half; y++) {
            ext2_t val[MAX_D], diff[MAX_D];
            for (int i = 0; i < d; i++) {
                const uint64_t *p = polys + (i * stride + 2 * y) * 2;
                ext2_t a = e2(p[0], p[1]), b = e2(p[2], p[3]);
                val[i] = a;
                diff[i] = e2_sub(b, a);
            }
            for (int c = 0; c <= d; c++) {
                ext2_t prod = e2(1, 0);
                for (int i = 0; i < d; i++) {
                    prod = e2_mul(prod, val[i]);
                    val[i] = e2_add(val[i], diff[i]);
                }
                loc[c] = e2_add(loc[c], prod);
            }
        }
#pragma omp critical
        for (int c = 0; c <= d; c++) acc[c] = e2_add(acc[c], loc[c]);
    }
    for (int c = 0; c <= d; c++) { out[2 * c] = acc[c].c0; out[2 * c + 1] = acc[c].c1; }
}

void oracle_gl_fold_ext2(const uint64_t *in, uint64_t *out, uint64_t r0, uint64_t r1,
                         int d, size_t stride, size_t half) {
    ext2_t r = e2(r0, r1);
    for (int i = 0; i < d; i++) {
#pragma omp parallel for schedule(static)
        for (size_t y = 0; y < half; y++) {
            const uint64_t *p = in + (i * stride + 2 * y) * 2;
            ext2_t a = e2(p[0], p[1]), b = e2(p[2], p[3]);
            ext2_t v = e2_add(a, e2_mul(r, e2_sub(b, a)));
            out[(i * stride + y) * 2] = v.c0;
            out[(i * stride + y) * 2 + 1] = v.c1;
        }
    }
}

/*
 * Whole protocol, zk-torch-3/src/sumcheck/cpu_ext2_prover.rs:21-113:
 *   new():   append_u64("num_var"), append_u64("num_poly")
 *   round:   append_ext2("round_message") for each of the d+1 evaluations,
 *            challenge_ext2("challenge"), fold on the low variable
 *   end:     final_eval = product of the d remaining values
 * Base-field inputs (`base_field` != 0: d tables of 2^num_var u64) are lifted
 * with c1 = 0 (goldilocks-cuda-rs/src/sumcheck_prover.rs:262).
 *
 * Outputs: round_msgs[num_var][d+1][2], challenges[num_var][2],
 * final_evals[d][2], final_eval[2]. Returns 0, or -1 on bad arguments.
 */
int oracle_gl_sumcheck_prove(const uint64_t *polys_in, int d, int num_var, int base_field,
                             const uint8_t *label, size_t label_len,
                             uint64_t *round_msgs, uint64_t *challenges,
                             uint64_t *final_evals, uint64_t *final_eval,
                             uint64_t *transcript_state_out /* 8, may be NULL */) {
    if (d < 1 || d > MAX_D || num_var < 0 || num_var > 40) return -1;
    size_t n = (size_t)1 << num_var;
    uint64_t *cur = (uint64_t *)malloc(sizeof(uint64_t) * 2 * n * d);
    uint64_t *nxt = (uint64_t *)malloc(sizeof(uint64_t) * 2 * n * d);
    if (!cur || !nxt) { free(cur); free(nxt); return -1; }
    if (base_field) {
        for (int i = 0; i < d; i++)
            for (size_t k = 0; k < n; k++) {
                cur[(i * n + k) * 2] = gl_canon(polys_in[i * n + k]);
                cur[(i * n + k) * 2 + 1] = 0;
            }
    } else {
        for (size_t k = 0; k < 2 * n * d; k++) cur[k] = gl_canon(polys_in[k]);
    }

    gl_transcript_t t;
    gl_transcript_new(&t, label, label_len);
    gl_transcript_append_u64(&t, "num_var", (uint64_t)num_var);
    gl_transcript_append_u64(&t, "num_poly", (uint64_t)d);

    size_t size = n;
    for (int round = 0; round < num_var; round++) {
        size_t half = size / 2;
        uint64_t *msg = round_msgs + (size_t)round * (d + 1) * 2;
        oracle_gl_round_message_ext2(cur, d, n, half, msg);
        for (int c = 0; c <= d; c++)
            gl_transcript_append_ext2(&t, "round_message", e2(msg[2 * c], msg[2 * c + 1]));
        ext2_t r = gl_transcript_challenge_ext2(&t, "challenge");
        challenges[2 * round] = r.c0;
        challenges[2 * round + 1] = r.c1;
        oracle_gl_fold_ext2(cur, nxt, r.c0, r.c1, d, n, half);
        uint64_t *tmp = cur; cur = nxt; nxt = tmp;
        size = half;
    }
    ext2_t fe = e2(1, 0);
    for (int i = 0; i < d; i++) {
        ext2_t v = e2(cur[(size_t)i * n * 2], cur[(size_t)i * n * 2 + 1]);
        final_evals[2 * i] = v.c0;
        final_evals[2 * i + 1] = v.c1;
        fe = e2_mul(fe, v);
    }
    final_eval[0] = fe.c0;
    final_eval[1] = fe.c1;
    if (transcript_state_out) memcpy(transcript_state_out, t.sponge, 64);
    free(cur);
    free(nxt);
    return 0;
}

/*
 * Verifier side of the same protocol, used to cross-check the prover
 * structurally (zk-torch-3/src/sumcheck/verifier.rs): P_round(0) + P_round(1)
 * must equal the running claim; the next claim is P_round(r) by Lagrange
 * interpolation on the points 0..d. Returns 0 when every round is consistent
 * and the last claim equals final_eval.
 */
int oracle_gl_sumcheck_verify(int d, int num_var, const uint8_t *label, size_t label_len,
                              const uint64_t *claim_in, const uint64_t *round_msgs,
                              const uint64_t *final_eval) {
    gl_transcript_t t;
    gl_transcript_new(&t, label, label_len);
    gl_transcript_append_u64(&t, "num_var", (uint64_t)num_var);
    gl_transcript_append_u64(&t, "num_poly", (uint64_t)d);
    ext2_t claim = e2(claim_in[0], claim_in[1]);
    for (int round = 0; round < num_var; round++) {
        const uint64_t *msg = round_msgs + (size_t)round * (d + 1) * 2;
        ext2_t p0 = e2(msg[0], msg[1]), p1 = e2(msg[2], msg[3]);
        ext2_t s = e2_add(p0, p1);
        if (s.c0 != claim.c0 || s.c1 != claim.c1) return -(round + 1);
        for (int c = 0; c <= d; c++)
            gl_transcript_append_ext2(&t, "round_message", e2(msg[2 * c], msg[2 * c + 1]));
        ext2_t r = gl_transcript_challenge_ext2(&t, "challenge");
        /* Lagrange: sum_c P(c) * prod_{k != c} (r - k) / (c - k) */
        ext2_t next = e2(0, 0);
        for (int c = 0; c <= d; c++) {
            ext2_t num = e2(1, 0);
            uint64_t den = 1;
            for (int k = 0; k <= d; k++) {
                if (k == c) continue;
                num = e2_mul(num, e2_sub(r, e2((uint64_t)k, 0)));
                den = gl_mul(den, gl_sub((uint64_t)c, (uint64_t)k));
            }
            ext2_t term = e2_mul(e2(msg[2 * c], msg[2 * c + 1]), e2_mul_base(num, gl_inv(den)));
            next = e2_add(next, term);
        }
        claim = next;
    }
    return (claim.c0 == final_eval[0] && claim.c1 == final_eval[1]) ? 0 : -1000;
}

/* Partial evaluation over Goldilocks (cuda/partial_eval.cuh:31-93): fix the m low variables. */
void oracle_gl_partial_eval(const uint64_t *in, uint64_t *out, const uint64_t *r, int log_n, int m) {
    size_t n = (size_t)1 << log_n;
    uint64_t *cur = (uint64_t *)malloc(sizeof(uint64_t) * n);
    for (size_t i = 0; i < n; i++) cur[i] = gl_canon(in[i]);
    for (int i = 0; i < m; i++) {
        n /= 2;
        uint64_t ri = gl_canon(r[i]);
        for (size_t y = 0; y < n; y++) cur[y] = gl_add(cur[2 * y], gl_mul(ri, gl_sub(cur[2 * y + 1], cur[2 * y])));
    }
    memcpy(out, cur, sizeof(uint64_t) * n);
    free(cur);
}
void oracle_gl_partial_eval_ext2_from_base(const uint64_t *in, uint64_t *out, const uint64_t *r, int log_n, int m) {
    size_t n = (size_t)1 << log_n;
    ext2_t *cur = (ext2_t *)malloc(sizeof(ext2_t) * n);
    for (size_t i = 0; i < n; i++) cur[i] = e2(gl_canon(in[i]), 0);
    for (int i = 0; i < m; i++) {
        n /= 2;
        ext2_t ri = e2(gl_canon(r[2 * i]), gl_canon(r[2 * i + 1]));
        for (size_t y = 0; y < n; y++) cur[y] = e2_add(cur[2 * y], e2_mul(ri, e2_sub(cur[2 * y + 1], cur[2 * y])));
    }
    for (size_t y = 0; y < n; y++) { out[2 * y] = cur[y].c0; out[2 * y + 1] = cur[y].c1; }
    free(cur);
}
