/*
 * CPU oracle (test infrastructure, not the product): batched degree-3 sumcheck
 * with a shared eq table over Goldilocks,
 *   S = sum_k alpha^k sum_x eq(t, x) a_k(x) b_k(x).
 *
 * The reference has no single function for this composition ("parity
 * unpinned"); it is assembled from pieces that are pinned separately: the
 * alpha-power combination and label scheme of prove_same_point
 * (zk-torch-4/src/fold/same_point_sumcheck.rs:58-157), the three-table linear
 * prover (zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100, low variable
 * first, evaluations at c = 0..3), the Goldilocks transcript
 * (zk-torch-3/src/transcript.rs:174-350) and the eq table
 * (zk-torch-3/src/poly/mod.rs:136-163).
 */
#include "gl.h"
#include <stdlib.h>
#include <string.h>

void oracle_gl_eq_ext2(const uint64_t *point, int nv, uint64_t *out);

/* m(c), c = 0..3, for extension tables: eq[len], ab[K][2][stride] (a_k then b_k), live length 2*half */
void oracle_gl_batched_message(const uint64_t *eq, const uint64_t *ab, const uint64_t *alpha_pows, int K, size_t stride,
                               size_t half, uint64_t *out8) {
    ext2_t m[4] = { e2(0, 0), e2(0, 0), e2(0, 0), e2(0, 0) };
#pragma omp parallel
    {
        ext2_t loc[4] = { e2(0, 0), e2(0, 0), e2(0, 0), e2(0, 0) };
#pragma omp for schedule(static) nowait
        for (size_t y = 0; y < half; y++) {
            ext2_t e0 = e2(eq[4 * y], eq[4 * y + 1]), e1 = e2(eq[4 * y + 2], eq[4 * y + 3]);
            ext2_t de = e2_sub(e1, e0);
            for (int k = 0; k < K; k++) {
                const uint64_t *pa = ab + ((size_t)(2 * k) * stride + 2 * y) * 2;
                const uint64_t *pb = ab + ((size_t)(2 * k + 1) * stride + 2 * y) * 2;
                ext2_t a0 = e2(pa[0], pa[1]), a1 = e2(pa[2], pa[3]), b0 = e2(pb[0], pb[1]), b1 = e2(pb[2], pb[3]);
                ext2_t da = e2_sub(a1, a0), db = e2_sub(b1, b0), w = e2(alpha_pows[2 * k], alpha_pows[2 * k + 1]);
                ext2_t va = a0, vb = b0, ve = e0;
                for (int c = 0; c < 4; c++) {
                    loc[c] = e2_add(loc[c], e2_mul(w, e2_mul(ve, e2_mul(va, vb))));
                    va = e2_add(va, da); vb = e2_add(vb, db); ve = e2_add(ve, de);
                }
            }
        }
#pragma omp critical
        for (int c = 0; c < 4; c++) m[c] = e2_add(m[c], loc[c]);
    }
    for (int c = 0; c < 4; c++) { out8[2 * c] = m[c].c0; out8[2 * c + 1] = m[c].c1; }
}

/* fold eq and every a_k, b_k on r, in place (results at the start of each table) */
void oracle_gl_batched_fold(uint64_t *eq, uint64_t *ab, uint64_t r0, uint64_t r1, int K, size_t stride, size_t half) {
    ext2_t r = e2(r0, r1);
    for (int t = -1; t < 2 * K; t++) {
        uint64_t *p = t < 0 ? eq : ab + (size_t)t * stride * 2;
        for (size_t y = 0; y < half; y++) {
            ext2_t lo = e2(p[4 * y], p[4 * y + 1]), hi = e2(p[4 * y + 2], p[4 * y + 3]);
            ext2_t v = e2_add(lo, e2_mul(r, e2_sub(hi, lo)));
            p[2 * y] = v.c0; p[2 * y + 1] = v.c1;
        }
    }
}

/* s_k = sum_x eq(x) a_k(x) b_k(x) over `size` live elements */
void oracle_gl_batched_claims(const uint64_t *eq, const uint64_t *ab, int K, size_t stride, size_t size, uint64_t *out) {
    for (int k = 0; k < K; k++) {
        ext2_t s = e2(0, 0);
        for (size_t x = 0; x < size; x++) {
            const uint64_t *pa = ab + ((size_t)(2 * k) * stride + x) * 2, *pb = ab + ((size_t)(2 * k + 1) * stride + x) * 2;
            s = e2_add(s, e2_mul(e2(eq[2 * x], eq[2 * x + 1]), e2_mul(e2(pa[0], pa[1]), e2(pb[0], pb[1]))));
        }
        out[2 * k] = s.c0; out[2 * k + 1] = s.c1;
    }
}

/*
 * Whole protocol. a, b: [K][2^nv] base field; point: nv extension coordinates.
 * Transcript (label scheme of prove_same_point): new(label); sp_num_var;
 * sp_num_inst; sp_y_i per claim; alpha = challenge(sp_alpha); per round the four
 * evaluations under sp_round_msg and challenge(sp_round_challenge); at the end
 * sp_f_eval for eq(R), then a_k(R), then b_k(R).
 * Outputs: claims[K][2], alpha[2], round_msgs[nv][4][2], challenges[nv][2],
 * finals[(2K+1)][2] = eq(R), a_k(R)..., b_k(R)..., final_eval[2], state[8].
 */
int oracle_gl_batched_prove(const uint64_t *a, const uint64_t *b, const uint64_t *point, int K, int nv,
                            const uint8_t *label, size_t label_len, uint64_t *claims, uint64_t *alpha_out,
                            uint64_t *round_msgs, uint64_t *challenges, uint64_t *finals, uint64_t *final_eval,
                            uint64_t *state_out) {
    if (K < 1 || nv < 1 || nv > 30) return -1;
    size_t n = (size_t)1 << nv;
    uint64_t *eq = (uint64_t *)malloc(16 * n), *ab = (uint64_t *)malloc(16 * n * 2 * K);
    uint64_t *pows = (uint64_t *)malloc(16 * (size_t)K);
    if (!eq || !ab || !pows) { free(eq); free(ab); free(pows); return -1; }
    oracle_gl_eq_ext2(point, nv, eq);
    for (int k = 0; k < K; k++)
        for (size_t x = 0; x < n; x++) {
            ab[((size_t)(2 * k) * n + x) * 2] = gl_canon(a[(size_t)k * n + x]); ab[((size_t)(2 * k) * n + x) * 2 + 1] = 0;
            ab[((size_t)(2 * k + 1) * n + x) * 2] = gl_canon(b[(size_t)k * n + x]); ab[((size_t)(2 * k + 1) * n + x) * 2 + 1] = 0;
        }
    gl_transcript_t t;
    gl_transcript_new(&t, label, label_len);
    gl_transcript_append_u64(&t, "sp_num_var", (uint64_t)nv);
    gl_transcript_append_u64(&t, "sp_num_inst", (uint64_t)K);
    oracle_gl_batched_claims(eq, ab, K, n, n, claims);
    for (int k = 0; k < K; k++) gl_transcript_append_ext2(&t, "sp_y_i", e2(claims[2 * k], claims[2 * k + 1]));
    ext2_t alpha = gl_transcript_challenge_ext2(&t, "sp_alpha");
    alpha_out[0] = alpha.c0; alpha_out[1] = alpha.c1;
    ext2_t p = e2(1, 0);
    for (int k = 0; k < K; k++) { pows[2 * k] = p.c0; pows[2 * k + 1] = p.c1; p = e2_mul(p, alpha); }
    size_t size = n;
    for (int round = 0; round < nv; round++) {
        size_t half = size / 2;
        uint64_t *msg = round_msgs + (size_t)round * 8;
        oracle_gl_batched_message(eq, ab, pows, K, n, half, msg);
        for (int c = 0; c < 4; c++) gl_transcript_append_ext2(&t, "sp_round_msg", e2(msg[2 * c], msg[2 * c + 1]));
        ext2_t r = gl_transcript_challenge_ext2(&t, "sp_round_challenge");
        challenges[2 * round] = r.c0; challenges[2 * round + 1] = r.c1;
        oracle_gl_batched_fold(eq, ab, r.c0, r.c1, K, n, half);
        size = half;
    }
    finals[0] = eq[0]; finals[1] = eq[1];
    ext2_t acc = e2(0, 0);
    for (int k = 0; k < K; k++) {
        const uint64_t *pa = ab + (size_t)(2 * k) * n * 2, *pb = ab + (size_t)(2 * k + 1) * n * 2;
        finals[2 + 2 * k] = pa[0]; finals[2 + 2 * k + 1] = pa[1];
        finals[2 + 2 * (K + k)] = pb[0]; finals[2 + 2 * (K + k) + 1] = pb[1];
        acc = e2_add(acc, e2_mul(e2(pows[2 * k], pows[2 * k + 1]), e2_mul(e2(pa[0], pa[1]), e2(pb[0], pb[1]))));
    }
    for (int i = 0; i < 2 * K + 1; i++) gl_transcript_append_ext2(&t, "sp_f_eval", e2(finals[2 * i], finals[2 * i + 1]));
    ext2_t fe = e2_mul(e2(eq[0], eq[1]), acc);
    final_eval[0] = fe.c0; final_eval[1] = fe.c1;
    if (state_out) memcpy(state_out, t.sponge, 64);
    free(eq); free(ab); free(pows);
    return 0;
}
