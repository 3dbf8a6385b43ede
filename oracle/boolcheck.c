/* CPU ORACLE (test infrastructure, never shipped or timed as the product): the sparse boolean-check
 * sumcheck  sum_t w_t sum_x eq(x) v_t(x) (v_t(x) - 1)  over sorted (position, value) lists, one slice of
 * the entry arrays per term; a round binds the LOW position bit.
 * Restates almost-goldilocks-cuda-rs/cuda/wrapper.cu:2690-2825 (mark, message, fold, new offsets, finish);
 * the reference pins no value for it (parity unpinned beyond this restatement; the tests check the
 * sumcheck identities the messages must satisfy). */
#include "agl.h"
#include <string.h>

static aext2_t ld(const uint64_t* p, uint64_t i) { return ae2(agl_canon(p[2 * i]), agl_canon(p[2 * i + 1])); }
static void st(uint64_t* p, uint64_t i, aext2_t v) { p[2 * i] = v.c0; p[2 * i + 1] = v.c1; }

static void group_values(const uint32_t* idx, const uint64_t* val, uint32_t i, uint32_t e, aext2_t* v0, aext2_t* v1) {
    const uint32_t pos = idx[i], rest = pos >> 1;
    *v0 = ae2(0, 0);
    *v1 = ae2(0, 0);
    if ((pos & 1u) == 0u) {
        *v0 = ld(val, i);
        if (i + 1 < e && idx[i + 1] == 2u * rest + 1u) *v1 = ld(val, i + 1);
    } else {
        *v1 = ld(val, i);
    }
}

/* flags, gid (n entries each), msg (8 words); returns the number of groups. */
uint32_t oracle_bool_round(const uint32_t* idx, const uint64_t* val, const uint32_t* term_off, const uint64_t* w, const uint64_t* eq,
                           int n_terms, uint32_t n, uint32_t* flags, uint32_t* gid, uint64_t* msg) {
    aext2_t acc[4];
    for (int k = 0; k < 4; k++) acc[k] = ae2(0, 0);
    memset(flags, 0, sizeof(uint32_t) * n);
    for (int t = 0; t < n_terms; t++) {
        const uint32_t s = term_off[t], e = term_off[t + 1];
        const aext2_t wt = ld(w, t), one = ae2(1, 0);
        for (uint32_t i = s; i < e; i++) {
            flags[i] = (i == s) ? 1u : (((idx[i] & 1u) && idx[i - 1] == idx[i] - 1u) ? 0u : 1u);
            if (!flags[i]) continue;
            aext2_t v0, v1;
            group_values(idx, val, i, e, &v0, &v1);
            const uint32_t rest = idx[i] >> 1;
            const aext2_t e0 = ld(eq, 2 * (uint64_t)rest), e1 = ld(eq, 2 * (uint64_t)rest + 1);
            const aext2_t vd = ae2_sub(v1, v0), ed = ae2_sub(e1, e0);
            aext2_t a = v0, ec = e0;
            for (int c = 0; c < 4; c++) {
                acc[c] = ae2_add(acc[c], ae2_mul(ae2_mul(wt, ae2_mul(a, ae2_sub(a, one))), ec));
                a = ae2_add(a, vd);
                ec = ae2_add(ec, ed);
            }
        }
    }
    uint32_t run = 0;
    for (uint32_t i = 0; i < n; i++) {
        gid[i] = run;
        run += flags[i];
    }
    for (int k = 0; k < 4; k++) st(msg, k, acc[k]);
    return run;
}

void oracle_bool_fold(const uint32_t* idx, const uint64_t* val, const uint32_t* flags, const uint32_t* gid, const uint32_t* term_off,
                      int n_terms, uint32_t n, uint64_t r0, uint64_t r1, uint32_t total, uint32_t* out_idx, uint64_t* out_val,
                      uint32_t* new_off) {
    const aext2_t ch = ae2(agl_canon(r0), agl_canon(r1));
    for (int t = 0; t < n_terms; t++) {
        const uint32_t s = term_off[t], e = term_off[t + 1];
        for (uint32_t i = s; i < e; i++) {
            if (!flags[i]) continue;
            aext2_t v0, v1;
            group_values(idx, val, i, e, &v0, &v1);
            out_idx[gid[i]] = idx[i] >> 1;
            st(out_val, gid[i], ae2_add(v0, ae2_mul(ch, ae2_sub(v1, v0))));
        }
    }
    for (int t = 0; t <= n_terms; t++) new_off[t] = (t == n_terms || term_off[t] >= n) ? total : gid[term_off[t]];
}
