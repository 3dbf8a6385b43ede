/* CPU ORACLE (test infrastructure, never shipped or timed as the product): the packed link
 * sumcheck over F_q[X]/(X^2 - 3), q = 2^64 - 2^32 - 31.
 *
 * Per round, with R(u) = u^3 - u and the HIGH index bit bound first (pairs (idx, half + idx)):
 *   S(k) = sum_e tag_e sum_idx eq[idx] R(w_e(k)[idx])      k = 0..3
 *   E(k) = sum_e       sum_idx omega_e(k)[idx] w_e(k)[idx]  k = 0..2
 * where w(k) = w_lo + k (w_hi - w_lo); in the first round k = 0, 1 of S are taken as zero
 * (committed coefficients lie in {-1, 0, 1}).          zk-torch-4/src/pcs/link.rs:284-346
 * fold: t[i] = lo + r (hi - lo)                         zk-torch-4/src/pcs/link.rs:349-357
 * eq table, most significant variable first            zk-torch-4/src/pcs/link.rs:199-213
 * Layouts of the device forms (bit-packed witnesses, support lists, interleaved blocks with
 * weights evaluated on demand): cuda_almost_goldilocks/link_sumcheck.cuh:59-787.
 *
 * The reference holds no golden value for these messages (its tests compare CPU and GPU
 * provers and run the verifier): parity unpinned beyond this restatement; the tests also
 * check the dense, listed, bit-packed and interleaved forms against one another.
 */
#include "agl.h"
#include <string.h>

static aext2_t ld(const uint64_t* p, uint64_t i) { return ae2(agl_canon(p[2 * i]), agl_canon(p[2 * i + 1])); }
static void st(uint64_t* p, uint64_t i, aext2_t v) { p[2 * i] = v.c0; p[2 * i + 1] = v.c1; }
static aext2_t range_poly(aext2_t u) { return ae2_sub(ae2_mul(ae2_mul(u, u), u), u); }
static aext2_t bit_at(const uint64_t* bits, uint64_t i) { return ae2((bits[i >> 6] >> (i & 63)) & 1, 0); }

/* one pair's contribution to the seven slots */
static void pair_terms(aext2_t acc[7], aext2_t w_lo, aext2_t w_hi, aext2_t o_lo, aext2_t o_hi, aext2_t eqs, int first_round) {
    aext2_t w_d = ae2_sub(w_hi, w_lo), o_d = ae2_sub(o_hi, o_lo);
    aext2_t w[4], o[3];
    w[0] = w_lo;
    for (int k = 1; k < 4; k++) w[k] = ae2_add(w[k - 1], w_d);
    o[0] = o_lo;
    for (int k = 1; k < 3; k++) o[k] = ae2_add(o[k - 1], o_d);
    for (int k = first_round ? 2 : 0; k < 4; k++) acc[k] = ae2_add(acc[k], ae2_mul(eqs, range_poly(w[k])));
    for (int k = 0; k < 3; k++) acc[4 + k] = ae2_add(acc[4 + k], ae2_mul(o[k], w[k]));
}

static void add_commit(aext2_t total[7], const aext2_t acc[7], aext2_t tag) {
    for (int k = 0; k < 7; k++) total[k] = ae2_add(total[k], k < 4 ? ae2_mul(tag, acc[k]) : acc[k]);
}

static aext2_t eq_pointwise(const uint64_t* pt, uint64_t l, int m) {
    aext2_t acc = ae2(1, 0);
    for (int k = 0; k < m; k++) {
        aext2_t r = ld(pt, k);
        acc = ae2_mul(acc, ((l >> (m - 1 - k)) & 1) ? r : ae2_sub(ae2(1, 0), r));
    }
    return acc;
}

/* The general round message. Witness: `bits` (n_commit rows of bits_stride_words words) when non-null, else
 * `w` (rows of w_stride elements). Index set: `list` slices (list_off, list_len) when non-null (eq indexed by
 * list position), else 0..half (eq indexed by idx). Weights: `omega` (rows of omega_stride) when non-null,
 * else scale[e][b] * eq(remaining leaf index, pts[e][b][round..]) with b = idx & block_mask. */
void oracle_link_round(const uint64_t* bits, const uint64_t* w, const uint64_t* omega, const uint64_t* pts, const uint64_t* scale,
                       const uint64_t* eq, const uint64_t* tags, const uint32_t* list, const uint64_t* list_off,
                       const uint64_t* list_len, uint64_t w_stride, uint64_t bits_stride_words, uint64_t omega_stride,
                       uint64_t half, uint64_t n_commit, uint32_t block_mask, int block_bits, int leaf_arity, int round,
                       int first_round, uint64_t* out) {
    aext2_t total[7];
    for (int k = 0; k < 7; k++) total[k] = ae2(0, 0);
    for (uint64_t e = 0; e < n_commit; e++) {
        aext2_t acc[7];
        for (int k = 0; k < 7; k++) acc[k] = ae2(0, 0);
        const uint64_t n = list ? list_len[e] : half;
        for (uint64_t t = 0; t < n; t++) {
            const uint64_t idx = list ? list[list_off[e] + t] : t;
            aext2_t w_lo, w_hi, o_lo, o_hi;
            if (bits) {
                w_lo = bit_at(bits + e * bits_stride_words, idx);
                w_hi = bit_at(bits + e * bits_stride_words, half + idx);
            } else {
                w_lo = ld(w + 2 * e * w_stride, idx);
                w_hi = ld(w + 2 * e * w_stride, half + idx);
            }
            if (omega) {
                o_lo = ld(omega + 2 * e * omega_stride, idx);
                o_hi = ld(omega + 2 * e * omega_stride, half + idx);
            } else {
                const uint64_t blocks = (uint64_t)block_mask + 1, b = idx & block_mask;
                const uint64_t* ptb = pts + 2 * ((e * blocks + b) * (uint64_t)leaf_arity + (uint64_t)round);
                const aext2_t sc = ld(scale, e * blocks + b);
                const int m = leaf_arity - round;
                o_lo = ae2_mul(sc, eq_pointwise(ptb, idx >> block_bits, m));
                o_hi = ae2_mul(sc, eq_pointwise(ptb, (half + idx) >> block_bits, m));
            }
            const aext2_t eqs = ld(eq, list ? list_off[e] + t : idx);
            pair_terms(acc, w_lo, w_hi, o_lo, o_hi, eqs, first_round);
        }
        add_commit(total, acc, ld(tags, e));
    }
    for (int k = 0; k < 7; k++) st(out, k, total[k]);
}

/* t[i] = lo + r (hi - lo) on rows of `stride`, in place, for i in the index set. */
void oracle_link_fold_rows(uint64_t* tab, uint64_t stride, uint64_t half, uint64_t n_commit, const uint32_t* list,
                           const uint64_t* list_off, const uint64_t* list_len, uint64_t r0, uint64_t r1) {
    const aext2_t r = ae2(agl_canon(r0), agl_canon(r1));
    for (uint64_t e = 0; e < n_commit; e++) {
        const uint64_t n = list ? list_len[e] : half;
        for (uint64_t t = 0; t < n; t++) {
            const uint64_t i = list ? list[list_off[e] + t] : t;
            const aext2_t lo = ld(tab + 2 * e * stride, i), hi = ld(tab + 2 * e * stride, half + i);
            st(tab + 2 * e * stride, i, ae2_add(lo, ae2_mul(r, ae2_sub(hi, lo))));
        }
    }
}

/* out[e][i] = lo + r (hi - lo) from bits (when non-null) or from w_in rows, into rows of out_stride. */
void oracle_link_fold_w(const uint64_t* bits, const uint64_t* w_in, uint64_t* w_out, uint64_t in_stride, uint64_t bits_stride_words,
                        uint64_t out_stride, uint64_t half, uint64_t n_commit, uint64_t r0, uint64_t r1) {
    const aext2_t r = ae2(agl_canon(r0), agl_canon(r1));
    for (uint64_t e = 0; e < n_commit; e++)
        for (uint64_t i = 0; i < half; i++) {
            aext2_t lo, hi;
            if (bits) {
                lo = bit_at(bits + e * bits_stride_words, i);
                hi = bit_at(bits + e * bits_stride_words, half + i);
            } else {
                lo = ld(w_in + 2 * e * in_stride, i);
                hi = ld(w_in + 2 * e * in_stride, half + i);
            }
            st(w_out + 2 * e * out_stride, i, ae2_add(lo, ae2_mul(r, ae2_sub(hi, lo))));
        }
}

/* One expansion step of an eq table built most-significant variable first: [0, span) -> [0, 2 span). */
void oracle_link_eq_expand(uint64_t* table, uint64_t span, uint64_t r0, uint64_t r1) {
    const aext2_t r = ae2(agl_canon(r0), agl_canon(r1)), om = ae2_sub(ae2(1, 0), r);
    for (uint64_t i = 0; i < span; i++) {
        const aext2_t v = ld(table, i);
        st(table, i, ae2_mul(v, om));
        st(table, span + i, ae2_mul(v, r));
    }
}

void oracle_link_expand_bits(const uint64_t* bits, uint64_t* out, uint64_t n_words) {
    for (uint64_t i = 0; i < n_words * 64; i++) st(out, i, bit_at(bits, i));
}

/* out[t] = eq(list[t], alpha), alpha most significant variable first. */
void oracle_link_eq_gather(const uint64_t* alpha, uint64_t n_vars, const uint32_t* list, uint64_t* out, uint64_t total) {
    for (uint64_t t = 0; t < total; t++) st(out, t, eq_pointwise(alpha, list[t], (int)n_vars));
}
