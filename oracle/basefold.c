/*
 * CPU oracle (test infrastructure, not the product): Basefold commit, opening
 * proof and verifier over Goldilocks with Poseidon2 Merkle trees.
 *
 * Restates:
 *   folding table        goldilocks-cuda-rs/src/basefold.rs:281-321
 *   commit (host spec)   cuda/basefold_kernels.cu:58-129,
 *                        goldilocks-cuda-rs/cuda/wrapper.cu:1242-1312,
 *                        cuda/basefold.cuh:57-205 (layer definitions)
 *   Merkle tree layout   goldilocks-cuda-rs/src/merkle.rs:145-159,266-280
 *   CPU opening          zk-torch-3/src/commit/cpu_basefold.rs:22-425
 *   verifier             goldilocks-cuda-rs/src/basefold.rs:1759-1925
 *   eq table             zk-torch-3/src/poly/mod.rs:136-163
 *
 * The reference pins no root or proof value for this path (its tests compare
 * CPU with GPU). Parity of this file is therefore anchored on: the Poseidon2
 * vectors produced by the reference's own code, the prover->verifier round
 * trip with tamper rejection, and structural properties checked in tests.
 */
#include "gl.h"
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* Proof wire layout shared by the oracle and the library              */
/* ------------------------------------------------------------------ */
/*
 *   eval                 2
 *   sumcheck oracles     nv * 6        (c0, c1, c2; extension elements)
 *   folded roots         (nv-1) * 4
 *   final codeword       2^lr * 2
 *   per query:           1             leaf index
 *                        nv * 4        value pairs (round 0 pair lifted with c1 = 0)
 *                        4 * (nv+lr-1) path in the commitment tree
 *                        4 * sum_{i=0}^{nv-2} (nv+lr-2-i)   paths in the folded trees
 */
size_t oracle_bf_query_words(int nv, int lr) {
    size_t w = 1 + (size_t)nv * 4 + 4 * (size_t)(nv + lr - 1);
    for (int i = 0; i <= nv - 2; i++) w += 4 * (size_t)(nv + lr - 2 - i);
    return w;
}
size_t oracle_bf_proof_words(int nv, int lr, int nq) {
    return 2 + (size_t)nv * 6 + (size_t)(nv - 1) * 4 + ((size_t)2 << lr) + (size_t)nq * oracle_bf_query_words(nv, lr);
}

/* ------------------------------------------------------------------ */
/* Folding table: basefold.rs:281-321                                   */
/* ------------------------------------------------------------------ */
size_t oracle_bf_table_entries(int nv, int lr, int num_rounds) {
    size_t t = 0;
    for (int i = 0; i < num_rounds; i++) t += (size_t)1 << (nv + lr - i - 1);
    return t;
}

/* entries_out: (point, weight) pairs, levels back to back. The xorshift
 * stream is sequential; the inversions (one per entry in the reference) are
 * done afterwards in parallel and give the same residues. */
void oracle_bf_table_generate(int nv, int lr, int num_rounds, uint64_t seed, uint64_t *entries_out) {
    uint64_t s = seed;
    size_t total = oracle_bf_table_entries(nv, lr, num_rounds);
    for (size_t k = 0; k < total; k++) {
        uint64_t x0, x1;
        s ^= s << 13; s ^= s >> 7; s ^= s << 17; x0 = s % GL_P;
        s ^= s << 13; s ^= s >> 7; s ^= s << 17; x1 = s % GL_P;
        while (x1 == x0) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; x1 = s % GL_P; }
        entries_out[2 * k] = x0;
        entries_out[2 * k + 1] = gl_sub(x1, x0);
    }
#pragma omp parallel for schedule(static)
    for (size_t k = 0; k < total; k++) entries_out[2 * k + 1] = gl_inv(entries_out[2 * k + 1]);
}

/* ------------------------------------------------------------------ */
/* Commit                                                               */
/* ------------------------------------------------------------------ */
static size_t bit_reverse(size_t x, int bits) {
    size_t y = 0;
    for (int i = 0; i < bits; i++) { y = (y << 1) | (x & 1); x >>= 1; }
    return y;
}

static void bit_reverse_permute(uint64_t *data, int log_n, int words) {
    size_t n = (size_t)1 << log_n;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        size_t r = bit_reverse(i, log_n);
        if (i < r) {
            for (int w = 0; w < words; w++) {
                uint64_t t = data[i * words + w];
                data[i * words + w] = data[r * words + w];
                data[r * words + w] = t;
            }
        }
    }
}
void oracle_bf_bit_reverse_gl(uint64_t *data, int log_n) { bit_reverse_permute(data, log_n, 1); }
void oracle_bf_bit_reverse_ext2(uint64_t *data, int log_n) { bit_reverse_permute(data, log_n, 2); }

/* evals -> multilinear coefficients (in place layers) and the bit-reversed
 * copy of the evaluations: wrapper.cu:1242-1275. */
void oracle_bf_bhc_interpolate(const uint64_t *evals, uint64_t *coeffs, uint64_t *bh_evals, int nv) {
    size_t n = (size_t)1 << nv;
    for (size_t i = 0; i < n; i++) { coeffs[i] = gl_canon(evals[i]); bh_evals[i] = gl_canon(evals[i]); }
    for (int k = 0; k < nv; k++) {
        size_t half_chunk = (size_t)1 << k;
#pragma omp parallel for schedule(static)
        for (size_t idx = 0; idx < n / 2; idx++) {
            size_t base = (idx / half_chunk) * 2 * half_chunk, pos = idx % half_chunk;
            coeffs[base + half_chunk + pos] = gl_sub(coeffs[base + half_chunk + pos], coeffs[base + pos]);
        }
    }
    oracle_bf_bit_reverse_gl(bh_evals, nv);
}

/* coefficients -> codeword: repetition, nv butterfly layers, bit reversal:
 * wrapper.cu:1277-1312. */
void oracle_bf_encode(const uint64_t *coeffs, uint64_t *codeword, int nv, int lr) {
    size_t n_out = (size_t)1 << (nv + lr);
    for (size_t i = 0; i < n_out; i++) codeword[i] = coeffs[i >> lr];
    for (int i = 0; i < nv; i++) {
        size_t half_chunk = (size_t)1 << (i + lr);
#pragma omp parallel for schedule(static)
        for (size_t idx = 0; idx < n_out / 2; idx++) {
            size_t lo = (idx / half_chunk) * 2 * half_chunk + idx % half_chunk, hi = lo + half_chunk;
            uint64_t a = codeword[lo], b = codeword[hi];
            codeword[lo] = gl_add(a, b);
            codeword[hi] = gl_sub(a, b);
        }
    }
    oracle_bf_bit_reverse_gl(codeword, nv + lr);
}

/* Tree buffer: leaves, then each layer, root last; 4 words per digest
 * (merkle.rs:266-280). ext2 != 0: leaves hash two extension elements. */
void oracle_bf_merkle_tree(const uint64_t *codeword, size_t num_leaves, int ext2, uint64_t *tree) {
#pragma omp parallel for schedule(static)
    for (size_t k = 0; k < num_leaves; k++) {
        if (ext2) {
            const uint64_t *p = codeword + 4 * k;
            gl_hash_ext2_leaf(e2(p[0], p[1]), e2(p[2], p[3]), tree + 4 * k);
        } else {
            gl_hash_gl_leaf(codeword[2 * k], codeword[2 * k + 1], tree + 4 * k);
        }
    }
    uint64_t *prev = tree;
    size_t size = num_leaves;
    while (size > 1) {
        uint64_t *next = prev + 4 * size;
        size_t half = size / 2;
#pragma omp parallel for schedule(static)
        for (size_t k = 0; k < half; k++) gl_compress(prev + 8 * k, prev + 8 * k + 4, next + 4 * k);
        prev = next;
        size = half;
    }
}

static const uint64_t *tree_root(const uint64_t *tree, size_t num_leaves) { return tree + 4 * (2 * num_leaves - 2); }

/* sibling idx^1 per layer, bottom-up: merkle.rs:145-159 */
static size_t tree_auth_path(const uint64_t *tree, size_t num_leaves, size_t leaf, uint64_t *out) {
    const uint64_t *layer = tree;
    size_t size = num_leaves, idx = leaf, n = 0;
    while (size > 1) {
        memcpy(out + 4 * n, layer + 4 * (idx ^ 1), 32);
        n++;
        layer += 4 * size;
        size /= 2;
        idx /= 2;
    }
    return n;
}

/* codeword[2^(nv+lr)], bh_evals[2^nv] (bit-reversed evaluations), tree over the
 * codeword's pairs ((2^(nv+lr) - 1) digests): BasefoldCommitment::commit_device,
 * basefold.rs:382-414. */
void oracle_bf_commit(const uint64_t *evals, int nv, int lr, uint64_t *codeword, uint64_t *bh_evals, uint64_t *tree) {
    size_t n = (size_t)1 << nv;
    uint64_t *coeffs = (uint64_t *)malloc(sizeof(uint64_t) * n);
    oracle_bf_bhc_interpolate(evals, coeffs, bh_evals, nv);
    oracle_bf_encode(coeffs, codeword, nv, lr);
    free(coeffs);
    oracle_bf_merkle_tree(codeword, ((size_t)1 << (nv + lr)) / 2, 0, tree);
}

/* ------------------------------------------------------------------ */
/* Opening                                                              */
/* ------------------------------------------------------------------ */

/* eq(r, x), bit i of x <-> r[i]: poly/mod.rs:136-163 */
void oracle_gl_eq_ext2(const uint64_t *point, int nv, uint64_t *out /* 2^nv ext2 */) {
    size_t n = (size_t)1 << nv;
    memset(out, 0, sizeof(uint64_t) * 2 * n);
    out[0] = 1;
    for (int i = 0; i < nv; i++) {
        ext2_t ri = e2(point[2 * i], point[2 * i + 1]);
        ext2_t omr = e2_sub(e2(1, 0), ri);
        size_t half = (size_t)1 << i;
#pragma omp parallel for schedule(static)
        for (size_t j = 0; j < half; j++) {
            ext2_t v = e2(out[2 * j], out[2 * j + 1]);
            ext2_t hi = e2_mul(v, ri), lo = e2_mul(v, omr);
            out[2 * (j | half)] = hi.c0; out[2 * (j | half) + 1] = hi.c1;
            out[2 * j] = lo.c0; out[2 * j + 1] = lo.c1;
        }
    }
}

void oracle_gl_eq_base(const uint64_t *point, int nv, uint64_t *out /* 2^nv */) {
    size_t n = (size_t)1 << nv;
    memset(out, 0, sizeof(uint64_t) * n);
    out[0] = 1;
    for (int i = 0; i < nv; i++) {
        uint64_t ri = gl_canon(point[i]), omr = gl_sub(1, ri);
        size_t half = (size_t)1 << i;
        for (size_t j = 0; j < half; j++) {
            uint64_t v = out[j];
            out[j | half] = gl_mul(v, ri);
            out[j] = gl_mul(v, omr);
        }
    }
}

#define INV2 9223372034707292161ULL /* cpu_basefold.rs:157 */

/* cpu_basefold.rs:161-221; bh_words = 1 (base field) or 2 (extension). */
static void compute_oracle(const uint64_t *bh, int bh_words, const uint64_t *eq, size_t size, uint64_t *out6) {
    size_t half = size / 2;
    ext2_t p0 = e2(0, 0), p1 = e2(0, 0), p2 = e2(0, 0);
#pragma omp parallel
    {
        ext2_t l0 = e2(0, 0), l1 = e2(0, 0), l2 = e2(0, 0);
#pragma omp for schedule(static) nowait
        for (size_t j = 0; j < half; j++) {
            ext2_t b0, b1;
            if (bh_words == 1) { b0 = e2(bh[2 * j], 0); b1 = e2(bh[2 * j + 1], 0); }
            else { b0 = e2(bh[4 * j], bh[4 * j + 1]); b1 = e2(bh[4 * j + 2], bh[4 * j + 3]); }
            ext2_t q0 = e2(eq[4 * j], eq[4 * j + 1]), q1 = e2(eq[4 * j + 2], eq[4 * j + 3]);
            l0 = e2_add(l0, e2_mul(q0, b0));
            l1 = e2_add(l1, e2_mul(q1, b1));
            ext2_t qi = e2_sub(e2_add(q1, q1), q0), bi = e2_sub(e2_add(b1, b1), b0);
            l2 = e2_add(l2, e2_mul(qi, bi));
        }
#pragma omp critical
        { p0 = e2_add(p0, l0); p1 = e2_add(p1, l1); p2 = e2_add(p2, l2); }
    }
    ext2_t c0 = p0;
    ext2_t c2 = e2_mul_base(e2_add(e2_sub(p0, e2_add(p1, p1)), p2), INV2);
    ext2_t c1 = e2_sub(e2_sub(p1, p0), c2);
    out6[0] = c0.c0; out6[1] = c0.c1; out6[2] = c1.c0; out6[3] = c1.c1; out6[4] = c2.c0; out6[5] = c2.c1;
}

/* cpu_basefold.rs:87-131: v0 + (r - x0) * ((v1 - v0) * w) */
static void fold_codeword(const uint64_t *cw, int words, const uint64_t *entries, ext2_t r, size_t pairs, uint64_t *out) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < pairs; i++) {
        ext2_t v0, v1;
        if (words == 1) { v0 = e2(cw[2 * i], 0); v1 = e2(cw[2 * i + 1], 0); }
        else { v0 = e2(cw[4 * i], cw[4 * i + 1]); v1 = e2(cw[4 * i + 2], cw[4 * i + 3]); }
        uint64_t x0 = entries[2 * i], w = entries[2 * i + 1];
        ext2_t diff_w = e2_mul_base(e2_sub(v1, v0), w);
        ext2_t cx = e2_sub(r, e2(x0, 0));
        ext2_t res = e2_add(v0, e2_mul(cx, diff_w));
        out[2 * i] = res.c0;
        out[2 * i + 1] = res.c1;
    }
}

static void observe_hash(gl_transcript_t *t, const uint64_t *h) { for (int i = 0; i < 4; i++) gl_transcript_absorb(t, h[i]); }
static void observe_ext2(gl_transcript_t *t, uint64_t c0, uint64_t c1) { gl_transcript_absorb(t, c0); gl_transcript_absorb(t, c1); }
static ext2_t sample_ext2(gl_transcript_t *t) { uint64_t a = gl_transcript_squeeze(t); uint64_t b = gl_transcript_squeeze(t); return e2(a, b); }

/*
 * cpu_full_open_ext2 (cpu_basefold.rs:235-425). Inputs: the commitment
 * (codeword, bit-reversed evaluations, its tree), the point (nv extension
 * coordinates), the folding table, the transcript label. Writes the proof in
 * the wire layout above. Returns 0, -1 on bad arguments or allocation failure.
 */
int oracle_bf_open_ext2(const uint64_t *codeword, const uint64_t *bh_evals, const uint64_t *commit_tree, int nv, int lr,
                        const uint64_t *point, const uint64_t *table, const uint8_t *label, size_t label_len,
                        int num_queries, uint64_t *proof, uint64_t *transcript_state_out) {
    if (nv < 2 || lr < 0 || nv + lr > 40) return -1;
    size_t n = (size_t)1 << nv, cw_len = (size_t)1 << (nv + lr);
    uint64_t *p_eval = proof, *p_oracles = proof + 2, *p_roots = p_oracles + (size_t)nv * 6;
    uint64_t *p_final = p_roots + (size_t)(nv - 1) * 4, *p_queries = p_final + ((size_t)2 << lr);
    size_t qwords = oracle_bf_query_words(nv, lr);

    gl_transcript_t t;
    gl_transcript_new(&t, label, label_len);
    observe_hash(&t, tree_root(commit_tree, cw_len / 2));
    for (int i = 0; i < nv; i++) observe_ext2(&t, point[2 * i], point[2 * i + 1]);

    uint64_t *eq = (uint64_t *)malloc(sizeof(uint64_t) * 2 * n);
    uint64_t *bh = (uint64_t *)malloc(sizeof(uint64_t) * n);  /* round >= 1: n/2 extension elements */
    if (!eq || !bh) { free(eq); free(bh); return -1; }
    oracle_gl_eq_ext2(point, nv, eq);

    /* The commitment stores the evaluations bit-reversed; the opening reverses
     * them back before use (cpu_basefold.rs:252-259, basefold.rs:600-602). */
    uint64_t *bhv = (uint64_t *)malloc(sizeof(uint64_t) * n);
    if (!bhv) { free(eq); free(bh); return -1; }
    for (size_t i = 0; i < n; i++) bhv[i] = gl_canon(bh_evals[i]);
    oracle_bf_bit_reverse_gl(bhv, nv);
    bh_evals = bhv;

    /* eval = <bh, eq> */
    ext2_t eval = e2(0, 0);
#pragma omp parallel
    {
        ext2_t loc = e2(0, 0);
#pragma omp for schedule(static) nowait
        for (size_t i = 0; i < n; i++) loc = e2_add(loc, e2_mul_base(e2(eq[2 * i], eq[2 * i + 1]), bh_evals[i]));
#pragma omp critical
        eval = e2_add(eval, loc);
    }
    p_eval[0] = eval.c0; p_eval[1] = eval.c1;

    compute_oracle(bh_evals, 1, eq, n, p_oracles);
    for (int k = 0; k < 3; k++) observe_ext2(&t, p_oracles[2 * k], p_oracles[2 * k + 1]);

    ext2_t r = sample_ext2(&t);
    size_t sc = n / 2;
    uint64_t *eq2 = (uint64_t *)malloc(sizeof(uint64_t) * n);      /* ping-pong partners so the folds can run in parallel */
    uint64_t *bh2 = (uint64_t *)malloc(sizeof(uint64_t) * (n / 2 > 2 ? n / 2 : 2));
    if (!eq2 || !bh2) { free(eq); free(bh); free(bhv); free(eq2); free(bh2); return -1; }
#pragma omp parallel for schedule(static)
    for (size_t j = 0; j < sc; j++) {
        ext2_t lo = e2(bh_evals[2 * j], 0), hi = e2(bh_evals[2 * j + 1], 0);
        ext2_t v = e2_add(lo, e2_mul(r, e2_sub(hi, lo)));
        bh[2 * j] = v.c0; bh[2 * j + 1] = v.c1;
        ext2_t ql = e2(eq[4 * j], eq[4 * j + 1]), qh = e2(eq[4 * j + 2], eq[4 * j + 3]);
        ext2_t q = e2_add(ql, e2_mul(r, e2_sub(qh, ql)));
        eq2[2 * j] = q.c0; eq2[2 * j + 1] = q.c1;
    }
    { uint64_t *tmp = eq; eq = eq2; eq2 = tmp; }
    compute_oracle(bh, 2, eq, sc, p_oracles + 6);
    for (int k = 0; k < 3; k++) observe_ext2(&t, p_oracles[6 + 2 * k], p_oracles[6 + 2 * k + 1]);

    /* folded codewords and their trees, all kept for the query phase */
    uint64_t **fcw = (uint64_t **)calloc((size_t)nv, sizeof(uint64_t *));
    uint64_t **ftree = (uint64_t **)calloc((size_t)nv, sizeof(uint64_t *));
    size_t *flen = (size_t *)calloc((size_t)nv, sizeof(size_t));
    const uint64_t *level = table;
    size_t pairs = cw_len / 2;
    fcw[0] = (uint64_t *)malloc(sizeof(uint64_t) * 2 * pairs);
    fold_codeword(codeword, 1, level, r, pairs, fcw[0]);
    flen[0] = pairs;
    ftree[0] = (uint64_t *)malloc(sizeof(uint64_t) * 4 * (pairs - 1));
    oracle_bf_merkle_tree(fcw[0], pairs / 2, 1, ftree[0]);
    memcpy(p_roots, tree_root(ftree[0], pairs / 2), 32);
    observe_hash(&t, p_roots);
    level += 2 * pairs;

    for (int round = 1; round < nv - 1; round++) {
        r = sample_ext2(&t);
        size_t half = sc / 2;
#pragma omp parallel for schedule(static)
        for (size_t j = 0; j < half; j++) {
            ext2_t ql = e2(eq[4 * j], eq[4 * j + 1]), qh = e2(eq[4 * j + 2], eq[4 * j + 3]);
            ext2_t q = e2_add(ql, e2_mul(r, e2_sub(qh, ql)));
            ext2_t bl = e2(bh[4 * j], bh[4 * j + 1]), bhh = e2(bh[4 * j + 2], bh[4 * j + 3]);
            ext2_t b = e2_add(bl, e2_mul(r, e2_sub(bhh, bl)));
            eq2[2 * j] = q.c0; eq2[2 * j + 1] = q.c1;
            bh2[2 * j] = b.c0; bh2[2 * j + 1] = b.c1;
        }
        { uint64_t *tmp = eq; eq = eq2; eq2 = tmp; tmp = bh; bh = bh2; bh2 = tmp; }
        sc = half;
        uint64_t *po = p_oracles + (size_t)(round + 1) * 6;
        compute_oracle(bh, 2, eq, sc, po);
        for (int k = 0; k < 3; k++) observe_ext2(&t, po[2 * k], po[2 * k + 1]);

        size_t in_len = flen[round - 1];
        pairs = in_len / 2;
        fcw[round] = (uint64_t *)malloc(sizeof(uint64_t) * 2 * pairs);
        fold_codeword(fcw[round - 1], 2, level, r, pairs, fcw[round]);
        flen[round] = pairs;
        ftree[round] = (uint64_t *)malloc(sizeof(uint64_t) * 4 * (pairs > 1 ? pairs - 1 : 1));
        oracle_bf_merkle_tree(fcw[round], pairs / 2, 1, ftree[round]);
        memcpy(p_roots + 4 * round, tree_root(ftree[round], pairs / 2), 32);
        observe_hash(&t, p_roots + 4 * round);
        level += 2 * pairs;
    }

    r = sample_ext2(&t);
    {
        size_t in_len = flen[nv - 2];
        fold_codeword(fcw[nv - 2], 2, level, r, in_len / 2, p_final);
    }

    for (int q = 0; q < num_queries; q++) {
        uint64_t *pq = p_queries + (size_t)q * qwords;
        uint64_t raw = gl_transcript_squeeze(&t);
        size_t leaf = (size_t)(raw % (uint64_t)(cw_len / 2));
        *pq++ = leaf;
        uint64_t *vals = pq;
        pq += (size_t)nv * 4;
        vals[0] = codeword[2 * leaf]; vals[1] = 0; vals[2] = codeword[2 * leaf + 1]; vals[3] = 0;
        pq += 4 * tree_auth_path(commit_tree, cw_len / 2, leaf, pq);
        size_t idx = leaf / 2;
        for (int i = 0; i <= nv - 2; i++) {
            memcpy(vals + 4 * (i + 1), fcw[i] + 4 * idx, 32);
            pq += 4 * tree_auth_path(ftree[i], flen[i] / 2, idx, pq);
            idx /= 2;
        }
    }
    if (transcript_state_out) memcpy(transcript_state_out, t.sponge, 64);
    for (int i = 0; i < nv; i++) { free(fcw[i]); free(ftree[i]); }
    free(fcw); free(ftree); free(flen); free(eq); free(bh); free(bhv); free(eq2); free(bh2);
    return 0;
}

/* ------------------------------------------------------------------ */
/* Verifier: basefold.rs:1759-1925                                      */
/* ------------------------------------------------------------------ */
static int verify_path(const uint64_t *leaf_hash, const uint64_t *path, size_t path_len, size_t idx, const uint64_t *root) {
    uint64_t cur[4];
    memcpy(cur, leaf_hash, 32);
    for (size_t k = 0; k < path_len; k++) {
        uint64_t nxt[4];
        if ((idx & 1) == 0) gl_compress(cur, path + 4 * k, nxt);
        else gl_compress(path + 4 * k, cur, nxt);
        memcpy(cur, nxt, 32);
        idx >>= 1;
    }
    return memcmp(cur, root, 32) == 0;
}

static ext2_t oracle_at(const uint64_t *o, ext2_t x) {
    ext2_t c0 = e2(o[0], o[1]), c1 = e2(o[2], o[3]), c2 = e2(o[4], o[5]);
    return e2_add(c0, e2_add(e2_mul(c1, x), e2_mul(c2, e2_mul(x, x))));
}

/* Returns 0 if the proof verifies, a negative code naming the failed check
 * otherwise. */
int oracle_bf_verify_ext2(const uint64_t *root, int nv, int lr, const uint64_t *point, const uint64_t *table,
                          const uint8_t *label, size_t label_len, int num_queries, const uint64_t *proof) {
    const uint64_t *p_eval = proof, *p_oracles = proof + 2, *p_roots = p_oracles + (size_t)nv * 6;
    const uint64_t *p_final = p_roots + (size_t)(nv - 1) * 4, *p_queries = p_final + ((size_t)2 << lr);
    size_t qwords = oracle_bf_query_words(nv, lr);
    gl_transcript_t t;
    gl_transcript_new(&t, label, label_len);
    observe_hash(&t, root);
    for (int i = 0; i < nv; i++) observe_ext2(&t, point[2 * i], point[2 * i + 1]);

    ext2_t one = e2(1, 0), zero = e2(0, 0);
    ext2_t s = e2_add(oracle_at(p_oracles, zero), oracle_at(p_oracles, one));
    if (s.c0 != p_eval[0] || s.c1 != p_eval[1]) return -1;
    for (int k = 0; k < 3; k++) observe_ext2(&t, p_oracles[2 * k], p_oracles[2 * k + 1]);

    ext2_t *ch = (ext2_t *)malloc(sizeof(ext2_t) * nv);
    for (int round = 0; round < nv - 1; round++) {
        ch[round] = sample_ext2(&t);
        ext2_t v = oracle_at(p_oracles + 6 * round, ch[round]);
        const uint64_t *on = p_oracles + 6 * (round + 1);
        ext2_t ns = e2_add(oracle_at(on, zero), oracle_at(on, one));
        if (v.c0 != ns.c0 || v.c1 != ns.c1) { free(ch); return -(10 + round); }
        for (int k = 0; k < 3; k++) observe_ext2(&t, on[2 * k], on[2 * k + 1]);
        observe_hash(&t, p_roots + 4 * round);
    }
    ch[nv - 1] = sample_ext2(&t);

    size_t cw_len = (size_t)1 << (nv + lr);
    int rc = 0;
    for (int q = 0; q < num_queries && rc == 0; q++) {
        const uint64_t *pq = p_queries + (size_t)q * qwords;
        uint64_t raw = gl_transcript_squeeze(&t);
        size_t index = (size_t)*pq++;
        if (index != (size_t)(raw % (uint64_t)(cw_len / 2))) { rc = -100; break; }
        const uint64_t *vals = pq;
        pq += (size_t)nv * 4;
        uint64_t lh[4];
        gl_hash_gl_leaf(vals[0], vals[2], lh);
        size_t plen = (size_t)(nv + lr - 1);
        if (vals[1] != 0 || vals[3] != 0 || !verify_path(lh, pq, plen, index, root)) { rc = -101; break; }
        pq += 4 * plen;
        size_t fold_idx = index;
        const uint64_t *level = table;
        for (int r_i = 0; r_i < nv; r_i++) {
            const uint64_t *v = vals + 4 * r_i;
            ext2_t v0 = e2(v[0], v[1]), v1 = e2(v[2], v[3]);
            uint64_t x0 = level[2 * fold_idx], w = level[2 * fold_idx + 1];
            ext2_t cx = e2_sub(ch[r_i], e2(x0, 0));
            ext2_t res = e2_add(v0, e2_mul_base(e2_mul(cx, e2_sub(v1, v0)), w));
            if (r_i < nv - 1) {
                const uint64_t *nv_ = vals + 4 * (r_i + 1);
                const uint64_t *ex = (fold_idx & 1) == 0 ? nv_ : nv_ + 2;
                if (res.c0 != ex[0] || res.c1 != ex[1]) { rc = -(200 + r_i); break; }
                uint64_t nh[4];
                gl_hash_ext2_leaf(e2(nv_[0], nv_[1]), e2(nv_[2], nv_[3]), nh);
                size_t fl = (size_t)(nv + lr - 2 - r_i);
                if (!verify_path(nh, pq, fl, fold_idx / 2, p_roots + 4 * r_i)) { rc = -(300 + r_i); break; }
                pq += 4 * fl;
            } else {
                const uint64_t *ex = p_final + 2 * fold_idx;
                if (res.c0 != ex[0] || res.c1 != ex[1]) { rc = -400; break; }
            }
            level += 2 * ((size_t)1 << (nv + lr - r_i - 1));
            fold_idx /= 2;
        }
    }
    free(ch);
    return rc;
}
