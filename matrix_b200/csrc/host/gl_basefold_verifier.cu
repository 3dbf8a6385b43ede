// Basefold opening verifier on the host (the Rust verifier of the reference, goldilocks-cuda-rs/src/basefold.rs:
// 1759-1925, with the query checks of :2222-2402), over the proof layout this library's provers write
// (gl_basefold_common.cuh: eval | oracles | folded roots | final codeword | queries) and the same transcript.
//
// Everything runs on the host (Poseidon2 or Monolith by basefold_set_merkle_hash, as for the prover); the one
// thing fetched from the device is the folding table's (point, weight) pairs at the queried positions: one small
// gather kernel after the query indices are known.
#include <cstring>
#include <vector>
#include "gl_basefold_common.cuh"
#include "gl_transcript.hpp"

using namespace mb;

namespace mbhost {
namespace {

using gl::E2;

inline Digest digest_of(int hash, uint64_t a, uint64_t b, uint64_t c, uint64_t d) {   // leaf of two elements (base: c = d = 0)
    const uint64_t l[4] = {a, b, c, d}, z[4] = {0, 0, 0, 0};
    return host_compress(hash, l, z);
}
inline Digest compress(int hash, const uint64_t* l, const uint64_t* r) { return host_compress(hash, l, r); }
bool path_ok(int hash, Digest cur, const uint64_t* path, size_t len, size_t idx, const uint64_t* root) {
    for (size_t k = 0; k < len; k++) {
        cur = (idx & 1) == 0 ? compress(hash, cur.w, path + 4 * k) : compress(hash, path + 4 * k, cur.w);
        idx >>= 1;
    }
    for (int i = 0; i < 4; i++)
        if (cur.w[i] != root[i]) return false;
    return true;
}
// Proof words are compared as they stand: every prover writes canonical words, so a non-canonical one is a
// mismatch, as it is for the reference's PartialEq on field elements after from_canonical_u64.
inline E2 ld(const uint64_t* w) { return E2{w[0], w[1]}; }
inline E2 canon(E2 a) { return gl::e2_canon(a); }
inline bool same(E2 a, E2 b) { return a.c0 == b.c0 && a.c1 == b.c1; }
// c0 + c1 x + c2 x^2 of a round's oracle (six words)
inline E2 oracle_at(const uint64_t* o, E2 x) {
    const E2 c0 = ld(o), c1 = ld(o + 2), c2 = ld(o + 4);
    return canon(gl::e2_add(c0, gl::e2_add(gl::e2_mul(c1, x), gl::e2_mul(c2, canon(gl::e2_mul(x, x))))));
}

// out[k] = the (point, weight) pair at entry index[k] of the table
__global__ void table_gather_kernel(const uint64_t* __restrict__ entries, const uint64_t* __restrict__ index, size_t count,
                                    uint64_t* __restrict__ out) {
    const size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (k < count) {
        out[2 * k] = entries[2 * index[k]];
        out[2 * k + 1] = entries[2 * index[k] + 1];
    }
}

// The pairs at `want` of a table that lives on the device: one gather kernel and one copy back.
int fetch_from_device_table(const BasefoldTable& table, const uint64_t* want, size_t count, uint64_t* got) {
    DevBuf d_want, d_got;
    int rc = d_want.alloc(count);
    if (rc == MB_OK) rc = d_got.alloc(2 * count);
    if (rc != MB_OK) return rc;
    MB_CUDA(cudaMemcpyAsync(d_want.p, want, sizeof(uint64_t) * count, cudaMemcpyHostToDevice, MB_STREAM));
    {
        MB_KERNEL_ON("table_gather", MB_STREAM);
        table_gather_kernel<<<(unsigned)((count + 127) / 128), 128, 0, MB_STREAM>>>(table.d_entries.p, d_want.p, count, d_got.p);
    }
    MB_CUDA(cudaMemcpyAsync(got, d_got.p, sizeof(uint64_t) * 2 * count, cudaMemcpyDeviceToHost, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    return MB_OK;
}

}  // namespace

// *result = 0 when the opening is accepted, otherwise a negative code naming the first failed check:
// -1 claimed value against the first oracle, -(10 + i) oracle chain at round i, -100 query index, -101 commitment
// path, -(200 + i) fold consistency at round i, -(300 + i) folded-tree path at round i, -400 final codeword.
// fetch(want, count, got): got[2k], got[2k+1] = the (point, weight) pair at entry want[k] of the folding table (levels
// back to back, level i of 2^(nv + lr - i - 1) entries); returns MB_OK or an error.
template <class Fetch>
int basefold_verify(const uint64_t* root, int nv, int lr, const uint64_t* point, Fetch fetch, Transcript& t,
                    int num_queries, int hash, const uint64_t* proof, int* result) {
    if (nv < 1 || lr < 0 || nv + lr > 34 || num_queries < 0) return MB_ERR_ARG;
    if (hash < 0) hash = g_merkle_hash.load();
    std::vector<size_t> level_offsets(nv);
    {
        size_t total = 0;
        for (int i = 0; i < nv; i++) { level_offsets[i] = total; total += (size_t)1 << (nv + lr - i - 1); }
    }
    const uint64_t *p_eval = proof, *p_oracles = proof + 2, *p_roots = p_oracles + (size_t)nv * 6;
    const uint64_t *p_final = p_roots + (size_t)(nv - 1) * 4, *p_queries = p_final + ((size_t)2 << lr);
    const size_t qw = query_words(nv, lr);
    *result = 0;
    t.observe_hash(root);
    for (int i = 0; i < nv; i++) t.observe_ext2(Ext2{point[2 * i], point[2 * i + 1]});
    const E2 zero{0, 0}, one{1, 0};
    if (!same(canon(gl::e2_add(oracle_at(p_oracles, zero), oracle_at(p_oracles, one))), ld(p_eval))) { *result = -1; return MB_OK; }
    for (int k = 0; k < 3; k++) t.observe_ext2(Ext2{p_oracles[2 * k], p_oracles[2 * k + 1]});
    std::vector<E2> ch(nv);
    for (int round = 0; round < nv - 1; round++) {
        const Ext2 c = t.sample_challenge_ext2();
        ch[round] = E2{c.c0, c.c1};
        const uint64_t* on = p_oracles + 6 * (size_t)(round + 1);
        if (!same(oracle_at(p_oracles + 6 * (size_t)round, ch[round]), canon(gl::e2_add(oracle_at(on, zero), oracle_at(on, one))))) {
            *result = -(10 + round);
            return MB_OK;
        }
        for (int k = 0; k < 3; k++) t.observe_ext2(Ext2{on[2 * k], on[2 * k + 1]});
        t.observe_hash(p_roots + 4 * (size_t)round);
    }
    {
        const Ext2 c = t.sample_challenge_ext2();
        ch[nv - 1] = E2{c.c0, c.c1};
    }
    if (num_queries == 0) return MB_OK;

    // query indices, then the table entries they meet: level i at position index >> i
    const size_t cw_len = (size_t)1 << (nv + lr);
    std::vector<uint64_t> index(num_queries), want((size_t)num_queries * nv), got((size_t)num_queries * nv * 2);
    for (int q = 0; q < num_queries; q++) {
        index[q] = t.sample_challenge() % (uint64_t)(cw_len / 2);
        for (int i = 0; i < nv; i++) want[(size_t)q * nv + i] = level_offsets[i] + (index[q] >> i);
    }
    {
        const int rc = fetch(want.data(), want.size(), got.data());
        if (rc != MB_OK) return rc;
    }
    for (int q = 0; q < num_queries; q++) {
        const uint64_t* pq = p_queries + (size_t)q * qw;
        if (*pq++ != index[q]) { *result = -100; return MB_OK; }
        const uint64_t* vals = pq;
        pq += (size_t)nv * 4;
        const size_t plen = (size_t)(nv + lr - 1);
        if (vals[1] != 0 || vals[3] != 0 ||
            !path_ok(hash, digest_of(hash, vals[0], vals[2], 0, 0), pq, plen, (size_t)index[q], root)) {
            *result = -101;
            return MB_OK;
        }
        pq += 4 * plen;
        size_t fold_idx = (size_t)index[q];
        for (int i = 0; i < nv; i++) {
            const uint64_t* v = vals + 4 * (size_t)i;
            const E2 v0 = ld(v), v1 = ld(v + 2);
            const uint64_t x0 = got[((size_t)q * nv + i) * 2], w = got[((size_t)q * nv + i) * 2 + 1];
            // v0 + (r - x0) (v1 - v0) w: the line through (x0, v0) and (x1, v1) at the round's challenge
            const E2 cx = gl::e2_sub(ch[i], E2{x0, 0});
            const E2 slope = canon(gl::e2_mul(canon(cx), canon(gl::e2_sub(v1, v0))));
            const E2 res = canon(gl::e2_add(v0, E2{gl::mul(slope.c0, w), gl::mul(slope.c1, w)}));
            if (i < nv - 1) {
                const uint64_t* nxt = vals + 4 * (size_t)(i + 1);
                if (!same(res, ld((fold_idx & 1) == 0 ? nxt : nxt + 2))) { *result = -(200 + i); return MB_OK; }
                const size_t fl = (size_t)(nv + lr - 2 - i);
                if (!path_ok(hash, digest_of(hash, nxt[0], nxt[1], nxt[2], nxt[3]), pq, fl, fold_idx / 2, p_roots + 4 * (size_t)i)) {
                    *result = -(300 + i);
                    return MB_OK;
                }
                pq += 4 * fl;
            } else if (!same(res, ld(p_final + 2 * fold_idx))) {
                *result = -400;
                return MB_OK;
            }
            fold_idx /= 2;
        }
    }
    return MB_OK;
}

}  // namespace mbhost

extern "C" {

// Verifies an opening written by basefold_open_ext2 / basefold_prove_* (any of the provers: the proofs are the
// same words). h_root: the commitment root; h_point: num_vars (c0, c1) pairs; table: the handle the prover used;
// the transcript starts as Transcript::new(label). *result = 0 when accepted, else the negative code of the first
// failed check (see basefold_verify). merkle_hash: 0 Poseidon2, 1 Monolith, negative = the current setting of
// basefold_set_merkle_hash. Returns 0 unless an argument or a CUDA call (the table gather) fails.
int basefold_verify_host(const uint64_t* h_root, int num_vars, int log_rate, const uint64_t* h_point, const void* table,
                         const uint8_t* label, size_t label_len, int num_queries, int merkle_hash, const uint64_t* h_proof,
                         int* result) {
    if (!h_root || !h_point || !table || !h_proof || !result || (!label && label_len)) return MB_ERR_ARG;
    const mbhost::BasefoldTable& tb = *static_cast<const mbhost::BasefoldTable*>(table);
    if (tb.num_vars != num_vars || tb.log_rate != log_rate || tb.rounds < num_vars) return MB_ERR_ARG;
    mbhost::Transcript t(label, label_len);
    auto fetch = [&tb](const uint64_t* want, size_t count, uint64_t* got) {
        return mbhost::fetch_from_device_table(tb, want, count, got);
    };
    return mbhost::basefold_verify(h_root, num_vars, log_rate, h_point, fetch, t, num_queries, merkle_hash > 1 ? 1 : merkle_hash,
                                   h_proof, result);
}

// The same verifier with the folding table in host memory (h_table: (point, weight) pairs, levels back to back, as
// basefold_table_download writes them): no device call at all, for a verifier on a machine without a GPU, which is
// where the reference's verifier runs (basefold.rs:1759-1925 is CPU code).
int basefold_verify_with_table_host(const uint64_t* h_root, int num_vars, int log_rate, const uint64_t* h_point,
                                    const uint64_t* h_table, const uint8_t* label, size_t label_len, int num_queries,
                                    int merkle_hash, const uint64_t* h_proof, int* result) {
    if (!h_root || !h_point || !h_table || !h_proof || !result || (!label && label_len)) return MB_ERR_ARG;
    mbhost::Transcript t(label, label_len);
    auto fetch = [h_table](const uint64_t* want, size_t count, uint64_t* got) {
        for (size_t k = 0; k < count; k++) {
            got[2 * k] = h_table[2 * want[k]];
            got[2 * k + 1] = h_table[2 * want[k] + 1];
        }
        return MB_OK;
    };
    return mbhost::basefold_verify(h_root, num_vars, log_rate, h_point, fetch, t, num_queries, merkle_hash > 1 ? 1 : merkle_hash,
                                   h_proof, result);
}

}  // extern "C"
