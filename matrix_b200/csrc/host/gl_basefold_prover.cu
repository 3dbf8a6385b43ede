// Host layer above the C-ABI for Basefold over Goldilocks: folding table,
// commitment and extension-field opening, written in C++ where the reference has
// Rust (no Rust toolchain on the build machine).
//
//   BasefoldTable        goldilocks-cuda-rs/src/basefold.rs:267-362
//   DeviceMerkleTree     goldilocks-cuda-rs/src/merkle.rs:20-160
//   BasefoldCommitment   goldilocks-cuda-rs/src/basefold.rs:368-414 (commit_device)
//   open_ext2            goldilocks-cuda-rs/src/basefold.rs:578-863
//   extract_ext2_queries goldilocks-cuda-rs/src/basefold.rs:2310-2402
//
// The protocol order, every transcript interaction and every value that enters
// the proof are the reference's. The work between them is organised for the
// B200: the claimed value is read off the first oracle (eval = p(0) + p(1), one
// pass fewer), the inner sumcheck keeps its tables as plain values and folds
// them in the same pass that accumulates the next oracle, partial sums are
// finished on the device, each round issues its sumcheck pass, codeword fold and
// Merkle tree back to back and synchronises once, and the query phase is one
// gather kernel and one copy.
#include "gl_basefold_common.cuh"

namespace mbhost {

// open_ext2 (basefold.rs:578-863). Writes the proof as
//   eval[2] | oracles[nv][3][2] | folded_roots[nv-1][4] | final_codeword[2^lr][2] |
//   per query: index, nv value pairs [2][2], path in the commitment tree,
//   paths in the nv-1 folded trees (sibling digests bottom-up).
int open_ext2(const BasefoldCommitment& cm, const uint64_t* point, const BasefoldTable& table, Transcript& t,
              int num_queries, uint64_t* proof) {
    const int nv = cm.num_vars, lr = cm.log_rate;
    if (nv < 2 || nv > 38 || table.num_vars != nv || table.log_rate != lr || table.rounds < nv || num_queries < 0)
        return MB_ERR_ARG;
    const size_t n = (size_t)1 << nv, cw_len = (size_t)1 << (nv + lr);
    uint64_t* p_eval = proof;
    uint64_t* p_oracles = proof + 2;
    uint64_t* p_roots = p_oracles + (size_t)nv * 6;
    uint64_t* p_final = p_roots + (size_t)(nv - 1) * 4;
    uint64_t* p_queries = p_final + ((size_t)2 << lr);

    t.observe_hash(cm.root);
    for (int i = 0; i < nv; i++) t.observe_ext2(Ext2{point[2 * i], point[2 * i + 1]});

    // device state
    DevBuf eq_a, eq_b, bh_fp, bh_a, bh_b, d_point, partial, small, stage;
    const int grid_max = grid_for(n / 2, 256, 4);
    int rc = eq_a.alloc(2 * n);
    if (rc == MB_OK) rc = eq_b.alloc(n);
    if (rc == MB_OK) rc = bh_fp.alloc(n);
    if (rc == MB_OK) rc = bh_a.alloc(n);
    if (rc == MB_OK) rc = bh_b.alloc(n / 2 > 2 ? n / 2 : 2);
    if (rc == MB_OK) rc = d_point.alloc(2 * (size_t)nv);
    if (rc == MB_OK) rc = partial.alloc(6 * (size_t)grid_max);
    if (rc == MB_OK) rc = small.alloc(16);  // [0..6) oracle words, [8] ticket counter
    if (rc != MB_OK) return rc;
    unsigned int* counter = reinterpret_cast<unsigned int*>(small.p + 8);
    MB_CUDA(cudaMemsetAsync(small.p, 0, 16 * sizeof(uint64_t), MB_STREAM));
    uint64_t* h_small = pinned_scratch();  // landing zone: 6 oracle words, then (from word 8) the tree's last device layer
    uint64_t* top_staging = pinned_arena(4 * (HOST_TOP - 1) * (size_t)nv);   // host-hashed tree tops on their way up
    if (!h_small || !top_staging) return MB_ERR_CUDA;

    MB_CUDA(cudaMemcpyAsync(d_point.p, point, sizeof(uint64_t) * 2 * nv, cudaMemcpyHostToDevice, MB_STREAM));
    // eq table; bh_a doubles as scratch for the two small tables (free until round 0 writes it)
    rc = eq::build<sc::GlExt2>(d_point.p, eq_a.p, bh_a.p, nv, MB_STREAM);
    if (rc != MB_OK) return rc;
    // evaluations back in natural order (basefold.rs:600-602)
    if (nv >= 12) {
        size_t tiles = (size_t)1 << (nv - 12);
        int g = (int)(tiles < (size_t)sm_count() * 4 ? tiles : (size_t)sm_count() * 4);
        {
            MB_KERNEL_ON("bit_reverse_tiled", MB_STREAM);
            bf::bit_reverse_tiled_kernel<<<g, 256, 0, MB_STREAM>>>(cm.d_bh_evals.p, bh_fp.p, nv, 1);
        }
    } else {
        {
            MB_KERNEL_ON("bit_reverse_copy", MB_STREAM);
            bf::bit_reverse_copy_kernel<<<grid_for(n, 256, 8), 256, 0, MB_STREAM>>>(cm.d_bh_evals.p, bh_fp.p, nv, 1);
        }
    }

    // oracle 0 and the claimed value eval = p(0) + p(1) = 2 c0 + c1 + c2
    {
        MB_KERNEL_ON("oracle0", MB_STREAM);
        oracle0_kernel<<<grid_for(n / 2, 256, 4), 256, 0, MB_STREAM>>>(eq_a.p, bh_fp.p, n / 2, partial.p, counter, small.p);
    }
    MB_CUDA(cudaMemcpyAsync(h_small, small.p, 48, cudaMemcpyDeviceToHost, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    std::memcpy(p_oracles, h_small, 48);
    {
        gl::E2 c0{h_small[0], h_small[1]}, c1{h_small[2], h_small[3]}, c2{h_small[4], h_small[5]};
        gl::E2 ev = gl::e2_canon(gl::e2_add(gl::e2_add(c0, c0), gl::e2_add(c1, c2)));
        p_eval[0] = ev.c0;
        p_eval[1] = ev.c1;
    }
    for (int k = 0; k < 3; k++) t.observe_ext2(Ext2{p_oracles[2 * k], p_oracles[2 * k + 1]});

    // folded codewords and trees, kept for the query phase
    std::vector<std::unique_ptr<DevBuf>> fcw(nv), ftree(nv - 1);
    {
        size_t len = cw_len / 2;
        for (int i = 0; i < nv; i++) {
            fcw[i].reset(new DevBuf);
            rc = fcw[i]->alloc(2 * len);
            if (rc != MB_OK) return rc;
            if (i < nv - 1) {
                ftree[i].reset(new DevBuf);
                rc = ftree[i]->alloc(4 * (len - 1 > 0 ? len - 1 : 1));
                if (rc != MB_OK) return rc;
            }
            len /= 2;
        }
    }

    const uint64_t *eq_cur = eq_a.p, *bh_cur = bh_fp.p;
    uint64_t *eq_nxt = eq_b.p, *bh_nxt = bh_a.p;
    size_t live = n;            // current length of the sumcheck tables
    size_t cw_pairs = cw_len / 2;
    for (int round = 0; round < nv - 1; round++) {
        Ext2 ch = t.sample_challenge_ext2();
        gl::E2 r{ch.c0, ch.c1};
        size_t quarter = live / 4;
        int g = grid_for(quarter, 256, 4);
        // the last block of the round kernel writes the finished oracle straight into pinned host memory, the last
        // block of the tree its root: a round is its launches and one stream synchronisation, no copy command
        if (round == 0) {
            {
                MB_KERNEL_ON("open_round", MB_STREAM);
                open_round_kernel<true><<<g, 256, 0, MB_STREAM>>>(eq_cur, bh_cur, r, eq_nxt, bh_nxt, quarter, partial.p,
                                                                  counter, h_small);
            }
        } else {
            {
                MB_KERNEL_ON("open_round", MB_STREAM);
                open_round_kernel<false><<<g, 256, 0, MB_STREAM>>>(eq_cur, bh_cur, r, eq_nxt, bh_nxt, quarter, partial.p,
                                                                   counter, h_small);
            }
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        // codeword fold with this round's table level, then its tree
        const uint64_t* level = table.device_level_ptr(round);
        int gf = grid_for(cw_pairs, 256, 8);
        if (round == 0) {
            {
                MB_KERNEL_ON("fold_mixed", MB_STREAM);
                bf::fold_mixed_kernel<<<gf, 256, 0, MB_STREAM>>>(cm.d_codeword.p, level, r, fcw[0]->p, cw_pairs);
            }
        } else {
            {
                MB_KERNEL_ON("fold_ext2", MB_STREAM);
                bf::fold_ext2_kernel<<<gf, 256, 0, MB_STREAM>>>(fcw[round - 1]->p, level, r, fcw[round]->p, cw_pairs);
            }
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        // the device stops at the layer of HOST_TOP digests; the host hashes the levels above it
        const size_t leaves = cw_pairs / 2;
        rc = cm.hash ? mk::build_tree<mk::HashMonolith, true>(fcw[round]->p, ftree[round]->p, leaves, MB_STREAM, h_small + 8, HOST_TOP)
                     : mk::build_tree<mk::HashPoseidon2, true>(fcw[round]->p, ftree[round]->p, leaves, MB_STREAM, h_small + 8, HOST_TOP);
        if (rc != MB_OK) return rc;
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        uint64_t* po = p_oracles + 6 * (size_t)(round + 1);
        std::memcpy(po, h_small, 48);
        rc = host_finish_top(cm.hash, h_small + 8, leaves < HOST_TOP ? leaves : HOST_TOP, top_staging + 4 * (HOST_TOP - 1) * (size_t)round,
                             ftree[round]->p, leaves, p_roots + 4 * (size_t)round, MB_STREAM);
        if (rc != MB_OK) return rc;
        for (int k = 0; k < 3; k++) t.observe_ext2(Ext2{po[2 * k], po[2 * k + 1]});
        t.observe_hash(p_roots + 4 * (size_t)round);

        // ping-pong: eq between eq_b and eq_a, bh between bh_a and bh_b
        eq_cur = eq_nxt;
        bh_cur = bh_nxt;
        eq_nxt = (eq_nxt == eq_b.p) ? eq_a.p : eq_b.p;
        bh_nxt = (bh_nxt == bh_a.p) ? bh_b.p : bh_a.p;
        live /= 2;
        cw_pairs /= 2;
    }

    // last challenge: final fold, no tree
    {
        Ext2 ch = t.sample_challenge_ext2();
        gl::E2 r{ch.c0, ch.c1};
        {
            MB_KERNEL_ON("fold_ext2", MB_STREAM);
            bf::fold_ext2_kernel<<<grid_for(cw_pairs, 256, 8), 256, 0, MB_STREAM>>>(
                fcw[nv - 2]->p, table.device_level_ptr(nv - 1), r, fcw[nv - 1]->p, cw_pairs);
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        MB_CUDA(cudaMemcpyAsync(p_final, fcw[nv - 1]->p, sizeof(uint64_t) * ((size_t)2 << lr), cudaMemcpyDeviceToHost,
                                MB_STREAM));
    }

    // queries: all indices first (basefold.rs:2321-2326), then one gather
    if (num_queries > 0) {
        std::vector<uint64_t> idx(num_queries);
        for (int q = 0; q < num_queries; q++) idx[q] = t.sample_challenge() % (uint64_t)(cw_len / 2);
        size_t qw = query_words(nv, lr);
        DevBuf d_idx, d_q;
        rc = d_idx.alloc(num_queries);
        if (rc == MB_OK) rc = d_q.alloc(qw * num_queries);
        if (rc != MB_OK) return rc;
        MB_CUDA(cudaMemcpyAsync(d_idx.p, idx.data(), sizeof(uint64_t) * num_queries, cudaMemcpyHostToDevice, MB_STREAM));
        QueryLevels lv;
        lv.nv = nv; lv.lr = lr;
        lv.commit_cw = cm.d_codeword.p;
        lv.commit_tree = cm.d_tree.p;
        for (int i = 0; i <= nv - 2; i++) { lv.fcw[i] = fcw[i]->p; lv.ftree[i] = ftree[i]->p; }
        {
            MB_KERNEL_ON("query_gather", MB_STREAM);
            query_gather_kernel<<<num_queries, 128, 0, MB_STREAM>>>(lv, d_idx.p, d_q.p, qw);
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        MB_CUDA(cudaMemcpyAsync(p_queries, d_q.p, sizeof(uint64_t) * qw * num_queries, cudaMemcpyDeviceToHost, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    } else {
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    }
    return MB_OK;
}

}  // namespace mbhost

// ---- C-ABI of the host layer -----------------------------------------------------------
using mbhost::BasefoldCommitment;
using mbhost::BasefoldTable;

extern "C" {

// Selects the Merkle hash of later commitments: 0 Poseidon2 (default), 1 Monolith.
int basefold_set_merkle_hash(int hash) {
    if (hash != 0 && hash != 1) return MB_ERR_ARG;
    mbhost::g_merkle_hash.store(hash);
    return MB_OK;
}

size_t basefold_proof_words(int num_vars, int log_rate, int num_queries) {
    return mbhost::proof_words(num_vars, log_rate, num_queries);
}

int basefold_table_create(int num_vars, int log_rate, int num_rounds, uint64_t seed, void** table) {
    if (!table) return MB_ERR_ARG;
    auto* t = new BasefoldTable;
    int rc = t->generate(num_vars, log_rate, num_rounds, seed);
    if (rc != MB_OK) { delete t; return rc; }
    *table = t;
    return MB_OK;
}
int basefold_table_destroy(void* table) { delete static_cast<BasefoldTable*>(table); return MB_OK; }
size_t basefold_table_entries(const void* table) { return static_cast<const BasefoldTable*>(table)->entries; }
// (point, weight) pairs, levels back to back, to host memory.
int basefold_table_download(const void* table, uint64_t* h_entries) {
    auto* t = static_cast<const BasefoldTable*>(table);
    MB_CUDA(cudaMemcpyAsync(h_entries, t->d_entries.p, t->entries * 16, cudaMemcpyDeviceToHost, MB_STREAM));
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
}
const uint64_t* basefold_table_level_ptr(const void* table, int level) {
    return static_cast<const BasefoldTable*>(table)->device_level_ptr(level);
}

int basefold_commit_device(const uint64_t* d_evals, int num_vars, int log_rate, void** commitment, uint64_t* h_root) {
    if (!commitment) return MB_ERR_ARG;
    auto* c = new BasefoldCommitment;
    int rc = c->commit_device(d_evals, num_vars, log_rate);
    if (rc != MB_OK) { delete c; return rc; }
    if (h_root) std::memcpy(h_root, c->root, 32);
    *commitment = c;
    return MB_OK;
}
int basefold_commit_host(const uint64_t* h_evals, int num_vars, int log_rate, void** commitment, uint64_t* h_root) {
    if (num_vars < 1 || num_vars > 32 || !h_evals) return MB_ERR_ARG;
    mbhost::DevBuf ev;
    int rc = ev.alloc((size_t)1 << num_vars);
    if (rc != MB_OK) return rc;
    MB_CUDA(cudaMemcpyAsync(ev.p, h_evals, sizeof(uint64_t) << num_vars, cudaMemcpyHostToDevice, MB_STREAM));
    return basefold_commit_device(ev.p, num_vars, log_rate, commitment, h_root);
}
int basefold_commitment_destroy(void* commitment) { delete static_cast<BasefoldCommitment*>(commitment); return MB_OK; }
// Device pointers of the commitment's parts (owned by the commitment).
const uint64_t* basefold_commitment_codeword(const void* c) { return static_cast<const BasefoldCommitment*>(c)->d_codeword.p; }
const uint64_t* basefold_commitment_bh_evals(const void* c) { return static_cast<const BasefoldCommitment*>(c)->d_bh_evals.p; }
const uint64_t* basefold_commitment_tree(const void* c) { return static_cast<const BasefoldCommitment*>(c)->d_tree.p; }

// Opening at an extension-field point (h_point: num_vars (c0, c1) pairs) with
// the transcript started as Transcript::new(label). h_proof must hold
// basefold_proof_words(...) words; h_transcript_state (8 words) may be NULL.
int basefold_open_ext2(const void* commitment, const uint64_t* h_point, const void* table, const uint8_t* label,
                       size_t label_len, int num_queries, uint64_t* h_proof, uint64_t* h_transcript_state) {
    if (!commitment || !h_point || !table || !h_proof) return MB_ERR_ARG;
    mbhost::Transcript t(label, label_len);
    int rc = mbhost::open_ext2(*static_cast<const BasefoldCommitment*>(commitment), h_point,
                               *static_cast<const BasefoldTable*>(table), t, num_queries, h_proof);
    if (rc == MB_OK && h_transcript_state) std::memcpy(h_transcript_state, t.state(), 64);
    return rc;
}

// Commit + open from host evaluations in one call; the commitment is dropped
// afterwards. h_root receives the commitment root.
int basefold_prove_host(const uint64_t* h_evals, int num_vars, int log_rate, const uint64_t* h_point, const void* table,
                        const uint8_t* label, size_t label_len, int num_queries, uint64_t* h_root, uint64_t* h_proof) {
    void* c = nullptr;
    int rc = basefold_commit_host(h_evals, num_vars, log_rate, &c, h_root);
    if (rc != MB_OK) return rc;
    rc = basefold_open_ext2(c, h_point, table, label, label_len, num_queries, h_proof, nullptr);
    basefold_commitment_destroy(c);
    return rc;
}

}  // extern "C"
