// One Basefold commitment and opening partitioned over G = 2^gamma GPUs (one host
// thread or process per GPU), bit-identical to the single-GPU proof.
//
// The reference runs one whole prover per device (zk-torch-3/src/commit/basefold.rs:119-146
// clones the tables per device); here the ranks share one proof. The protocol,
// the transcript and every proof word are those of open_ext2
// (goldilocks-cuda-rs/src/basefold.rs:578-863) on top of commit_device (:382-414).
//
// Partition. Rank g holds evaluations [g n/G, (g+1) n/G) (n = 2^nv) and owns the
// codeword positions [g C, (g+1) C), C = 2^(nv+lr) / G, of the commitment and of
// every folded codeword. Folds pair neighbours and sumcheck rounds pair
// neighbours, so both stay inside a rank until its piece is short.
//
//   commit   The codeword is 2^lr equal blocks of T in bit-reversed order, where T
//            is the tensor power of the map (e0, e1) -> (e1, 2 e0 - e1) applied to
//            the evaluations (interpolation followed by the encoder's butterfly,
//            bit by bit). A rank's codeword range is the slice of T whose low
//            m = gamma - lr index bits are fixed: each rank transforms its low m
//            bits, one device all-to-all moves the slices (the whole polynomial
//            crosses the links once), the remaining nv - m bits are the ordinary
//            interpolate + encode passes on the slice. The 2^lr ranks that hold
//            equal slices hash one 1/2^lr part of the slice's leaves each; the G
//            part roots are gathered and the top of the tree is hashed on the
//            host by every rank.
//   open     eq is built per rank from the low coordinates and scaled by the eq
//            value of the rank's high bits; the evaluations themselves are the
//            other sumcheck table. A round is the single-GPU round on the rank's
//            piece, then one gather of ten words per rank (three partial oracle
//            coefficients, the root of the rank's subtree of the folded
//            codeword); the top gamma levels of each tree are hashed on the host.
//            When a rank's sumcheck piece is down to 2^TAIL_LOG = 4 elements the
//            pieces are gathered and every rank finishes the remaining rounds on
//            the whole (small) tables, replicated.
//   queries  Every rank packs the values and the lower path levels of the
//            (query, level) pairs whose leaves it hashed; one gather moves the
//            packed pieces (about 1 / G of the query section per rank); the upper
//            levels come from the gathered roots, the levels after the gather from
//            the rank's own copies.
//
// Exchanges go through mb_exchange (exchange.hpp); no kernel waits on another rank.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include "gl_basefold_common.cuh"
#include "exchange.hpp"

namespace mbhost {

// Sumcheck piece length (log2) at which the ranks gather and finish together. Small on purpose: a round on a
// rank's piece hashes a subtree that is log2(world) levels shallower than the whole tree (those levels are seven
// host permutations), and a tree level costs the latency of one permutation on the device whatever its width, so
// rounds are cheaper before the gather than after it.
constexpr int TAIL_LOG = 2;
constexpr int MAX_SLICE_BITS = 4;  // low index bits transformed before the exchange (G <= 16 * 2^lr)

// Low-`m`-bit part of the commitment transform and packing for the all-to-all:
// send[r][xh] = A[xh 2^m + tau_r], A = the evaluations with (e0, e1) -> (e1, 2 e0 - e1) applied on bits 0..m-1,
// tau_r = the m-bit reversal of rank r's slice index.
__global__ void __launch_bounds__(256)
slice_pack_kernel(const uint64_t* __restrict__ evals, uint64_t* __restrict__ send, size_t pieces, int m, int world) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    const int width = 1 << m;
    for (size_t xh = (size_t)blockIdx.x * blockDim.x + threadIdx.x; xh < pieces; xh += step) {
        uint64_t a[1 << MAX_SLICE_BITS];
#pragma unroll
        for (int k = 0; k < (1 << MAX_SLICE_BITS); k++)
            if (k < width) a[k] = evals[xh * width + k];
#pragma unroll
        for (int bit = 0; bit < MAX_SLICE_BITS; bit++) {
            if (bit < m) {
#pragma unroll
                for (int k = 0; k < (1 << MAX_SLICE_BITS); k++) {
                    if (k < width && !((k >> bit) & 1)) {
                        uint64_t e0 = a[k], e1 = a[k | (1 << bit)];
                        a[k] = e1;
                        a[k | (1 << bit)] = gl::sub(gl::add(e0, e0), e1);
                    }
                }
            }
        }
        for (int r = 0; r < world; r++) {
            int s = r & (width - 1), tau = 0;
            for (int b = 0; b < m; b++) tau |= ((s >> b) & 1) << (m - 1 - b);
            uint64_t v = 0;
#pragma unroll
            for (int k = 0; k < (1 << MAX_SLICE_BITS); k++)
                if (k == tau) v = a[k];
            send[(size_t)r * pieces + xh] = gl::canon(v);
        }
    }
}

// Where a rank's data for the query phase lives.
struct ShardQuery {
    int nv, lr, gamma, rank, world, switch_round;
    int part;                      // index of the commitment-tree part this rank hashed
    size_t part_leaves;            // leaves per part
    size_t slice_first_leaf;       // first block leaf of this rank's codeword slice
    const uint64_t* slice;         // this rank's slice of the codeword block
    const uint64_t* part_tree;     // tree over the part's leaves
    const uint64_t* fcw[40];       // folded codewords: the rank's piece before the switch, whole after
    const uint64_t* ftree[40];
};

// Block q writes this rank's share of query q. Levels hashed before the gather belong to one rank each: their
// values and lower path levels (an "item": 4 + 4 * depth words) go to `packed` at the offset the host computed
// for (query, level) in item_off (entries of other ranks' items are not read). Levels after the gather are held
// by every rank: they go straight to their place in `out`, laid out like the proof's query section.
__global__ void query_gather_sharded_kernel(ShardQuery sq, const uint64_t* __restrict__ leaf_idx,
                                            const uint32_t* __restrict__ item_off, uint64_t* __restrict__ packed,
                                            uint64_t* __restrict__ out, size_t qwords) {
    const int nv = sq.nv, lr = sq.lr;
    const int items = sq.switch_round + 1;
    uint64_t* pq = out + (size_t)blockIdx.x * qwords;
    const size_t leaf = (size_t)leaf_idx[blockIdx.x];
    const uint32_t* off = item_off + (size_t)blockIdx.x * items;
    if (threadIdx.x == 0) pq[0] = leaf;
    // commitment tree: the block repeats, a leaf belongs to the part that hashed its image in the first block
    {
        const size_t bl = leaf & (((size_t)1 << (nv - 1)) - 1);
        if ((int)(bl / sq.part_leaves) == sq.part) {
            uint64_t* dst = packed + off[0];
            const size_t in_slice = bl - sq.slice_first_leaf;
            if (threadIdx.x == 0) {
                dst[0] = sq.slice[2 * in_slice];
                dst[1] = 0;
                dst[2] = sq.slice[2 * in_slice + 1];
                dst[3] = 0;
            }
            copy_path(sq.part_tree, sq.part_leaves, bl - (size_t)sq.part * sq.part_leaves, dst + 4);
        }
    }
    uint64_t* vals = pq + 1;
    uint64_t* pp = vals + 4 * nv + 4 * (nv + lr - 1);
    for (int i = 0; i <= nv - 2; i++) {
        const size_t tree_leaves = (size_t)1 << (nv + lr - 2 - i);
        const size_t idx = leaf >> (i + 1);
        if (i < sq.switch_round) {
            const size_t local = tree_leaves >> sq.gamma;
            if ((int)(idx / local) == sq.rank) {
                uint64_t* dst = packed + off[i + 1];
                const size_t li = idx - (size_t)sq.rank * local;
                if (threadIdx.x < 4) dst[threadIdx.x] = sq.fcw[i][4 * li + threadIdx.x];
                copy_path(sq.ftree[i], local, li, dst + 4);
            }
        } else {
            if (threadIdx.x < 4) vals[4 * (i + 1) + threadIdx.x] = sq.fcw[i][4 * idx + threadIdx.x];
            copy_path(sq.ftree[i], tree_leaves, idx, pp);
        }
        pp += 4 * (nv + lr - 2 - i);
    }
}

namespace {

// Host-side stopwatch of the phases of one proof, printed by rank 0 when MB_SHARD_TIMING is set
// (a line per proof on stderr: milliseconds per phase). Costs a few clock reads otherwise.
struct PhaseClock {
    using clk = std::chrono::steady_clock;
    clk::time_point last = clk::now();
    double ms[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    void lap(int phase) {
        auto now = clk::now();
        ms[phase] += std::chrono::duration<double, std::milli>(now - last).count();
        last = now;
    }
    void report(int rank) const {
        static const bool on = std::getenv("MB_SHARD_TIMING") != nullptr;
        if (!on || rank != 0) return;
        std::fprintf(stderr, "[sharded basefold] pack+all-to-all %.3f  slice transform+part tree %.3f  eq+oracle0 %.3f  "
                             "rounds before the gather %.3f  gather %.3f  rounds after %.3f  queries %.3f ms\n",
                     ms[0], ms[1], ms[2], ms[3], ms[4], ms[5], ms[6]);
    }
};

// levels[0] = the given digests, levels[k + 1][j] = compress(levels[k][2j], levels[k][2j+1]).
std::vector<std::vector<Digest>> host_top_tree(int hash, std::vector<Digest> leaves) {
    std::vector<std::vector<Digest>> levels;
    levels.push_back(std::move(leaves));
    while (levels.back().size() > 1) {
        const auto& cur = levels.back();
        std::vector<Digest> next(cur.size() / 2);
        for (size_t j = 0; j < next.size(); j++) next[j] = host_compress(hash, cur[2 * j], cur[2 * j + 1]);
        levels.push_back(std::move(next));
    }
    return levels;
}

int ilog2(size_t x) {
    int l = 0;
    while (((size_t)1 << l) < x) l++;
    return l;
}

}  // namespace

// d_evals: this rank's n / world evaluations. proof: the whole proof on every rank (query part OR-ed together).
int prove_sharded(const uint64_t* d_evals, int nv, int lr, const uint64_t* point, const BasefoldTable& table, Transcript& t,
                  int num_queries, const mb_exchange* ex, uint64_t* h_root, uint64_t* proof) {
    const int G = ex->world, g = ex->rank;
    if (G < 2 || (G & (G - 1)) || g < 0 || g >= G) return MB_ERR_ARG;
    const int gamma = ilog2((size_t)G);
    const int m = gamma - lr;
    if (lr < 0 || m < 0 || m > MAX_SLICE_BITS) return MB_ERR_UNSUPPORTED;
    const int switch_round = nv - gamma - TAIL_LOG;   // first round on gathered tables
    if (switch_round < 1 || nv > 38) return MB_ERR_UNSUPPORTED;
    if (table.num_vars != nv || table.log_rate != lr || table.rounds < nv || num_queries < 0) return MB_ERR_ARG;
    const int hash = g_merkle_hash.load();

    const size_t n = (size_t)1 << nv, cw_len = (size_t)1 << (nv + lr);
    const size_t n_loc = n >> gamma;            // evaluations per rank
    const size_t C = cw_len >> gamma;           // codeword positions per rank
    const size_t piece = n_loc >> m;            // words each rank sends to each rank
    const int b_idx = g >> m, s_idx = g & ((1 << m) - 1);
    const size_t part_leaves = (n / 2) >> gamma;
    const int part = s_idx * (1 << lr) + b_idx;

    uint64_t* p_eval = proof;
    uint64_t* p_oracles = proof + 2;
    uint64_t* p_roots = p_oracles + (size_t)nv * 6;
    uint64_t* p_final = p_roots + (size_t)(nv - 1) * 4;
    uint64_t* p_queries = p_final + ((size_t)2 << lr);

    std::vector<uint64_t> h_mine, h_all;
    uint64_t* h_small = pinned_scratch();   // words 0..5 oracle, 6..9 subtree root, 16..47 the subtree's last device layer
    uint64_t* top_staging = pinned_arena(4 * (HOST_TOP - 1) * (size_t)nv);
    if (!h_small || !top_staging) return MB_ERR_CUDA;

    PhaseClock pc;
    // ---- commit ---------------------------------------------------------------------------------
    DevBuf send, slice, part_tree;
    int rc = send.alloc(C);
    if (rc == MB_OK) rc = slice.alloc(C);
    if (rc == MB_OK) rc = part_tree.alloc(4 * (2 * part_leaves - 1));
    if (rc != MB_OK) return rc;
    {
        MB_KERNEL_ON("slice_pack", MB_STREAM);
        slice_pack_kernel<<<grid_for(piece, 256, 8), 256, 0, MB_STREAM>>>(d_evals, send.p, piece, m, G);
    }
    if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    rc = ex->all_to_all_device(ex->ctx, send.p, slice.p, piece);
    if (rc != MB_OK) return rc;
    pc.lap(0);
    // the remaining nv - m bits: coefficients in `send`, butterflies in place, reversal into `slice`
    rc = bf::interpolate_async(slice.p, send.p, nullptr, nv - m, MB_STREAM);
    if (rc == MB_OK) rc = bf::encode_async(send.p, send.p, slice.p, nv - m, 0, MB_STREAM);
    if (rc != MB_OK) return rc;
    // this rank's part of the commitment tree: 1 / 2^lr of the slice's leaves
    {
        const uint64_t* leaves = slice.p + 2 * (size_t)b_idx * part_leaves;
        rc = hash ? mk::build_tree<mk::HashMonolith, false>(leaves, part_tree.p, part_leaves, MB_STREAM)
                  : mk::build_tree<mk::HashPoseidon2, false>(leaves, part_tree.p, part_leaves, MB_STREAM);
        if (rc != MB_OK) return rc;
    }
    MB_CUDA(cudaMemcpyAsync(h_small, part_tree.p + 4 * (2 * part_leaves - 2), 32, cudaMemcpyDeviceToHost, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    h_all.resize(4 * (size_t)G);
    rc = ex->all_gather_host(ex->ctx, h_small, 4, h_all.data());
    if (rc != MB_OK) return rc;
    // parts in block order, the block's tree above them, then lr levels whose two children are equal
    std::vector<std::vector<Digest>> commit_top;
    {
        std::vector<Digest> parts(G);
        for (int r = 0; r < G; r++) {
            int pr = (r & ((1 << m) - 1)) * (1 << lr) + (r >> m);
            std::memcpy(parts[pr].w, h_all.data() + 4 * r, 32);
        }
        commit_top = host_top_tree(hash, std::move(parts));
        for (int k = 0; k < lr; k++) {
            Digest top = commit_top.back()[0];
            commit_top.push_back({host_compress(hash, top, top)});
        }
    }
    uint64_t root[4];
    std::memcpy(root, commit_top.back()[0].w, 32);
    if (h_root) std::memcpy(h_root, root, 32);
    pc.lap(1);

    // ---- open ------------------------------------------------------------------------------------
    t.observe_hash(root);
    for (int i = 0; i < nv; i++) t.observe_ext2(Ext2{point[2 * i], point[2 * i + 1]});

    const int nv_loc = nv - gamma;
    DevBuf eq_a, eq_b, bh_a, bh_b, d_point, partial, small;
    const int grid_max = grid_for(n_loc / 2, 256, 4);
    rc = eq_a.alloc(2 * n_loc);
    if (rc == MB_OK) rc = eq_b.alloc(n_loc);
    if (rc == MB_OK) rc = bh_a.alloc(n_loc);
    if (rc == MB_OK) rc = bh_b.alloc(n_loc / 2 > 2 ? n_loc / 2 : 2);
    if (rc == MB_OK) rc = d_point.alloc(2 * (size_t)nv + 2);
    if (rc == MB_OK) rc = partial.alloc(6 * (size_t)grid_max);
    if (rc == MB_OK) rc = small.alloc(16);
    if (rc != MB_OK) return rc;
    unsigned int* counter = reinterpret_cast<unsigned int*>(small.p + 8);
    MB_CUDA(cudaMemsetAsync(small.p, 0, 16 * sizeof(uint64_t), MB_STREAM));

    // eq over the rank's low coordinates, scaled by the eq value of its high bits
    {
        std::vector<uint64_t> hp(2 * (size_t)nv + 2);
        std::memcpy(hp.data(), point, sizeof(uint64_t) * 2 * nv);
        gl::E2 scale{1, 0};
        for (int k = 0; k < gamma; k++) {
            gl::E2 r{point[2 * (nv_loc + k)], point[2 * (nv_loc + k) + 1]};
            gl::E2 f = ((g >> k) & 1) ? r : gl::e2_sub(gl::E2{1, 0}, r);
            scale = gl::e2_mul(scale, f);
        }
        scale = gl::e2_canon(scale);
        hp[2 * nv] = scale.c0;
        hp[2 * nv + 1] = scale.c1;
        MB_CUDA(cudaMemcpyAsync(d_point.p, hp.data(), sizeof(uint64_t) * hp.size(), cudaMemcpyHostToDevice, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    }
    rc = eq::build<sc::GlExt2>(d_point.p, eq_a.p, bh_a.p, nv_loc, MB_STREAM, d_point.p + 2 * nv);
    if (rc != MB_OK) return rc;

    // oracle 0: partial coefficients per rank, summed by everyone
    {
        MB_KERNEL_ON("oracle0", MB_STREAM);
        oracle0_kernel<<<grid_for(n_loc / 2, 256, 4), 256, 0, MB_STREAM>>>(eq_a.p, d_evals, n_loc / 2, partial.p, counter, small.p);
    }
    MB_CUDA(cudaMemcpyAsync(h_small, small.p, 48, cudaMemcpyDeviceToHost, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    h_all.resize(16 * (size_t)G);
    rc = ex->all_gather_host(ex->ctx, h_small, 6, h_all.data());
    if (rc != MB_OK) return rc;
    auto sum_oracle = [&](const uint64_t* all, size_t stride, uint64_t* out6) {
        for (int k = 0; k < 6; k++) {
            uint64_t s = 0;
            for (int r = 0; r < G; r++) s = gl::add(s, all[(size_t)r * stride + k]);
            out6[k] = gl::canon(s);
        }
    };
    sum_oracle(h_all.data(), 6, p_oracles);
    {
        gl::E2 c0{p_oracles[0], p_oracles[1]}, c1{p_oracles[2], p_oracles[3]}, c2{p_oracles[4], p_oracles[5]};
        gl::E2 ev = gl::e2_canon(gl::e2_add(gl::e2_add(c0, c0), gl::e2_add(c1, c2)));
        p_eval[0] = ev.c0;
        p_eval[1] = ev.c1;
    }
    for (int k = 0; k < 3; k++) t.observe_ext2(Ext2{p_oracles[2 * k], p_oracles[2 * k + 1]});
    pc.lap(2);

    // folded codewords and trees: the rank's piece before the switch, whole from the switch on
    std::vector<std::unique_ptr<DevBuf>> fcw(nv), ftree(nv - 1);
    for (int i = 0; i < nv; i++) {
        size_t len = (cw_len / 2) >> i;             // elements of folded codeword i
        if (i < switch_round) len >>= gamma;
        fcw[i].reset(new DevBuf);
        rc = fcw[i]->alloc(2 * len);
        if (rc != MB_OK) return rc;
        if (i < nv - 1) {
            ftree[i].reset(new DevBuf);
            rc = ftree[i]->alloc(4 * (len - 1 > 0 ? len - 1 : 1));
            if (rc != MB_OK) return rc;
        }
    }
    std::vector<std::vector<std::vector<Digest>>> ftop(switch_round);   // top gamma levels of the trees before the switch

    // tables of the tail: gathered pieces, ping-pong
    const size_t tail_live = ((size_t)1 << TAIL_LOG) << gamma;
    DevBuf tail_eq[2], tail_bh[2], tail_cw;
    for (int k = 0; k < 2; k++) {
        rc = tail_eq[k].alloc(2 * tail_live);
        if (rc == MB_OK) rc = tail_bh[k].alloc(2 * tail_live);
        if (rc != MB_OK) return rc;
    }
    rc = tail_cw.alloc(2 * ((cw_len / 2) >> (switch_round - 1)));
    if (rc != MB_OK) return rc;

    const uint64_t *eq_cur = eq_a.p, *bh_cur = d_evals;
    uint64_t *eq_nxt = eq_b.p, *bh_nxt = bh_a.p;
    const uint64_t* cw_prev = nullptr;   // input of this round's codeword fold (round >= 1)
    size_t live = n_loc;                 // length of the sumcheck tables this rank works on
    size_t cw_pairs = C / 2;             // pairs of the codeword this rank folds
    bool distributed = true;
    for (int round = 0; round < nv - 1; round++) {
        if (round == switch_round) {
            pc.lap(3);
            // gather the sumcheck pieces and the last folded codeword; from here on every rank holds everything
            // one message per rank: its eq piece, its bh piece, its piece of the last folded codeword
            const size_t w_sc = 2 * live, w_cw = 4 * cw_pairs, w_all = 2 * w_sc + w_cw;
            h_mine.resize(w_all);
            MB_CUDA(cudaMemcpyAsync(h_mine.data(), eq_cur, w_sc * sizeof(uint64_t), cudaMemcpyDeviceToHost, MB_STREAM));
            MB_CUDA(cudaMemcpyAsync(h_mine.data() + w_sc, bh_cur, w_sc * sizeof(uint64_t), cudaMemcpyDeviceToHost, MB_STREAM));
            MB_CUDA(cudaMemcpyAsync(h_mine.data() + 2 * w_sc, fcw[round - 1]->p, w_cw * sizeof(uint64_t), cudaMemcpyDeviceToHost, MB_STREAM));
            MB_CUDA(cudaStreamSynchronize(MB_STREAM));
            h_all.resize(w_all * (size_t)G);
            rc = ex->all_gather_host(ex->ctx, h_mine.data(), w_all, h_all.data());
            if (rc != MB_OK) return rc;
            for (int q = 0; q < G; q++) {
                const uint64_t* src = h_all.data() + (size_t)q * w_all;
                MB_CUDA(cudaMemcpyAsync(tail_eq[0].p + (size_t)q * w_sc, src, w_sc * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM));
                MB_CUDA(cudaMemcpyAsync(tail_bh[0].p + (size_t)q * w_sc, src + w_sc, w_sc * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM));
                MB_CUDA(cudaMemcpyAsync(tail_cw.p + (size_t)q * w_cw, src + 2 * w_sc, w_cw * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM));
            }
            MB_CUDA(cudaStreamSynchronize(MB_STREAM));   // h_all is pageable and reused later
            eq_cur = tail_eq[0].p; bh_cur = tail_bh[0].p;
            eq_nxt = tail_eq[1].p; bh_nxt = tail_bh[1].p;
            cw_prev = tail_cw.p;
            live <<= gamma;
            cw_pairs <<= gamma;
            distributed = false;
            pc.lap(4);
        }
        Ext2 ch = t.sample_challenge_ext2();
        gl::E2 r{ch.c0, ch.c1};
        const size_t quarter = live / 4;
        const int gq = grid_for(quarter, 256, 4);
        {
            MB_KERNEL_ON("open_round", MB_STREAM);
            if (round == 0)
                open_round_kernel<true><<<gq, 256, 0, MB_STREAM>>>(eq_cur, bh_cur, r, eq_nxt, bh_nxt, quarter, partial.p, counter, h_small);
            else
                open_round_kernel<false><<<gq, 256, 0, MB_STREAM>>>(eq_cur, bh_cur, r, eq_nxt, bh_nxt, quarter, partial.p, counter, h_small);
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        // (the kernel's last block and the tree's last block write into the pinned landing zone themselves)
        // codeword fold on this rank's pairs with its entries of the round's table level, then the tree
        const uint64_t* level = table.device_level_ptr(round) + (distributed ? 2 * (size_t)g * cw_pairs : 0);
        const int gf = grid_for(cw_pairs, 256, 8);
        if (round == 0) {
            MB_KERNEL_ON("fold_mixed", MB_STREAM);
            bf::fold_mixed_kernel<<<gf, 256, 0, MB_STREAM>>>(slice.p, level, r, fcw[0]->p, cw_pairs);
        } else {
            MB_KERNEL_ON("fold_ext2", MB_STREAM);
            bf::fold_ext2_kernel<<<gf, 256, 0, MB_STREAM>>>(cw_prev, level, r, fcw[round]->p, cw_pairs);
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        // the device stops at the layer of HOST_TOP digests of this rank's (sub)tree; the host hashes the levels above
        const size_t leaves = cw_pairs / 2;
        rc = hash ? mk::build_tree<mk::HashMonolith, true>(fcw[round]->p, ftree[round]->p, leaves, MB_STREAM, h_small + 16, HOST_TOP)
                  : mk::build_tree<mk::HashPoseidon2, true>(fcw[round]->p, ftree[round]->p, leaves, MB_STREAM, h_small + 16, HOST_TOP);
        if (rc != MB_OK) return rc;
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        rc = host_finish_top(hash, h_small + 16, leaves < HOST_TOP ? leaves : HOST_TOP, top_staging + 4 * (HOST_TOP - 1) * (size_t)round,
                             ftree[round]->p, leaves, h_small + 6, MB_STREAM);
        if (rc != MB_OK) return rc;
        uint64_t* po = p_oracles + 6 * (size_t)(round + 1);
        uint64_t* pr = p_roots + 4 * (size_t)round;
        if (distributed) {
            h_all.resize(10 * (size_t)G);
            rc = ex->all_gather_host(ex->ctx, h_small, 10, h_all.data());
            if (rc != MB_OK) return rc;
            sum_oracle(h_all.data(), 10, po);
            std::vector<Digest> sub(G);
            for (int q = 0; q < G; q++) std::memcpy(sub[q].w, h_all.data() + 10 * (size_t)q + 6, 32);
            ftop[round] = host_top_tree(hash, std::move(sub));
            std::memcpy(pr, ftop[round].back()[0].w, 32);
        } else {
            std::memcpy(po, h_small, 48);
            std::memcpy(pr, h_small + 6, 32);
        }
        for (int k = 0; k < 3; k++) t.observe_ext2(Ext2{po[2 * k], po[2 * k + 1]});
        t.observe_hash(pr);

        eq_cur = eq_nxt;
        bh_cur = bh_nxt;
        if (distributed) {
            eq_nxt = (eq_nxt == eq_b.p) ? eq_a.p : eq_b.p;
            bh_nxt = (bh_nxt == bh_a.p) ? bh_b.p : bh_a.p;
        } else {
            eq_nxt = (eq_nxt == tail_eq[1].p) ? tail_eq[0].p : tail_eq[1].p;
            bh_nxt = (bh_nxt == tail_bh[1].p) ? tail_bh[0].p : tail_bh[1].p;
        }
        cw_prev = fcw[round]->p;
        live /= 2;
        cw_pairs /= 2;
    }

    // last challenge: final fold, no tree (replicated: the switch always comes before)
    {
        Ext2 ch = t.sample_challenge_ext2();
        gl::E2 r{ch.c0, ch.c1};
        {
            MB_KERNEL_ON("fold_ext2", MB_STREAM);
            bf::fold_ext2_kernel<<<grid_for(cw_pairs, 256, 8), 256, 0, MB_STREAM>>>(cw_prev, table.device_level_ptr(nv - 1), r,
                                                                                     fcw[nv - 1]->p, cw_pairs);
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        MB_CUDA(cudaMemcpyAsync(p_final, fcw[nv - 1]->p, sizeof(uint64_t) * ((size_t)2 << lr), cudaMemcpyDeviceToHost, MB_STREAM));
    }

    pc.lap(5);
    // ---- queries ------------------------------------------------------------------------------------
    if (num_queries > 0) {
        std::vector<uint64_t> idx(num_queries);
        for (int q = 0; q < num_queries; q++) idx[q] = t.sample_challenge() % (uint64_t)(cw_len / 2);
        const size_t qw = query_words(nv, lr);
        const size_t total = qw * (size_t)num_queries;
        const int items = switch_round + 1;      // per query: the commitment tree and the trees hashed before the gather
        const int part_depth = ilog2(part_leaves);
        // every rank lays out every rank's packed buffer the same way: item (q, level) of owner r at offset[r]
        std::vector<uint32_t> item_off((size_t)num_queries * items), item_owner((size_t)num_queries * items);
        std::vector<uint32_t> fill(G, 0);
        auto item_words = [&](int level) {   // level 0: commitment tree; level i + 1: folded tree i
            if (level == 0) return (uint32_t)(4 + 4 * part_depth);
            return (uint32_t)(4 + 4 * (nv + lr - 2 - (level - 1) - gamma));
        };
        for (int q = 0; q < num_queries; q++) {
            const size_t leaf = (size_t)idx[q];
            for (int level = 0; level < items; level++) {
                int owner;
                if (level == 0) {
                    const int pr = (int)((leaf & (((size_t)1 << (nv - 1)) - 1)) / part_leaves);
                    owner = ((pr & ((1 << lr) - 1)) << m) | (pr >> lr);   // the rank whose part index is pr
                } else {
                    const size_t local = ((size_t)1 << (nv + lr - 2 - (level - 1))) >> gamma;
                    owner = (int)((leaf >> level) / local);
                }
                item_owner[(size_t)q * items + level] = (uint32_t)owner;
                item_off[(size_t)q * items + level] = fill[owner];
                fill[owner] += item_words(level);
            }
        }
        uint32_t packed_words = 16;
        for (int r = 0; r < G; r++) packed_words = fill[r] > packed_words ? fill[r] : packed_words;
        DevBuf d_idx, d_q, d_off, d_packed;
        rc = d_idx.alloc(num_queries);
        if (rc == MB_OK) rc = d_q.alloc(total);
        if (rc == MB_OK) rc = d_off.alloc((item_off.size() + 1) / 2);
        if (rc == MB_OK) rc = d_packed.alloc(packed_words);
        if (rc != MB_OK) return rc;
        MB_CUDA(cudaMemcpyAsync(d_idx.p, idx.data(), sizeof(uint64_t) * num_queries, cudaMemcpyHostToDevice, MB_STREAM));
        MB_CUDA(cudaMemcpyAsync(d_off.p, item_off.data(), sizeof(uint32_t) * item_off.size(), cudaMemcpyHostToDevice, MB_STREAM));
        MB_CUDA(cudaMemsetAsync(d_q.p, 0, sizeof(uint64_t) * total, MB_STREAM));
        MB_CUDA(cudaMemsetAsync(d_packed.p, 0, sizeof(uint64_t) * packed_words, MB_STREAM));
        ShardQuery sq;
        sq.nv = nv; sq.lr = lr; sq.gamma = gamma; sq.rank = g; sq.world = G; sq.switch_round = switch_round;
        sq.part = part;
        sq.part_leaves = part_leaves;
        sq.slice_first_leaf = (size_t)s_idx * (C / 2);
        sq.slice = slice.p;
        sq.part_tree = part_tree.p;
        for (int i = 0; i <= nv - 2; i++) { sq.fcw[i] = fcw[i]->p; sq.ftree[i] = ftree[i]->p; }
        {
            MB_KERNEL_ON("query_gather", MB_STREAM);
            query_gather_sharded_kernel<<<num_queries, 128, 0, MB_STREAM>>>(sq, d_idx.p, reinterpret_cast<const uint32_t*>(d_off.p),
                                                                              d_packed.p, d_q.p, qw);
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        h_mine.resize(packed_words);
        MB_CUDA(cudaMemcpyAsync(p_queries, d_q.p, sizeof(uint64_t) * total, cudaMemcpyDeviceToHost, MB_STREAM));
        MB_CUDA(cudaMemcpyAsync(h_mine.data(), d_packed.p, sizeof(uint64_t) * packed_words, cudaMemcpyDeviceToHost, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        h_all.resize((size_t)packed_words * G);
        rc = ex->all_gather_host(ex->ctx, h_mine.data(), packed_words, h_all.data());
        if (rc != MB_OK) return rc;
        // items from their owners, then the upper path levels from the gathered roots
        for (int q = 0; q < num_queries; q++) {
            uint64_t* pq = p_queries + (size_t)q * qw;
            const size_t leaf = (size_t)idx[q];
            uint64_t* vals = pq + 1;
            uint64_t* pp = vals + 4 * (size_t)nv;
            {
                const uint64_t* src = h_all.data() + (size_t)item_owner[(size_t)q * items] * packed_words + item_off[(size_t)q * items];
                std::memcpy(vals, src, 32);
                std::memcpy(pp, src + 4, 32 * (size_t)part_depth);
                const size_t pidx = (leaf & (((size_t)1 << (nv - 1)) - 1)) / part_leaves;
                for (int l = part_depth; l < nv + lr - 1; l++) {
                    const int k = l - part_depth;   // level above the parts
                    const Digest& sib = k < gamma ? commit_top[k][(pidx >> k) ^ 1] : commit_top[k][0];
                    std::memcpy(pp + 4 * (size_t)l, sib.w, 32);
                }
            }
            pp += 4 * (size_t)(nv + lr - 1);
            for (int i = 0; i <= nv - 2; i++) {
                if (i < switch_round) {
                    const size_t it = (size_t)q * items + i + 1;
                    const uint64_t* src = h_all.data() + (size_t)item_owner[it] * packed_words + item_off[it];
                    const int local_depth = nv + lr - 2 - i - gamma;
                    std::memcpy(vals + 4 * (size_t)(i + 1), src, 32);
                    std::memcpy(pp, src + 4, 32 * (size_t)local_depth);
                    const size_t owner = item_owner[it];
                    for (int k = 0; k < gamma; k++)
                        std::memcpy(pp + 4 * (size_t)(local_depth + k), ftop[i][k][(owner >> k) ^ 1].w, 32);
                }
                pp += 4 * (size_t)(nv + lr - 2 - i);
            }
        }
    } else {
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    }
    pc.lap(6);
    pc.report(g);
    return MB_OK;
}

}  // namespace mbhost

extern "C" {

// Commit + opening of one polynomial shared by ex->world ranks (a power of two >= 2, at least 2^log_rate). Every
// rank calls this with its own contiguous 1 / world range of the evaluations in device memory (rank r: elements
// [r n / world, (r + 1) n / world)) and the same point, table, label and query count. h_root and h_proof receive
// the same words on every rank: exactly those of basefold_prove_host on the whole polynomial. -3 when the shape is
// not supported (num_vars < log2(world) + 3, or world > 16 * 2^log_rate).
int basefold_prove_sharded_device(const uint64_t* d_evals_shard, int num_vars, int log_rate, const uint64_t* h_point,
                                  const void* table, const uint8_t* label, size_t label_len, int num_queries,
                                  const mb_exchange* ex, uint64_t* h_root, uint64_t* h_proof) {
    if (!d_evals_shard || !h_point || !table || !ex || !h_proof || !ex->all_gather_host || !ex->all_to_all_device)
        return MB_ERR_ARG;
    mbhost::Transcript t(label, label_len);
    return mbhost::prove_sharded(d_evals_shard, num_vars, log_rate, h_point, *static_cast<const mbhost::BasefoldTable*>(table), t,
                                 num_queries, ex, h_root, h_proof);
}

// The same from host memory: h_evals_shard holds this rank's range; the copy to the device is part of the call.
int basefold_prove_sharded_host(const uint64_t* h_evals_shard, int num_vars, int log_rate, const uint64_t* h_point,
                                const void* table, const uint8_t* label, size_t label_len, int num_queries,
                                const mb_exchange* ex, uint64_t* h_root, uint64_t* h_proof) {
    if (!h_evals_shard || !ex || ex->world < 1 || num_vars < 1 || num_vars > 38) return MB_ERR_ARG;
    size_t words = ((size_t)1 << num_vars) / (size_t)ex->world;
    mbhost::DevBuf ev;
    int rc = ev.alloc(words);
    if (rc != MB_OK) return rc;
    MB_CUDA(cudaMemcpyAsync(ev.p, h_evals_shard, words * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM));
    return basefold_prove_sharded_device(ev.p, num_vars, log_rate, h_point, table, label, label_len, num_queries, ex, h_root,
                                         h_proof);
}

}  // extern "C"
