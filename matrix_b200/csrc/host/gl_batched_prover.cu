// Host layer for the batched degree-3 sumcheck (shared eq table, K instances
// combined with powers of alpha) over Goldilocks, one shard of the hypercube.
//
// A shard holds the slice of every table whose top index bits equal the shard
// number: a_k, b_k slices of 2^n_loc base-field elements, and the eq slice
// eq(t_low, x_low) * eq(t_top, shard) (the scalar is passed in). The per-round
// API mirrors the reference's state objects (compute message, then fold on the
// challenge; almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:127-436): the
// caller adds the shards' messages, runs the transcript and broadcasts the
// challenge. With one shard it is the whole prover. The C-ABI below also exposes
// the host transcript (zk-torch-3/src/transcript.rs:174-350) so that callers in
// any language run the same Fiat-Shamir.
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "../batched_kernels.cuh"
#include "../eq_kernels.cuh"
#include "exchange.hpp"
#include "gl_transcript.hpp"

using namespace mb;
using namespace mb::sc;

namespace mbhost {

class BatchedEqAbState {
public:
    ~BatchedEqAbState() { release(); }

    int init(const uint64_t* d_a, const uint64_t* d_b, const uint64_t* h_point_low, const uint64_t* h_eq_scale, int K,
             int n_loc) {
        if (!d_a || !d_b || !h_eq_scale || K < 1 || K > bt::MAX_K || n_loc < 1 || n_loc > 34) return MB_ERR_ARG;
        if (n_loc > 0 && !h_point_low) return MB_ERR_ARG;
        K_ = K; n_loc_ = n_loc; n_ = (size_t)1 << n_loc; round_ = 0; have_msg_ = false; have_alpha_ = false; have_inst_ = false;
        pt_.assign(h_point_low, h_point_low + 2 * (size_t)n_loc);
        a0_ = d_a;  // the caller's tables are read in place during round 0 and never written
        b0_ = d_b;
        size_t half = n_ / 2, quarter = n_ >= 4 ? n_ / 4 : 1;
        MB_CUDA(pool_alloc((void**)&eq0_, 16 * n_));
        MB_CUDA(pool_alloc((void**)&eq_a_, 16 * half));
        MB_CUDA(pool_alloc((void**)&eq_b_, 16 * quarter));
        MB_CUDA(pool_alloc((void**)&ab_a_, 16 * 2 * K * half));
        MB_CUDA(pool_alloc((void**)&ab_b_, 16 * 2 * K * quarter));
        grid_max_ = grid_for(half, 256, 4);
        // round-0 kernel: lane groups of Kp lanes, two output pairs per lane and step
        Kp_ = 1;
        while (Kp_ < K && Kp_ < 32) Kp_ *= 2;
        const size_t per_step = (size_t)2 * (32 / Kp_);
        grid_inst_ = grid_for(((half + per_step - 1) / per_step) * 32, 256, 3);
        size_t partial_words = 2 * (size_t)bt::NC * (size_t)grid_max_;
        if (partial_words < 2 * (size_t)bt::NC * K * grid_inst_) partial_words = 2 * (size_t)bt::NC * K * grid_inst_;
        MB_CUDA(pool_alloc((void**)&partial_, sizeof(uint64_t) * partial_words));
        MB_CUDA(pool_alloc((void**)&small_, sizeof(uint64_t) * (16 + 2 * bt::MAX_K + 2 * 40 + 2 + 4 * bt::MAX_K + 8 * bt::MAX_K)));
        msg_dev_ = small_;                      // 8 words
        counter_ = reinterpret_cast<unsigned int*>(small_ + 8);
        alpha_dev_ = small_ + 16;               // 2 * MAX_K words
        uint64_t* point_dev = alpha_dev_ + 2 * bt::MAX_K;  // 2 * 40 words
        uint64_t* scale_dev = point_dev + 80;               // 2 words
        wtab_dev_ = scale_dev + 2;                          // 4 * MAX_K words
        inst_dev_ = wtab_dev_ + 4 * bt::MAX_K;              // 8 * MAX_K words
        MB_CUDA(cudaMemsetAsync(small_, 0, 16 * sizeof(uint64_t), MB_STREAM));
        MB_CUDA(cudaMemcpyAsync(point_dev, h_point_low, 16 * (size_t)n_loc, cudaMemcpyHostToDevice, MB_STREAM));
        MB_CUDA(cudaMemcpyAsync(scale_dev, h_eq_scale, 16, cudaMemcpyHostToDevice, MB_STREAM));
        // eq slice scaled by eq(t_top, shard); ab_a_ is free until the first fold and serves as scratch
        int rc = eq::build<GlExt2>(point_dev, eq0_, ab_a_, n_loc, MB_STREAM, scale_dev);
        if (rc != MB_OK) return rc;
        // the table build and the copies above are complete before the handle is handed out, so that the
        // first call on it may come from another host thread (whose stream knows nothing of this one)
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        return MB_OK;
    }

    // Per-instance round-0 messages m_k(0..3) of this shard, one pass over the caller's tables.
    int instance_messages() {
        if (have_inst_) return MB_OK;
        const size_t half = n_ / 2;
        dim3 grid(grid_inst_, (K_ + 31) / 32);
        const size_t smem = sizeof(uint64_t) * 8 * 2 * (size_t)(2 * (32 / Kp_)) * 2;
        if (smem > 48 * 1024)
            MB_CUDA(cudaFuncSetAttribute(bt::instance_messages_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        {
            MB_KERNEL("batched_instance_messages");
            bt::instance_messages_kernel<<<grid, 256, smem, MB_STREAM>>>(eq0_, a0_, b0_, K_, Kp_, n_, half, partial_);
        }
        {
            MB_KERNEL("reduce_partials");
            reduce_partials_kernel<256, GlAdd, GlCanon><<<1, 256, 0, MB_STREAM>>>(partial_, grid_inst_, 2 * bt::NC * K_, inst_dev_);
        }
        inst_.resize(2 * (size_t)bt::NC * K_);
        MB_CUDA(cudaMemcpyAsync(inst_.data(), inst_dev_, sizeof(uint64_t) * inst_.size(), cudaMemcpyDeviceToHost, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        have_inst_ = true;
        return MB_OK;
    }

    // m(0..3) = lambda(c) T(c) from T(0), T(1) and the leading coefficient T2 (six words) for the
    // variable bound in `round`: lambda(c) = (1 - t) + c (2 t - 1), T(2) = 2 T(1) + 2 T2 - T(0),
    // T(3) = 3 T(1) + 6 T2 - 2 T(0).
    void expand_message(const uint64_t* t6, int round, gl::E2 (&out)[4]) const {
        const gl::E2 T0{t6[0], t6[1]}, T1{t6[2], t6[3]}, T2{t6[4], t6[5]};
        const gl::E2 t{gl::canon(pt_[2 * (size_t)round]), gl::canon(pt_[2 * (size_t)round + 1])};
        const gl::E2 s12 = gl::e2_add(T1, T2), s122 = gl::e2_add(s12, T2);
        gl::E2 T[4] = {T0, T1, gl::e2_sub(gl::e2_add(s12, s12), T0),
                       gl::e2_sub(gl::e2_sub(gl::e2_add(gl::e2_add(s122, s122), s122), T0), T0)};
        gl::E2 lam = gl::e2_sub(gl::E2{1, 0}, t);                 // lambda(0) = 1 - t
        const gl::E2 step = gl::e2_sub(gl::e2_add(t, t), gl::E2{1, 0});  // 2 t - 1
        for (int c = 0; c < 4; c++) {
            out[c] = gl::e2_canon(gl::e2_mul(lam, T[c]));
            lam = gl::e2_add(lam, step);
        }
    }

    // Local share of the per-instance claims s_k = m_k(0) + m_k(1) (K extension elements).
    int claims(uint64_t* h_out) {
        int rc = instance_messages();
        if (rc != MB_OK) return rc;
        for (int k = 0; k < K_; k++) {
            gl::E2 m[4];
            expand_message(inst_.data() + 2 * bt::NC * (size_t)k, 0, m);
            const gl::E2 s = gl::e2_canon(gl::e2_add(m[0], m[1]));
            h_out[2 * k] = s.c0;
            h_out[2 * k + 1] = s.c1;
        }
        return MB_OK;
    }

    int set_alpha(Ext2 alpha) {
        std::vector<uint64_t>& pows = pows_;
        pows.resize(2 * (size_t)K_);
        gl::E2 p{1, 0}, a{gl::canon(alpha.c0), gl::canon(alpha.c1)};
        for (int k = 0; k < K_; k++) {
            pows[2 * k] = p.c0;
            pows[2 * k + 1] = p.c1;
            p = gl::e2_canon(gl::e2_mul(p, a));
        }
        MB_CUDA(cudaMemcpyAsync(alpha_dev_, pows.data(), 16 * (size_t)K_, cudaMemcpyHostToDevice, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        have_alpha_ = true;
        return MB_OK;
    }

    // Local share of m(0..3) for the current round.
    int round_message(uint64_t* h_msg) {
        if (!have_alpha_ || round_ >= n_loc_) return MB_ERR_ARG;
        if (round_ == 0) {
            // sum_k alpha^k m_k(c) from the per-instance messages
            int rc = instance_messages();
            if (rc != MB_OK) return rc;
            gl::E2 acc[4] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};
            for (int k = 0; k < K_; k++) {
                gl::E2 m[4];
                expand_message(inst_.data() + 2 * bt::NC * (size_t)k, 0, m);
                const gl::E2 w{pows_[2 * k], pows_[2 * k + 1]};
                for (int c = 0; c < 4; c++) acc[c] = gl::e2_add(acc[c], gl::e2_mul(w, m[c]));
            }
            for (int c = 0; c < 4; c++) {
                acc[c] = gl::e2_canon(acc[c]);
                h_msg[2 * c] = acc[c].c0;
                h_msg[2 * c + 1] = acc[c].c1;
            }
            return MB_OK;
        }
        if (!have_msg_) return MB_ERR_ARG;
        uint64_t* h = landing_;
        if (h) {
            // the fold kernel's last block wrote the six words straight into pinned host memory
            MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        } else {
            h = pinned_scratch();   // the calling thread's landing zone, not the creating thread's
            if (!h) return MB_ERR_CUDA;
            MB_CUDA(cudaMemcpyAsync(h, msg_dev_, 16 * bt::NC, cudaMemcpyDeviceToHost, MB_STREAM));
            MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        }
        gl::E2 m[4];
        expand_message(h, round_, m);
        for (int c = 0; c < 4; c++) {
            h_msg[2 * c] = m[c].c0;
            h_msg[2 * c + 1] = m[c].c1;
        }
        return MB_OK;
    }

    int fold(Ext2 ch) {
        if (!have_alpha_ || round_ >= n_loc_) return MB_ERR_ARG;
        gl::E2 r{gl::canon(ch.c0), gl::canon(ch.c1)};
        size_t live = n_ >> round_, quarter = live / 4;
        bool first = round_ == 0;
        const uint64_t* eq_in = first ? eq0_ : eq_cur_;
        const uint64_t* ab_in = first ? a0_ : ab_cur_;
        size_t stride_in = first ? n_ : ab_stride_;
        bool to_a = first || ab_cur_ == ab_b_;
        uint64_t* eq_out = to_a ? eq_a_ : eq_b_;
        uint64_t* ab_out = to_a ? ab_a_ : ab_b_;
        size_t stride_out = to_a ? n_ / 2 : (n_ >= 4 ? n_ / 4 : 1);
        if (quarter >= 1) {
            int grid = grid_for(quarter, 256, 4);
            if (first) {
                // per instance: alpha^k and alpha^k r
                std::vector<uint64_t> wt(4 * (size_t)K_);
                for (int k = 0; k < K_; k++) {
                    gl::E2 w{pows_[2 * k], pows_[2 * k + 1]}, wr = gl::e2_canon(gl::e2_mul(w, r));
                    wt[4 * k] = w.c0; wt[4 * k + 1] = w.c1; wt[4 * k + 2] = wr.c0; wt[4 * k + 3] = wr.c1;
                }
                MB_CUDA(cudaMemcpyAsync(wtab_dev_, wt.data(), sizeof(uint64_t) * wt.size(), cudaMemcpyHostToDevice, MB_STREAM));
                MB_CUDA(cudaStreamSynchronize(MB_STREAM));  // wt leaves scope
            }
            MB_KERNEL("batched_fold_message");
            uint64_t* msg_out = landing_ ? landing_ : msg_dev_;
            if (first)
                bt::fold_message_kernel<true><<<grid, 256, 0, MB_STREAM>>>(
                    eq_in, eq_out, ab_in, b0_, ab_out, wtab_dev_, r, K_, stride_in, stride_out, quarter, partial_, counter_, msg_out);
            else
                bt::fold_message_kernel<false><<<grid, 256, 0, MB_STREAM>>>(
                    eq_in, eq_out, ab_in, b0_, ab_out, wtab_dev_, r, K_, stride_in, stride_out, quarter, partial_, counter_, msg_out);
            have_msg_ = true;
        } else {
            MB_KERNEL("batched_final_fold");
            int threads = 2 * K_ + 1;
            if (first)
                bt::final_fold_kernel<GlBase, GlExt2, true><<<(threads + 127) / 128, 128, 0, MB_STREAM>>>(
                    eq_in, eq_out, ab_in, b0_, ab_out, alpha_dev_, r, K_, stride_in, stride_out);
            else
                bt::final_fold_kernel<GlBase, GlExt2, false><<<(threads + 127) / 128, 128, 0, MB_STREAM>>>(
                    eq_in, eq_out, ab_in, b0_, ab_out, alpha_dev_, r, K_, stride_in, stride_out);
            have_msg_ = false;
        }
        if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
        eq_cur_ = eq_out;
        ab_cur_ = ab_out;
        ab_stride_ = stride_out;
        round_++;
        return MB_OK;
    }

    // Round messages land in `pinned` (six words of page-locked host memory of the calling thread) instead of
    // being copied back: a round is then one launch and one stream synchronisation. Used by the whole-proof loop,
    // which stays on one thread; the per-round C-ABI keeps the copy because its callers may change threads.
    void set_landing(uint64_t* pinned) { landing_ = pinned; }

    // After n_loc folds: eq, then alpha^k a_k, b_k for every k: (2K + 1) extension elements.
    int finals(uint64_t* h_out) {
        if (round_ != n_loc_) return MB_ERR_ARG;
        MB_CUDA(cudaMemcpyAsync(h_out, eq_cur_, 16, cudaMemcpyDeviceToHost, MB_STREAM));
        for (int t = 0; t < 2 * K_; t++) {
            int k = t >> 1, which = t & 1;  // output order: a'_0 .. a'_{K-1}, b_0 .. b_{K-1}
            uint64_t* dst = h_out + 2 + 2 * (size_t)(which * K_ + k);
            MB_CUDA(cudaMemcpyAsync(dst, ab_cur_ + (size_t)t * ab_stride_ * 2, 16, cudaMemcpyDeviceToHost, MB_STREAM));
        }
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        return MB_OK;
    }

private:
    void release() {
        pool_free(eq0_); pool_free(eq_a_); pool_free(eq_b_); pool_free(ab_a_); pool_free(ab_b_);
        pool_free(partial_); pool_free(small_);
        eq0_ = eq_a_ = eq_b_ = ab_a_ = ab_b_ = partial_ = small_ = nullptr;
    }
    int K_ = 0, Kp_ = 1, n_loc_ = 0, round_ = 0, grid_max_ = 0, grid_inst_ = 0;
    bool have_inst_ = false;
    std::vector<uint64_t> inst_, pows_, pt_;
    uint64_t *wtab_dev_ = nullptr, *inst_dev_ = nullptr;
    size_t n_ = 0, ab_stride_ = 0;
    bool have_msg_ = false, have_alpha_ = false;
    const uint64_t *a0_ = nullptr, *b0_ = nullptr;
    uint64_t *eq0_ = nullptr, *eq_a_ = nullptr, *eq_b_ = nullptr, *ab_a_ = nullptr, *ab_b_ = nullptr;
    uint64_t *partial_ = nullptr, *small_ = nullptr, *msg_dev_ = nullptr, *alpha_dev_ = nullptr, *eq_cur_ = nullptr, *ab_cur_ = nullptr;
    unsigned int* counter_ = nullptr;
    uint64_t* landing_ = nullptr;
};

}  // namespace mbhost


// ---- one proof over `world` shards: round loop, recombination, transcript and the last log2(world) rounds ----
namespace {

using gl::E2;
inline E2 e2c(E2 a) { return gl::e2_canon(a); }
inline E2 e2_load(const uint64_t* w) { return E2{gl::canon(w[0]), gl::canon(w[1])}; }

// Sum over the ranks of `width` extension elements each (rank-major words).
void sum_shares(const uint64_t* all, int world, int width, E2* out) {
    for (int i = 0; i < width; i++) {
        E2 t{0, 0};
        for (int g = 0; g < world; g++) t = gl::e2_add(t, e2_load(all + ((size_t)g * width + i) * 2));
        out[i] = e2c(t);
    }
}

struct RoundClock {
    bool on = std::getenv("MB_SHARD_TIMING") != nullptr;
    std::chrono::steady_clock::time_point t0;
    double kernel = 0, gather = 0, host = 0;
    void start() { if (on) t0 = std::chrono::steady_clock::now(); }
    void stop(double& acc) {
        if (!on) return;
        auto t1 = std::chrono::steady_clock::now();
        acc += std::chrono::duration<double, std::micro>(t1 - t0).count();
        t0 = t1;
    }
};

}  // namespace

namespace mbhost {

// Every rank passes its slices; all outputs are identical on every rank.
int batched_prove_sharded(const mb_exchange* ex, const uint64_t* d_a, const uint64_t* d_b, int K, int num_vars,
                          const uint64_t* h_point, const uint8_t* label, size_t label_len, uint64_t* h_claims,
                          uint64_t* h_alpha, uint64_t* h_round_msgs, uint64_t* h_challenges, uint64_t* h_finals,
                          uint64_t* h_final_eval, uint64_t* h_transcript_state, double* h_round_us) {
    if (!ex || !d_a || !d_b || !h_point || (!label && label_len) || K < 1 || K > bt::MAX_K) return MB_ERR_ARG;
    const int world = ex->world, rank = ex->rank;
    int g_bits = 0;
    while ((1 << g_bits) < world) g_bits++;
    if (world < 1 || (1 << g_bits) != world || rank < 0 || rank >= world) return MB_ERR_ARG;
    const int n_loc = num_vars - g_bits;
    if (n_loc < 1 || n_loc > 34) return MB_ERR_UNSUPPORTED;

    // eq(t_top, rank): bit i of the rank pairs with coordinate n_loc + i
    E2 scale{1, 0};
    for (int i = 0; i < g_bits; i++) {
        const E2 t = e2_load(h_point + 2 * (size_t)(n_loc + i));
        scale = e2c(gl::e2_mul(scale, (rank >> i) & 1 ? t : gl::e2_sub(E2{1, 0}, t)));
    }
    const uint64_t scale_w[2] = {scale.c0, scale.c1};
    uint64_t* pin = pinned_scratch();
    if (!pin) return MB_ERR_CUDA;

    BatchedEqAbState st;
    int rc = st.init(d_a, d_b, h_point, scale_w, K, n_loc);
    if (rc != MB_OK) return rc;
    st.set_landing(pin);

    const int T = 2 * K + 1;
    std::vector<uint64_t> mine((size_t)2 * (T > 4 ? T : 4)), all((size_t)world * mine.size());
    std::vector<E2> claims(K);
    Transcript tr(label, label_len);
    tr.append_u64("sp_num_var", (uint64_t)num_vars);
    tr.append_u64("sp_num_inst", (uint64_t)K);
    rc = st.claims(mine.data());
    if (rc != MB_OK) return rc;
    rc = ex->all_gather_host(ex->ctx, mine.data(), 2 * (size_t)K, all.data());
    if (rc != MB_OK) return rc;
    sum_shares(all.data(), world, K, claims.data());
    for (int k = 0; k < K; k++) {
        tr.append_ext2("sp_y_i", Ext2{claims[k].c0, claims[k].c1});
        if (h_claims) { h_claims[2 * k] = claims[k].c0; h_claims[2 * k + 1] = claims[k].c1; }
    }
    const Ext2 alpha = tr.challenge_ext2("sp_alpha");
    if (h_alpha) { h_alpha[0] = alpha.c0; h_alpha[1] = alpha.c1; }
    rc = st.set_alpha(alpha);
    if (rc != MB_OK) return rc;

    RoundClock clock;
    int round = 0;
    bool label_absorbed = false;   // the first label of a round goes in while the round's kernel runs
    auto publish = [&](const E2* msg) {
        for (int c = 0; c < 4; c++) {
            if (c > 0 || !label_absorbed) tr.begin_append("sp_round_msg");
            tr.finish_append_ext2(Ext2{msg[c].c0, msg[c].c1});
            if (h_round_msgs) {
                h_round_msgs[(size_t)round * 8 + 2 * c] = msg[c].c0;
                h_round_msgs[(size_t)round * 8 + 2 * c + 1] = msg[c].c1;
            }
        }
        const Ext2 r = tr.challenge_ext2("sp_round_challenge");
        if (h_challenges) { h_challenges[2 * (size_t)round] = r.c0; h_challenges[2 * (size_t)round + 1] = r.c1; }
        round++;
        label_absorbed = false;
        return r;
    };
    for (int i = 0; i < n_loc; i++) {
        clock.start();
        rc = st.round_message(mine.data());
        if (rc != MB_OK) return rc;
        clock.stop(clock.kernel);
        E2 msg[4];
        if (world > 1) {
            rc = ex->all_gather_host(ex->ctx, mine.data(), 8, all.data());
            if (rc != MB_OK) return rc;
            clock.stop(clock.gather);
            sum_shares(all.data(), world, 4, msg);
        } else {
            for (int c = 0; c < 4; c++) msg[c] = e2_load(mine.data() + 2 * c);
        }
        const Ext2 r = publish(msg);
        clock.stop(clock.host);
        rc = st.fold(r);
        if (rc != MB_OK) return rc;
        if (round < num_vars) {
            tr.begin_append("sp_round_msg");
            label_absorbed = true;
        }
    }
    // one value per table and rank: eq, alpha^k a_k, b_k; the top variables are finished on the host
    clock.start();
    rc = st.finals(mine.data());
    if (rc != MB_OK) return rc;
    clock.stop(clock.kernel);
    rc = ex->all_gather_host(ex->ctx, mine.data(), 2 * (size_t)T, all.data());
    if (rc != MB_OK) return rc;
    clock.stop(clock.gather);
    std::vector<std::vector<E2>> tab(T, std::vector<E2>(world));
    for (int g = 0; g < world; g++)
        for (int i = 0; i < T; i++) tab[i][g] = e2_load(all.data() + ((size_t)g * T + i) * 2);
    for (int size = world; size > 1; size /= 2) {
        const int half = size / 2;
        E2 msg[4];
        for (int c = 0; c < 4; c++) {
            const E2 cc{(uint64_t)c, 0};
            E2 tot{0, 0};
            for (int y = 0; y < half; y++) {
                auto at = [&](const std::vector<E2>& t) {
                    return e2c(gl::e2_add(t[2 * y], gl::e2_mul(cc, gl::e2_sub(t[2 * y + 1], t[2 * y]))));
                };
                E2 inner{0, 0};
                for (int k = 0; k < K; k++) inner = gl::e2_add(inner, gl::e2_mul(at(tab[1 + k]), at(tab[1 + K + k])));
                tot = gl::e2_add(tot, gl::e2_mul(at(tab[0]), e2c(inner)));
            }
            msg[c] = e2c(tot);
        }
        const Ext2 rr = publish(msg);
        const E2 r{rr.c0, rr.c1};
        for (auto& t : tab)
            for (int y = 0; y < half; y++) t[y] = e2c(gl::e2_add(t[2 * y], gl::e2_mul(r, gl::e2_sub(t[2 * y + 1], t[2 * y]))));
    }
    // a_k(R) is reported without the alpha^k factor the shards carry
    std::vector<E2> fin(T);
    fin[0] = tab[0][0];
    E2 pw{1, 0}, acc{0, 0};
    const E2 al{alpha.c0, alpha.c1};
    for (int k = 0; k < K; k++) {
        fin[1 + k] = e2c(gl::e2_mul(tab[1 + k][0], gl::e2_inv(pw)));
        acc = gl::e2_add(acc, gl::e2_mul(tab[1 + k][0], tab[1 + K + k][0]));
        pw = e2c(gl::e2_mul(pw, al));
        fin[1 + K + k] = tab[1 + K + k][0];
    }
    for (int i = 0; i < T; i++) {
        tr.append_ext2("sp_f_eval", Ext2{fin[i].c0, fin[i].c1});
        if (h_finals) { h_finals[2 * i] = fin[i].c0; h_finals[2 * i + 1] = fin[i].c1; }
    }
    const E2 fe = e2c(gl::e2_mul(tab[0][0], e2c(acc)));
    if (h_final_eval) { h_final_eval[0] = fe.c0; h_final_eval[1] = fe.c1; }
    if (h_transcript_state) std::memcpy(h_transcript_state, tr.state(), 64);
    clock.stop(clock.host);
    if (h_round_us) {
        // what the local rounds cost besides their kernels, per round: exchange, recombination and transcript
        h_round_us[0] = clock.on ? clock.kernel / (n_loc + 1) : -1.0;
        h_round_us[1] = clock.on ? clock.gather / (n_loc + 1) : -1.0;
        h_round_us[2] = clock.on ? clock.host / (n_loc + 1) : -1.0;
    }
    return MB_OK;
}

}  // namespace mbhost

using mbhost::BatchedEqAbState;
using mbhost::Ext2;
using mbhost::Transcript;

extern "C" {

// ---- one shard of the batched eq * a_k * b_k sumcheck ----
// d_a, d_b: [K][2^n_loc] base-field slices (read in place until the first fold, never written); h_point_low: n_loc (c0, c1) pairs (the
// shard-local coordinates of the eq point); h_eq_scale: eq of the top coordinates
// at this shard's index ((1, 0) for a single shard).
int gl_batched_state_create(const uint64_t* d_a, const uint64_t* d_b, const uint64_t* h_point_low,
                            const uint64_t* h_eq_scale, int K, int n_loc, void** state) {
    if (!state) return MB_ERR_ARG;
    auto* s = new BatchedEqAbState;
    int rc = s->init(d_a, d_b, h_point_low, h_eq_scale, K, n_loc);
    if (rc != MB_OK) { delete s; return rc; }
    *state = s;
    return MB_OK;
}
int gl_batched_state_destroy(void* state) { delete static_cast<BatchedEqAbState*>(state); return MB_OK; }
int gl_batched_state_claims(void* state, uint64_t* h_claims) { return static_cast<BatchedEqAbState*>(state)->claims(h_claims); }
int gl_batched_state_set_alpha(void* state, uint64_t c0, uint64_t c1) { return static_cast<BatchedEqAbState*>(state)->set_alpha(Ext2{c0, c1}); }
int gl_batched_state_round_message(void* state, uint64_t* h_msg) { return static_cast<BatchedEqAbState*>(state)->round_message(h_msg); }
int gl_batched_state_fold(void* state, uint64_t c0, uint64_t c1) { return static_cast<BatchedEqAbState*>(state)->fold(Ext2{c0, c1}); }
int gl_batched_state_finals(void* state, uint64_t* h_out) { return static_cast<BatchedEqAbState*>(state)->finals(h_out); }

// ---- the whole proof over the shards of an exchange (world = 1: an mb_exchange_local_create(1) object) ----
// d_a, d_b: this rank's slices [K][2^(num_vars - log2 world)]; h_point: num_vars (c0, c1) pairs, the same on every
// rank. Outputs (each may be null), identical on every rank: claims [K][2], alpha [2], round messages
// [num_vars][4][2], challenges [num_vars][2], finals [2K + 1][2] (eq, a_k, b_k at the challenge point), final
// evaluation [2], transcript state [8]; h_round_us [3]: with MB_SHARD_TIMING set, microseconds per local round spent
// waiting for the kernel, in the exchange, and on the host (recombination and transcript); -1 otherwise.
int gl_batched_prove_sharded(const mb_exchange* ex, const uint64_t* d_a, const uint64_t* d_b, int K, int num_vars,
                             const uint64_t* h_point, const uint8_t* label, size_t label_len, uint64_t* h_claims,
                             uint64_t* h_alpha, uint64_t* h_round_msgs, uint64_t* h_challenges, uint64_t* h_finals,
                             uint64_t* h_final_eval, uint64_t* h_transcript_state, double* h_round_us) {
    return mbhost::batched_prove_sharded(ex, d_a, d_b, K, num_vars, h_point, label, label_len, h_claims, h_alpha, h_round_msgs,
                                         h_challenges, h_finals, h_final_eval, h_transcript_state, h_round_us);
}

// ---- host transcript ----
int gl_transcript_create(const uint8_t* label, size_t label_len, void** transcript) {
    if (!transcript) return MB_ERR_ARG;
    *transcript = new Transcript(label, label_len);
    return MB_OK;
}
int gl_transcript_destroy(void* t) { delete static_cast<Transcript*>(t); return MB_OK; }
int gl_transcript_append_u64(void* t, const char* label, uint64_t v) { static_cast<Transcript*>(t)->append_u64(label, v); return MB_OK; }
int gl_transcript_append_ext2(void* t, const char* label, uint64_t c0, uint64_t c1) {
    static_cast<Transcript*>(t)->append_ext2(label, Ext2{c0, c1});
    return MB_OK;
}
int gl_transcript_challenge_ext2(void* t, const char* label, uint64_t* out2) {
    Ext2 r = static_cast<Transcript*>(t)->challenge_ext2(label);
    out2[0] = r.c0;
    out2[1] = r.c1;
    return MB_OK;
}
int gl_transcript_state(const void* t, uint64_t* out8) { std::memcpy(out8, static_cast<const Transcript*>(t)->state(), 64); return MB_OK; }

// Verifier of the batched eq * a * b proof on the host (no device call): replays the transcript of
// gl_batched_prove_sharded, checks P(0) + P(1) against the running claim in every round (the first claim is
// sum_k alpha^k y_k), takes P(r) by interpolation on 0..3 as the next claim, and at the end checks that the last
// claim equals eq(R) sum_k alpha^k a_k(R) b_k(R) and that the revealed eq(R) is the eq polynomial of h_point at the
// challenges (round i binds variable i). The revealed a_k(R), b_k(R) are the openings the caller checks against its
// commitments. h_claims [K][2], h_round_msgs [num_vars][4][2], h_finals [2K + 1][2]; h_challenges [num_vars][2]
// (may be null) receives the challenges. *ok = 1 when accepted.
int gl_batched_verify_host(int K, int num_vars, const uint64_t* h_point, const uint8_t* label, size_t label_len,
                           const uint64_t* h_claims, const uint64_t* h_round_msgs, const uint64_t* h_finals,
                           uint64_t* h_challenges, int* ok) {
    using namespace mbhost;
    if (K < 1 || num_vars < 1 || num_vars > 40 || !h_point || !h_claims || !h_round_msgs || !h_finals || !ok || (!label && label_len))
        return MB_ERR_ARG;
    *ok = 0;
    Transcript tr(label, label_len);
    tr.append_u64("sp_num_var", (uint64_t)num_vars);
    tr.append_u64("sp_num_inst", (uint64_t)K);
    for (int k = 0; k < K; k++) tr.append_ext2("sp_y_i", Ext2{gl::canon(h_claims[2 * k]), gl::canon(h_claims[2 * k + 1])});
    const Ext2 a = tr.challenge_ext2("sp_alpha");
    const E2 alpha{a.c0, a.c1};
    E2 claim{0, 0}, pw{1, 0};
    for (int k = 0; k < K; k++) {
        claim = e2c(gl::e2_add(claim, gl::e2_mul(pw, e2_load(h_claims + 2 * k))));
        pw = e2c(gl::e2_mul(pw, alpha));
    }
    // 1 / ((c - 0)(c - 1)...(c - 3)) without the factor c - c, for c = 0..3: -1/6, 1/2, -1/2, 1/6
    const uint64_t inv2 = gl::canon(gl::inv(2)), inv6 = gl::canon(gl::inv(6));
    const uint64_t wgt[4] = {gl::canon(gl::sub(0, inv6)), inv2, gl::canon(gl::sub(0, inv2)), inv6};
    E2 eq_at_r{1, 0};
    for (int round = 0; round < num_vars; round++) {
        E2 msg[4];
        for (int c = 0; c < 4; c++) msg[c] = e2_load(h_round_msgs + (size_t)round * 8 + 2 * c);
        const E2 sum = e2c(gl::e2_add(msg[0], msg[1]));
        if (sum.c0 != claim.c0 || sum.c1 != claim.c1) return MB_OK;
        for (int c = 0; c < 4; c++) tr.append_ext2("sp_round_msg", Ext2{msg[c].c0, msg[c].c1});
        const Ext2 rr = tr.challenge_ext2("sp_round_challenge");
        const E2 r{rr.c0, rr.c1};
        if (h_challenges) { h_challenges[2 * round] = r.c0; h_challenges[2 * round + 1] = r.c1; }
        // P(r) = sum_c P(c) w_c prod_{k != c} (r - k)
        E2 next{0, 0};
        for (int c = 0; c < 4; c++) {
            E2 num{wgt[c], 0};
            for (int k = 0; k < 4; k++)
                if (k != c) num = e2c(gl::e2_mul(num, gl::e2_sub(r, E2{(uint64_t)k, 0})));
            next = gl::e2_add(next, gl::e2_mul(msg[c], num));
        }
        claim = e2c(next);
        // eq factor of variable `round`: p r + (1 - p)(1 - r)
        const E2 p = e2_load(h_point + 2 * round), one{1, 0};
        const E2 f = gl::e2_add(gl::e2_mul(p, r), gl::e2_mul(gl::e2_sub(one, p), gl::e2_sub(one, r)));
        eq_at_r = e2c(gl::e2_mul(eq_at_r, e2c(f)));
    }
    const int T = 2 * K + 1;
    for (int i = 0; i < T; i++) tr.append_ext2("sp_f_eval", Ext2{gl::canon(h_finals[2 * i]), gl::canon(h_finals[2 * i + 1])});
    const E2 eq_rev = e2_load(h_finals);
    if (eq_rev.c0 != eq_at_r.c0 || eq_rev.c1 != eq_at_r.c1) return MB_OK;
    E2 acc{0, 0};
    pw = E2{1, 0};
    for (int k = 0; k < K; k++) {
        acc = e2c(gl::e2_add(acc, gl::e2_mul(pw, e2c(gl::e2_mul(e2_load(h_finals + 2 * (1 + k)), e2_load(h_finals + 2 * (1 + K + k)))))));
        pw = e2c(gl::e2_mul(pw, alpha));
    }
    const E2 last = e2c(gl::e2_mul(eq_rev, acc));
    *ok = last.c0 == claim.c0 && last.c1 == claim.c1;
    return MB_OK;
}


}  // extern "C"
