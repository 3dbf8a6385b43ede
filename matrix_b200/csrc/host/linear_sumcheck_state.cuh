// State object of the linear (product of d tables) sumcheck prover, shared by the
// Goldilocks and the almost-Goldilocks host layers: the per-round API of the
// reference's Rust drivers
//
//   GpuSumcheckStateExt2   goldilocks-cuda-rs/src/sumcheck_prover.rs:206-436
//                          almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:127-436
//
// (compute_round_message, fold, final_evaluations). Two things differ in how the
// work is done, not in what comes out:
//  * base-field tables are not widened on upload; round 0 runs on the 8-byte
//    tables and the first fold lifts them with the extension challenge;
//  * fold(r) also accumulates the next round's message in the same pass, and
//    the block partials are summed on the device, so compute_round_message()
//    after a fold only reads (d+1) extension elements back.
// Base / Ext are the field traits of sumcheck_kernels.cuh (GlBase, GlExt2) or
// agl_traits.cuh (AglBase, AglExt2).
//  * once a table is down to host_tail(d) elements the live tables are read back and the remaining rounds run on
//    the host: a round on the device costs a launch and a synchronisation (about 20 us) whatever its size, the
//    same round on a few hundred elements takes a host core less (about 7 ns per extension product). The field
//    arithmetic is exact, so the messages are the same words.
#pragma once
#include <vector>
#include "../agl_field.cuh"
#include "../gl_sumcheck_launch.cuh"
#include "ext2_words.hpp"
#include "host_field.hpp"

namespace mbhost {

using namespace mb;
using namespace mb::sc;

// Host-side extension arithmetic for the tail rounds, by element type: canonical words in and out (the tables are
// made canonical when they come to the host), through the host forms of host_field.hpp.
template <class T> struct HostExt;
template <class T, class F> struct HostExtOps {
    static T add(T a, T b) { return T{F::add(a.c0, b.c0), F::add(a.c1, b.c1)}; }
    static T sub(T a, T b) { return T{F::sub(a.c0, b.c0), F::sub(a.c1, b.c1)}; }
    static T mul(T a, T b) {
        T r;
        hf::e2_mul<F>(a.c0, a.c1, b.c0, b.c1, r.c0, r.c1);
        return r;
    }
    static T canon(T a) { return T{F::canon(a.c0), F::canon(a.c1)}; }
};
template <> struct HostExt<gl::E2> : HostExtOps<gl::E2, hf::GlE2Ops> {};
template <> struct HostExt<agl::E2> : HostExtOps<agl::E2, hf::AglE2Ops> {};

// Live elements per table at which the rounds move to the host: a host round costs live / 2 x (d^2 - 1 + d)
// extension products, about 9 us at 512 elements of two tables and 10 us at 256 elements of three.
inline size_t host_tail(int d) { return d <= 2 ? 512 : 256; }

template <class Base, class Ext>
class LinearSumcheckState {
public:
    ~LinearSumcheckState() { release(); }

    // d tables of 2^num_vars elements, poly-major, already on the device
    // (base field: u64 each; extension: (c0, c1) each). The tables are read in
    // place and never written.
    int init_device(const uint64_t* d_tables, int d, int num_vars, bool base_field) {
        if (d < 1 || d > MAX_D || num_vars < 0 || num_vars > 40 || !d_tables) return MB_ERR_ARG;
        d_ = d;
        num_vars_ = num_vars;
        n_ = (size_t)1 << num_vars;
        base_ = base_field;
        src_ = d_tables;
        round_ = 0;
        cur_ = nullptr;
        host_mode_ = false;
        size_t cap_a = n_ >= 2 ? n_ / 2 : 1, cap_b = n_ >= 4 ? n_ / 4 : 1;
        stride_a_ = cap_a;
        stride_b_ = cap_b;
        MB_CUDA(pool_alloc((void**)&buf_a_, sizeof(uint64_t) * 2 * cap_a * d));
        MB_CUDA(pool_alloc((void**)&buf_b_, sizeof(uint64_t) * 2 * cap_b * d));
        max_blocks_ = prover_grid(n_ / 2 > 0 ? n_ / 2 : 1);
        MB_CUDA(pool_alloc((void**)&partial_, sizeof(uint64_t) * 2 * (d + 1) * (size_t)max_blocks_));
        MB_CUDA(pool_alloc((void**)&counter_, sizeof(unsigned int)));
        MB_CUDA(cudaMemsetAsync(counter_, 0, sizeof(unsigned int), MB_STREAM));
        // The finished message is written by the last block of a kernel straight into pinned host memory
        // (device-addressable under unified addressing), so a round costs one stream synchronisation and no
        // copy call.
        msg_host_ = pinned_scratch();
        if (!msg_host_) return MB_ERR_CUDA;
        msg_dev_ = msg_host_;
        have_msg_ = false;
        return MB_OK;
    }

    // Evaluations P(0..d) of the current round polynomial, canonical.
    int compute_round_message(std::vector<Ext2>& out) {
        if (round_ >= num_vars_) return MB_ERR_ARG;
        size_t live = n_ >> round_, half = live / 2;
        if (host_mode_) return host_message(out, half);
        if (!have_msg_) {
            // Only round 0 gets here: every fold leaves the next message behind.
            int grid = prover_grid(half);
            int rc;
            if (base_) {
                rc = launch_round_message<Base>(src_, partial_, d_, n_, half, grid, MB_STREAM, counter_, msg_dev_);
            } else {
                rc = launch_round_message<Ext>(src_, partial_, d_, n_, half, grid, MB_STREAM, counter_, msg_dev_);
            }
            if (rc != MB_OK) return rc;
            msg_words_ = base_ ? 1 : 2;
        }
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        out.resize(d_ + 1);
        for (int c = 0; c <= d_; c++) {
            if (msg_words_ == 1) {
                out[c].c0 = msg_host_[c];
                out[c].c1 = 0;
            } else {
                out[c].c0 = msg_host_[2 * c];
                out[c].c1 = msg_host_[2 * c + 1];
            }
        }
        return MB_OK;
    }

    // Fold every table on `challenge`; leaves the next round's message ready.
    int fold(Ext2 challenge) {
        if (round_ >= num_vars_) return MB_ERR_ARG;
        size_t live = n_ >> round_, half = live / 2, quarter = live / 4;
        const typename Ext::WordCanon canon;
        typename Ext::T r{canon(challenge.c0), canon(challenge.c1)};
        if (!host_mode_ && round_ >= 1 && live <= host_tail(d_)) {
            int rc = to_host(live);
            if (rc != MB_OK) return rc;
        }
        if (host_mode_) {
            using H = HostExt<typename Ext::T>;
            for (int i = 0; i < d_; i++) {
                typename Ext::T* t = host_tab_.data() + (size_t)i * host_stride_;
                for (size_t j = 0; j < half; j++) t[j] = H::canon(H::add(t[2 * j], H::mul(r, H::sub(t[2 * j + 1], t[2 * j]))));
            }
            round_++;
            return MB_OK;
        }
        const uint64_t* in = round_ == 0 ? src_ : cur_;
        size_t stride_in = round_ == 0 ? n_ : cur_stride_;
        bool to_a = (round_ == 0) || (cur_ == buf_b_);
        uint64_t* out = to_a ? buf_a_ : buf_b_;
        size_t stride_out = to_a ? stride_a_ : stride_b_;
        bool in_base = base_ && round_ == 0;
        int rc;
        if (quarter >= 1) {
            int grid = prover_grid(quarter);
            if (in_base) {
                rc = launch_fold_message<Base, Ext>(in, out, r, nullptr, d_, stride_in, stride_out, quarter,
                                                         partial_, grid, MB_STREAM, counter_, msg_dev_);
            } else {
                rc = launch_fold_message<Ext, Ext>(in, out, r, nullptr, d_, stride_in, stride_out, quarter,
                                                         partial_, grid, MB_STREAM, counter_, msg_dev_);
            }
            have_msg_ = true;
            msg_words_ = 2;
        } else {
            if (in_base) {
                rc = launch_fold_lift<Base, Ext>(in, out, r, nullptr, d_, stride_in, stride_out, half, MB_STREAM);
            } else {
                rc = launch_fold_lift<Ext, Ext>(in, out, r, nullptr, d_, stride_in, stride_out, half, MB_STREAM);
            }
            have_msg_ = false;
        }
        if (rc != MB_OK) return rc;
        cur_ = out;
        cur_stride_ = stride_out;
        round_++;
        return MB_OK;
    }

    // One value per table once every variable is bound.
    int final_evaluations(std::vector<Ext2>& out) {
        if (round_ != num_vars_) return MB_ERR_ARG;
        out.resize(d_);
        if (host_mode_) {
            for (int i = 0; i < d_; i++) {
                const typename Ext::T v = host_tab_[(size_t)i * host_stride_];
                out[i].c0 = v.c0;
                out[i].c1 = v.c1;
            }
            return MB_OK;
        }
        for (int i = 0; i < d_; i++) {
            uint64_t w[2] = {0, 0};
            if (num_vars_ == 0) {
                const uint64_t* p = base_ ? src_ + i : src_ + 2 * (size_t)i;
                MB_CUDA(cudaMemcpyAsync(w, p, base_ ? 8 : 16, cudaMemcpyDeviceToHost, MB_STREAM));
            } else {
                MB_CUDA(cudaMemcpyAsync(w, cur_ + 2 * (size_t)i * cur_stride_, 16, cudaMemcpyDeviceToHost, MB_STREAM));
            }
            MB_CUDA(cudaStreamSynchronize(MB_STREAM));
            const typename Ext::WordCanon canon;
            out[i].c0 = canon(w[0]);
            out[i].c1 = canon(w[1]);
        }
        return MB_OK;
    }

    int num_vars() const { return num_vars_; }
    int num_polys() const { return d_; }
    int current_round() const { return round_; }

private:
    // The live elements of the (extension) tables come to the host; the rounds continue there.
    int to_host(size_t live) {
        host_stride_ = live;
        host_tab_.resize((size_t)d_ * live);
        for (int i = 0; i < d_; i++)
            MB_CUDA(cudaMemcpyAsync(host_tab_.data() + (size_t)i * live, cur_ + 2 * (size_t)i * cur_stride_, 16 * live,
                                    cudaMemcpyDeviceToHost, MB_STREAM));
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        const typename Ext::WordCanon canon;
        for (auto& v : host_tab_) v = typename Ext::T{canon(v.c0), canon(v.c1)};
        host_mode_ = true;
        have_msg_ = false;
        return MB_OK;
    }
    // P(c) = sum_j prod_i (t_i[2j] + c (t_i[2j+1] - t_i[2j])), c = 0..d, on the host tables.
    int host_message(std::vector<Ext2>& out, size_t half) {
        using H = HostExt<typename Ext::T>;
        using T = typename Ext::T;
        std::vector<T> acc(d_ + 1, T{0, 0});
        T val[MAX_D], diff[MAX_D];
        for (size_t j = 0; j < half; j++) {
            for (int i = 0; i < d_; i++) {
                const T* t = host_tab_.data() + (size_t)i * host_stride_;
                val[i] = t[2 * j];
                diff[i] = H::sub(t[2 * j + 1], t[2 * j]);
            }
            for (int c = 0; c <= d_; c++) {
                T p = val[0];
                for (int i = 1; i < d_; i++) p = H::mul(p, val[i]);
                acc[c] = H::add(acc[c], p);
                for (int i = 0; i < d_; i++) val[i] = H::add(val[i], diff[i]);
            }
        }
        out.resize(d_ + 1);
        for (int c = 0; c <= d_; c++) {
            const T v = H::canon(acc[c]);
            out[c].c0 = v.c0;
            out[c].c1 = v.c1;
        }
        return MB_OK;
    }

    void release() {
        pool_free(buf_a_);
        pool_free(buf_b_);
        pool_free(partial_);
        pool_free(counter_);
        buf_a_ = buf_b_ = partial_ = msg_dev_ = nullptr;
        counter_ = nullptr;
        msg_host_ = nullptr;
    }

    int d_ = 0, num_vars_ = 0, round_ = 0, max_blocks_ = 0, msg_words_ = 2;
    size_t n_ = 0, stride_a_ = 0, stride_b_ = 0, cur_stride_ = 0;
    bool base_ = false, have_msg_ = false;
    const uint64_t* src_ = nullptr;
    uint64_t *buf_a_ = nullptr, *buf_b_ = nullptr, *cur_ = nullptr, *partial_ = nullptr, *msg_dev_ = nullptr;
    unsigned int* counter_ = nullptr;
    uint64_t* msg_host_ = nullptr;
    bool host_mode_ = false;
    size_t host_stride_ = 0;
    std::vector<typename Ext::T> host_tab_;
};

}  // namespace mbhost
