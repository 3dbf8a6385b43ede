// Host-side Fiat-Shamir transcript over Goldilocks: a duplex sponge on
// Poseidon2 width 8, rate 4, overwrite mode.
//
// Mirrors the reference's `Transcript` (zk-torch-3/src/transcript.rs:174-350):
// same method names, same absorb/squeeze order, same label rule (length, then
// bytes; empty labels absorb nothing; the constructor absorbs its label bytes
// without a length). The empty-label observe_* / sample_* forms are the ones
// the Basefold opening uses (transcript.rs:332-350).
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include "gl_poseidon2_host.hpp"
#include "ext2_words.hpp"

namespace mbhost {

class Transcript {
public:
    Transcript() { std::memset(this, 0, sizeof(*this)); }
    explicit Transcript(const uint8_t* label, size_t n) {
        std::memset(this, 0, sizeof(*this));
        for (size_t i = 0; i < n; i++) absorb(label[i]);
    }

    void append_scalar(const char* label, uint64_t v) { absorb_label(label); absorb(v); }
    void append_u64(const char* label, uint64_t v) { absorb_label(label); absorb(v); }
    void append_ext2(const char* label, Ext2 v) { absorb_label(label); absorb(v.c0); absorb(v.c1); }
    // append_ext2 in two halves, for a caller that knows the label before the value exists (a round loop absorbs
    // the next message's label while the kernel that computes the message runs).
    void begin_append(const char* label) { absorb_label(label); }
    void finish_append_ext2(Ext2 v) { absorb(v.c0); absorb(v.c1); }
    uint64_t challenge_scalar(const char* label) { absorb_label(label); return squeeze(); }
    Ext2 challenge_ext2(const char* label) {
        absorb_label(label);
        Ext2 r;
        r.c0 = squeeze();
        r.c1 = squeeze();
        return r;
    }
    Transcript fork(uint64_t partition_id) const {
        Transcript t = *this;
        t.absorb(partition_id);
        return t;
    }

    // BasefoldTranscript view (empty labels).
    void observe_field(uint64_t v) { absorb(v); }
    void observe_ext2(Ext2 v) { absorb(v.c0); absorb(v.c1); }
    void observe_hash(const uint64_t h[4]) { for (int i = 0; i < 4; i++) absorb(h[i]); }
    uint64_t sample_challenge() { return squeeze(); }
    Ext2 sample_challenge_ext2() { Ext2 r; r.c0 = squeeze(); r.c1 = squeeze(); return r; }

    const uint64_t* state() const { return sponge_; }
    uint64_t permutations() const { return perms_; }

    void absorb(uint64_t v) {
        out_count_ = 0;
        in_buf_[in_count_++] = gl::canon(v);
        if (in_count_ == 4) duplexing();
    }
    uint64_t squeeze() {
        if (out_count_ == 0) duplexing();
        return out_buf_[--out_count_];
    }

private:
    void absorb_label(const char* label) {
        size_t n = label ? std::strlen(label) : 0;
        if (n == 0) return;
        absorb((uint64_t)n);
        for (size_t i = 0; i < n; i++) absorb((uint8_t)label[i]);
    }
    void duplexing() {
        for (int i = 0; i < in_count_; i++) sponge_[i] = in_buf_[i];
        for (int i = in_count_; i < 4; i++) sponge_[i] = 0;
        in_count_ = 0;
        p2host::permute(sponge_);   // canonical out
        perms_++;
        for (int i = 0; i < 4; i++) out_buf_[3 - i] = sponge_[i];
        out_count_ = 4;
    }

    uint64_t sponge_[8];
    uint64_t in_buf_[4];
    uint64_t out_buf_[4];
    int in_count_;
    int out_count_;
    uint64_t perms_;
};

}  // namespace mbhost
