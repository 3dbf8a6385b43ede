// Host-side Monolith permutation over almost-Goldilocks and the Fiat-Shamir
// transcript built on it (duplex sponge, width 12, rate 8, overwrite mode,
// LIFO output buffer).
//
// Mirrors zk-torch-4/src/crypto/monolith.rs:66-208 (permutation and the SHA-256
// derivation of its round constants) and zk-torch-4/src/transcript.rs:22-243
// (same method names, absorb/squeeze order and label rule: length then bytes,
// empty labels absorb nothing, the constructor absorbs its label bytes without
// a length, appended values are reduced mod q first).
#pragma once
#include <cstdint>
#include <cstring>
#include <mutex>
#include "../agl_field.cuh"
#include "sha256.hpp"
#include "host_field.hpp"

namespace mbhost {
namespace aglm {

constexpr int WIDTH = 12;
constexpr int N_ROUNDS = 6;
constexpr int RATE = 8;

// [round][position]; rounds 0 and 6 are zero, rounds 1..5 are
// SHA-256("AGL-Monolith-RC-v1" || round || pos || salt)[0..8] little-endian with
// the salt counted up until the value is below q (crypto/monolith.rs:66-107).
inline const uint64_t (*round_constants())[WIDTH] {
    static uint64_t table[N_ROUNDS + 1][WIDTH];
    static std::once_flag once;
    std::call_once(once, [] {
        std::memset(table, 0, sizeof(table));
        for (uint32_t r = 1; r < (uint32_t)N_ROUNDS; r++)
            for (uint32_t i = 0; i < (uint32_t)WIDTH; i++)
                for (uint32_t salt = 0;; salt++) {
                    Sha256 h;
                    h.update("AGL-Monolith-RC-v1", 18);
                    h.update_u32_le(r);
                    h.update_u32_le(i);
                    h.update_u32_le(salt);
                    uint8_t d[32];
                    h.finalize(d);
                    uint64_t v = 0;
                    for (int b = 7; b >= 0; b--) v = (v << 8) | d[b];
                    if (v < agl::P) { table[r][i] = v; break; }
                }
    });
    return table;
}

// The byte S-box on all eight bytes (crypto/monolith.rs:147-154).
inline uint64_t bar(uint64_t x) {
    uint64_t nx = ~x;
    uint64_t l1 = ((nx & 0x8080808080808080ULL) >> 7) | ((nx & 0x7F7F7F7F7F7F7F7FULL) << 1);
    uint64_t l2 = ((x & 0xC0C0C0C0C0C0C0C0ULL) >> 6) | ((x & 0x3F3F3F3F3F3F3F3FULL) << 2);
    uint64_t l3 = ((x & 0xE0E0E0E0E0E0E0E0ULL) >> 5) | ((x & 0x1F1F1F1F1F1F1F1FULL) << 3);
    uint64_t t = x ^ (l1 & l2 & l3);
    return ((t & 0x8080808080808080ULL) >> 7) | ((t & 0x7F7F7F7F7F7F7F7FULL) << 1);
}

// Host arithmetic of the permutation. A round loop's host side is a chain of these permutations between two kernel
// launches, so this is written for a host core (64 x 64 -> 128 multiplier, 128-bit sums, no unpredictable branches)
// rather than shared with the device's 32-bit limb forms.
using hf::u128;
inline uint64_t reduce_small(u128 x) { return hf::agl_red_small(x); }   // high word below 2^31
inline uint64_t reduce_wide(u128 x) { return hf::agl_red(x); }          // any 128-bit value

using hf::circulant12;   // the MDS layer (host_field.hpp)

// s <- MDS s + rc, loose words out: low and high halves go through the circulant separately and each output is
// reduced once (L + 2^32 H + rc is below 162 * 2^64).
inline void concrete(uint64_t* s, const uint64_t* rc) {
    int64_t lo[WIDTH], hi[WIDTH], L[WIDTH], H[WIDTH];
    for (int j = 0; j < WIDTH; j++) { lo[j] = (int64_t)(s[j] & 0xFFFFFFFFULL); hi[j] = (int64_t)(s[j] >> 32); }
    circulant12(lo, L);
    circulant12(hi, H);
    for (int i = 0; i < WIDTH; i++) s[i] = reduce_small(((u128)(uint64_t)H[i] << 32) + (uint64_t)L[i] + rc[i]);
}

// In place; any 64-bit words in, canonical residues out (crypto/monolith.rs:201-208).
inline void permute(uint64_t* s) {
    static const uint64_t(*const rc)[WIDTH] = round_constants();
    concrete(s, rc[0]);
    for (int r = 1; r <= N_ROUNDS; r++) {
        for (int i = 0; i < 4; i++) s[i] = bar(s[i] >= agl::P ? s[i] - agl::P : s[i]);   // bars act on the canonical word
        // bricks: s_i += s_{i-1}^2 on the values before the layer
        uint64_t sq[WIDTH];
        for (int i = 1; i < WIDTH; i++) sq[i] = reduce_wide((u128)s[i - 1] * s[i - 1]);
        for (int i = 1; i < WIDTH; i++) s[i] = reduce_small((u128)s[i] + sq[i]);
        concrete(s, rc[r]);
    }
    for (int i = 0; i < WIDTH; i++) s[i] = s[i] >= agl::P ? s[i] - agl::P : s[i];
}

class Transcript {
public:
    Transcript() { std::memset(this, 0, sizeof(*this)); }
    Transcript(const uint8_t* label, size_t n) {
        std::memset(this, 0, sizeof(*this));
        for (size_t i = 0; i < n; i++) absorb(label[i]);
    }
    void append_scalar(const uint8_t* l, size_t n, uint64_t v) { absorb_label(l, n); absorb(agl::canon(v)); }
    void append_u64(const uint8_t* l, size_t n, uint64_t v) { absorb_label(l, n); absorb(agl::canon(v)); }
    void append_u64_slice(const uint8_t* l, size_t n, const uint64_t* v, size_t count) {
        absorb_label(l, n);
        for (size_t i = 0; i < count; i++) absorb(agl::canon(v[i]));
    }
    void append_ext2(const uint8_t* l, size_t n, uint64_t c0, uint64_t c1) {
        absorb_label(l, n);
        absorb(agl::canon(c0));
        absorb(agl::canon(c1));
    }
    // append_ext2 in two halves, for a caller that knows the label before the value exists (a round loop absorbs
    // the next message's label while the kernel that computes the message runs).
    void begin_append(const uint8_t* l, size_t n) { absorb_label(l, n); }
    void finish_append_ext2(uint64_t c0, uint64_t c1) { absorb(agl::canon(c0)); absorb(agl::canon(c1)); }
    uint64_t challenge_scalar(const uint8_t* l, size_t n) { absorb_label(l, n); return squeeze(); }
    void challenge_vector(const uint8_t* l, size_t n, uint64_t* out, size_t count) {
        absorb_label(l, n);
        for (size_t i = 0; i < count; i++) out[i] = squeeze();
    }
    // Clone, then absorb the family label and the branch id (transcript.rs:168-173).
    Transcript fork(const uint8_t* family, size_t n, uint64_t branch_id) const {
        Transcript t = *this;
        t.absorb_label(family, n);
        t.absorb(branch_id);
        return t;
    }
    const uint64_t* state() const { return sponge_; }

private:
    void absorb_label(const uint8_t* l, size_t n) {
        if (n == 0) return;
        absorb((uint64_t)n);
        for (size_t i = 0; i < n; i++) absorb(l[i]);
    }
    void duplexing() {
        for (int i = 0; i < in_count_; i++) sponge_[i] = in_buf_[i];
        for (int i = in_count_; i < RATE; i++) sponge_[i] = 0;
        in_count_ = 0;
        permute(sponge_);
        for (int i = 0; i < RATE; i++) out_buf_[RATE - 1 - i] = sponge_[i];
        out_count_ = RATE;
    }
    void absorb(uint64_t v) {
        out_count_ = 0;
        in_buf_[in_count_++] = v;
        if (in_count_ == RATE) duplexing();
    }
    uint64_t squeeze() {
        if (out_count_ == 0) duplexing();
        return out_buf_[--out_count_];
    }
    uint64_t sponge_[WIDTH];
    uint64_t in_buf_[RATE];
    uint64_t out_buf_[RATE];
    int in_count_, out_count_;
};

}  // namespace aglm
}  // namespace mbhost
