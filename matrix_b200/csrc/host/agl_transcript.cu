// C-ABI over the host-side almost-Goldilocks Monolith and transcript. The
// reference keeps both in Rust (zk-torch-4/src/crypto/monolith.rs,
// zk-torch-4/src/transcript.rs); these entry points are what a binding calls
// instead when the transcript is driven from this library. Labels are byte
// strings with an explicit length (an empty label absorbs nothing).
#include "../common.cuh"
#include "agl_transcript.hpp"

using mbhost::aglm::Transcript;

extern "C" {

int agl_monolith_permute_host(uint64_t* state12) {
    if (!state12) return MB_ERR_ARG;
    mbhost::aglm::permute(state12);
    return MB_OK;
}

// 7 x 12 words, round-major.
int agl_monolith_round_constants(uint64_t* out84) {
    if (!out84) return MB_ERR_ARG;
    std::memcpy(out84, mbhost::aglm::round_constants(), sizeof(uint64_t) * 84);
    return MB_OK;
}

int agl_transcript_create(const uint8_t* label, size_t label_len, void** transcript) {
    if (!transcript || (!label && label_len)) return MB_ERR_ARG;
    *transcript = new Transcript(label, label_len);
    return MB_OK;
}
int agl_transcript_destroy(void* transcript) {
    delete static_cast<Transcript*>(transcript);
    return MB_OK;
}
int agl_transcript_fork(const void* transcript, const uint8_t* family, size_t family_len, uint64_t branch_id, void** forked) {
    if (!transcript || !forked || (!family && family_len)) return MB_ERR_ARG;
    *forked = new Transcript(static_cast<const Transcript*>(transcript)->fork(family, family_len, branch_id));
    return MB_OK;
}
int agl_transcript_append_scalar(void* transcript, const uint8_t* label, size_t label_len, uint64_t v) {
    if (!transcript) return MB_ERR_ARG;
    static_cast<Transcript*>(transcript)->append_scalar(label, label_len, v);
    return MB_OK;
}
int agl_transcript_append_u64(void* transcript, const uint8_t* label, size_t label_len, uint64_t v) {
    if (!transcript) return MB_ERR_ARG;
    static_cast<Transcript*>(transcript)->append_u64(label, label_len, v);
    return MB_OK;
}
int agl_transcript_append_u64_slice(void* transcript, const uint8_t* label, size_t label_len, const uint64_t* values, size_t n) {
    if (!transcript || (!values && n)) return MB_ERR_ARG;
    static_cast<Transcript*>(transcript)->append_u64_slice(label, label_len, values, n);
    return MB_OK;
}
int agl_transcript_append_ext2(void* transcript, const uint8_t* label, size_t label_len, uint64_t c0, uint64_t c1) {
    if (!transcript) return MB_ERR_ARG;
    static_cast<Transcript*>(transcript)->append_ext2(label, label_len, c0, c1);
    return MB_OK;
}
int agl_transcript_challenge_scalar(void* transcript, const uint8_t* label, size_t label_len, uint64_t* out) {
    if (!transcript || !out) return MB_ERR_ARG;
    *out = static_cast<Transcript*>(transcript)->challenge_scalar(label, label_len);
    return MB_OK;
}
// challenge_ext2 is n = 2; challenge_vector any n (transcript.rs:115-134).
int agl_transcript_challenge_vector(void* transcript, const uint8_t* label, size_t label_len, uint64_t* out, size_t n) {
    if (!transcript || (!out && n)) return MB_ERR_ARG;
    static_cast<Transcript*>(transcript)->challenge_vector(label, label_len, out, n);
    return MB_OK;
}
int agl_transcript_state(const void* transcript, uint64_t* out12) {
    if (!transcript || !out12) return MB_ERR_ARG;
    std::memcpy(out12, static_cast<const Transcript*>(transcript)->state(), sizeof(uint64_t) * 12);
    return MB_OK;
}

}  // extern "C"
