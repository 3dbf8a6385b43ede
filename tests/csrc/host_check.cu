// Test-only shim: exposes the host-callable instantiations of the library's
// field, Poseidon2 and transcript code so they can be compared with the CPU
// oracle on a machine without a GPU. Not part of the product libraries.
#include "gl_field.cuh"
#include "gl_ext5.cuh"
#include "gl_poseidon2.cuh"
#include "agl_field.cuh"
#include "host/gl_transcript.hpp"
#include "host/host_field.hpp"
#include "gl_monolith.cuh"
#include "host/agl_transcript.hpp"
#include "host/gl_monolith_host.hpp"
#include "host/host_tree_top.hpp"
#include "agl_mcommit.cuh"

extern "C" {
uint64_t hc_gl_add(uint64_t a, uint64_t b) { return gl::add(a, b); }
uint64_t hc_gl_sub(uint64_t a, uint64_t b) { return gl::sub(a, b); }
uint64_t hc_gl_mul(uint64_t a, uint64_t b) { return gl::mul(a, b); }
uint64_t hc_gl_mul_small(uint64_t a, uint32_t k) { return gl::mul_small(a, k); }
uint64_t hc_gl_inv(uint64_t a) { return gl::inv(a); }
void hc_e2_mul(const uint64_t* a, const uint64_t* b, uint64_t* o) {
    gl::E2 r = gl::e2_mul(gl::E2{a[0], a[1]}, gl::E2{b[0], b[1]});
    o[0] = r.c0; o[1] = r.c1;
}
void hc_e2_inv(const uint64_t* a, uint64_t* o) {
    gl::E2 r = gl::e2_inv(gl::E2{a[0], a[1]});
    o[0] = r.c0; o[1] = r.c1;
}
void hc_e5_mul(const uint64_t* a, const uint64_t* b, uint64_t* o) { gl::e5_store(o, gl::e5_mul(gl::e5_load(a), gl::e5_load(b))); }
void hc_e5_inv(const uint64_t* a, uint64_t* o) { gl::e5_store(o, gl::e5_inv(gl::e5_load(a))); }
void hc_e5_pow(const uint64_t* a, uint64_t e, uint64_t* o) { gl::e5_store(o, gl::e5_pow(gl::e5_load(a), e)); }
void hc_e5_frobenius(const uint64_t* a, uint64_t* o) { gl::e5_store(o, gl::e5_frobenius<1>(gl::e5_load(a))); }
uint64_t hc_gl_mul_add(uint64_t a, uint64_t b, uint64_t c) { return gl::mul_add(a, b, c); }
uint64_t hc_gl_reduce_limb_sums(uint64_t L, uint64_t H) { return gl::reduce_limb_sums(L, H); }
uint64_t hc_gl_reduce_limbs(uint32_t z0, uint32_t z1, uint32_t z2, uint32_t z3) { return gl::reduce_limbs(z0, z1, z2, z3); }
uint64_t hc_agl_add(uint64_t a, uint64_t b) { return agl::add(a, b); }
uint64_t hc_agl_sub(uint64_t a, uint64_t b) { return agl::sub(a, b); }
uint64_t hc_agl_mul(uint64_t a, uint64_t b) { return agl::mul(a, b); }
uint64_t hc_agl_inv(uint64_t a) { return agl::inv(a); }
void hc_aext2_mul(const uint64_t* a, const uint64_t* b, uint64_t* o) {
    agl::E2 r = agl::e2_mul(agl::E2{a[0], a[1]}, agl::E2{b[0], b[1]});
    o[0] = r.c0; o[1] = r.c1;
}
void hc_aext2_mul_lazy(const uint64_t* a, const uint64_t* b, uint64_t* o) {
    agl::E2 r = agl::e2_mul_lazy(agl::E2{a[0], a[1]}, agl::E2{b[0], b[1]});
    o[0] = agl::canon(r.c0); o[1] = agl::canon(r.c1);
}
void hc_aext2_fma_pre(const uint64_t* r, const uint64_t* d, const uint64_t* a, uint64_t* o) {
    agl::E2 v = agl::e2_fma_pre(agl::e2_pre(agl::E2{r[0], r[1]}), agl::E2{d[0], d[1]}, agl::E2{a[0], a[1]});
    o[0] = agl::canon(v.c0); o[1] = agl::canon(v.c1);
}
void hc_aext2_fma_pre_base(const uint64_t* r, uint64_t d, uint64_t a, uint64_t* o) {
    agl::E2 v = agl::e2_fma_pre_base(agl::e2_pre(agl::E2{r[0], r[1]}), d, a);
    o[0] = agl::canon(v.c0); o[1] = agl::canon(v.c1);
}
void hc_mcm_shake(const uint32_t* seed, uint32_t counter, const uint32_t* nonce, uint32_t* out) {
    mcm::shake_key_block(seed, counter, nonce, out);
}
void hc_mcm_key_block(const uint32_t* seed, uint32_t kind, uint32_t row, uint64_t col, uint32_t b, uint64_t* vals) {
    mcm::key_block8(seed, kind, row, col, b, vals);
}
void hc_poseidon2(uint64_t* s) { gl::poseidon2_permute(s); }
// the host-side form (transcripts, tree tops) and the reductions underneath both host permutations
void hc_poseidon2_host(uint64_t* s) { mbhost::p2host::permute(s); }
// host-form extension arithmetic (the last rounds of a sumcheck): o = a * b, a + b, a - b on canonical words
void hc_hf_e2(int agl_field, const uint64_t* a, const uint64_t* b, uint64_t* o) {
    using namespace mbhost::hf;
    if (agl_field) {
        e2_mul<AglE2Ops>(a[0], a[1], b[0], b[1], o[0], o[1]);
        o[2] = agl_add(a[0], b[0]); o[3] = agl_add(a[1], b[1]);
        o[4] = agl_sub(a[0], b[0]); o[5] = agl_sub(a[1], b[1]);
    } else {
        e2_mul<GlE2Ops>(a[0], a[1], b[0], b[1], o[0], o[1]);
        o[2] = gl_add(a[0], b[0]); o[3] = gl_add(a[1], b[1]);
        o[4] = gl_sub(a[0], b[0]); o[5] = gl_sub(a[1], b[1]);
    }
}
void hc_aglm_circulant12(const int64_t* x, int64_t* out) { mbhost::hf::circulant12(x, out); }
uint64_t hc_p2host_red(uint64_t lo, uint64_t hi) { return mbhost::p2host::red(((unsigned __int128)hi << 64) | lo); }
uint64_t hc_aglm_reduce_wide(uint64_t lo, uint64_t hi) { return mbhost::aglm::reduce_wide(((unsigned __int128)hi << 64) | lo); }
uint64_t hc_aglm_reduce_small(uint64_t lo, uint64_t hi) { return mbhost::aglm::reduce_small(((unsigned __int128)hi << 64) | lo); }
// sum_i x[i] * y[i] + c through the lazy accumulator
uint64_t hc_gl_dot(const uint64_t* x, const uint64_t* y, int n, uint64_t c) {
    gl::Acc s = gl::acc_from(c);
    for (int i = 0; i < n; i++) gl::acc_mul(s, x[i], y[i]);
    return gl::canon(gl::acc_reduce(s));
}
uint64_t hc_gl_sub_canon(uint64_t a, uint64_t b) { return gl::sub_canon(a, b); }
// a + r * d with the precomputed-factor form
void hc_e2_fma_pre(const uint64_t* r, const uint64_t* d, const uint64_t* a, uint64_t* o) {
    gl::E2 v = gl::e2_canon(gl::e2_fma_pre(gl::e2_pre(gl::E2{r[0], r[1]}), gl::E2{d[0], d[1]}, gl::E2{a[0], a[1]}));
    o[0] = v.c0; o[1] = v.c1;
}
// sum_i a[i] * b[i] over the extension through the lazy accumulator
void hc_e2_dot(const uint64_t* a, const uint64_t* b, int n, uint64_t* o) {
    gl::E2Acc q = gl::e2acc_zero();
    for (int i = 0; i < n; i++) gl::e2acc_mul(q, gl::E2{a[2 * i], a[2 * i + 1]}, gl::E2{b[2 * i], b[2 * i + 1]});
    gl::E2 v = gl::e2_canon(gl::e2acc_reduce(q));
    o[0] = v.c0; o[1] = v.c1;
}
void hc_gl_monolith(uint64_t* s) {
    gl::monolith_permute(s);
    for (int i = 0; i < 12; i++) s[i] = gl::canon(s[i]);
}
// the host-hashed top of a Merkle tree: upper layers and root above a layer of `count` digests
void hc_tree_top(int hash, const uint64_t* nodes, size_t count, uint64_t* upper, uint64_t* root) {
    mbhost::host_hash_top(hash, nodes, count, upper, root);
}
void hc_gl_monolith_host(uint64_t* s) { mbhost::monohost::permute(s); }
void hc_agl_monolith(uint64_t* s) { mbhost::aglm::permute(s); }
uint64_t hc_agl_reduce_limb_sums(uint64_t L, uint64_t H) { return agl::reduce_limb_sums(L, H); }

// Replays a script of transcript operations: op 0 = absorb(v), 1 = squeeze -> out.
int hc_transcript_script(const uint8_t* label, size_t n, const int* ops, const uint64_t* vals, int nops, uint64_t* out) {
    mbhost::Transcript t(label, n);
    int k = 0;
    for (int i = 0; i < nops; i++) {
        if (ops[i] == 0) t.absorb(vals[i]);
        else out[k++] = t.squeeze();
    }
    return k;
}
}
