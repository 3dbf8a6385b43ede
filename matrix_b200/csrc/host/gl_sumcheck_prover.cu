// Host layer above the C-ABI for the Goldilocks sumcheck: the prover loop the
// reference keeps in Rust, written in C++ because no Rust toolchain exists on
// the build machine.
//
//   GpuSumcheckStateExt2      goldilocks-cuda-rs/src/sumcheck_prover.rs:206-436
//                             (linear_sumcheck_state.cuh, shared with almost-Goldilocks)
//   GpuLinearSumcheckProver   zk-torch-3/src/sumcheck/gpu_prover.rs:13-150
//
// Method names and protocol order follow the reference.
#include <vector>
#include <memory>
#include "linear_sumcheck_state.cuh"
#include "gl_transcript.hpp"

using namespace mb;
using namespace mb::sc;

namespace mbhost {

using GpuSumcheckStateExt2 = LinearSumcheckState<GlBase, GlExt2>;

static Ext2 ext2_mul_host(Ext2 a, Ext2 b) {
    gl::E2 r = gl::e2_canon(gl::e2_mul(gl::E2{a.c0, a.c1}, gl::E2{b.c0, b.c1}));
    return Ext2{r.c0, r.c1};
}

// The prover loop of GpuLinearSumcheckProver::prove / prove_ext2.
static int prove_linear(const uint64_t* d_tables, int d, int num_var, bool base_field, Transcript& t,
                        uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval) {
    t.append_u64("num_var", (uint64_t)num_var);
    t.append_u64("num_poly", (uint64_t)d);
    GpuSumcheckStateExt2 st;
    int rc = st.init_device(d_tables, d, num_var, base_field);
    if (rc != MB_OK) return rc;
    std::vector<Ext2> msg;
    bool label_absorbed = false;   // the first label of a round goes in while the round's kernel runs
    for (int round = 0; round < num_var; round++) {
        rc = st.compute_round_message(msg);
        if (rc != MB_OK) return rc;
        for (int c = 0; c <= d; c++) {
            if (c > 0 || !label_absorbed) t.begin_append("round_message");
            t.finish_append_ext2(msg[c]);
            round_msgs[((size_t)round * (d + 1) + c) * 2] = msg[c].c0;
            round_msgs[((size_t)round * (d + 1) + c) * 2 + 1] = msg[c].c1;
        }
        Ext2 r = t.challenge_ext2("challenge");
        challenges[2 * round] = r.c0;
        challenges[2 * round + 1] = r.c1;
        rc = st.fold(r);
        if (rc != MB_OK) return rc;
        label_absorbed = round + 1 < num_var;
        if (label_absorbed) t.begin_append("round_message");
    }
    std::vector<Ext2> fe;
    rc = st.final_evaluations(fe);
    if (rc != MB_OK) return rc;
    Ext2 prod{1, 0};
    for (int i = 0; i < d; i++) {
        final_evals[2 * i] = fe[i].c0;
        final_evals[2 * i + 1] = fe[i].c1;
        prod = ext2_mul_host(prod, fe[i]);
    }
    final_eval[0] = prod.c0;
    final_eval[1] = prod.c1;
    return MB_OK;
}

// Lagrange interpolation through x = 0..n-1, evaluated at x (zk-torch-3/src/sumcheck/verifier.rs: the next claim is
// P_round(r)).
static Ext2 interpolate_and_evaluate(const Ext2* evals, int n, Ext2 x) {
    gl::E2 result{0, 0};
    const gl::E2 xx{x.c0, x.c1};
    for (int i = 0; i < n; i++) {
        gl::E2 num{1, 0};
        uint64_t den = 1;
        for (int j = 0; j < n; j++) {
            if (j == i) continue;
            num = gl::e2_canon(gl::e2_mul(num, gl::e2_sub(xx, gl::E2{(uint64_t)j, 0})));
            den = gl::mul(den, gl::sub((uint64_t)i, (uint64_t)j));
        }
        const uint64_t inv = gl::canon(gl::inv(den));
        const gl::E2 basis{gl::mul(num.c0, inv), gl::mul(num.c1, inv)};
        result = gl::e2_add(result, gl::e2_mul(gl::E2{evals[i].c0, evals[i].c1}, basis));
    }
    result = gl::e2_canon(result);
    return Ext2{result.c0, result.c1};
}

}  // namespace mbhost

extern "C" {

// The verifier of the same protocol on the host (zk-torch-3/src/sumcheck/verifier.rs): *ok = 1 when every round's
// P(0) + P(1) equals the running claim and the last claim equals final_eval; the challenges (num_var pairs) are
// written when `challenges` is not NULL. The transcript starts as Transcript::new(label) and is advanced exactly as
// the prover's, up to the round that fails. No device call.
int gl_sumcheck_verify_ffi(const uint64_t* round_msgs, const uint64_t* final_eval, const uint64_t* claimed_sum, int d, int num_var,
                           const uint8_t* label, size_t label_len, uint64_t* challenges, int* ok) {
    using namespace mbhost;
    if (!ok || !final_eval || !claimed_sum || d < 1 || d > MAX_D || num_var < 0 || (num_var && !round_msgs) || (!label && label_len))
        return MB_ERR_ARG;
    *ok = 0;
    Transcript t(label, label_len);
    t.append_u64("num_var", (uint64_t)num_var);
    t.append_u64("num_poly", (uint64_t)d);
    Ext2 current{gl::canon(claimed_sum[0]), gl::canon(claimed_sum[1])};
    std::vector<Ext2> msg(d + 1);
    for (int round = 0; round < num_var; round++) {
        for (int c = 0; c <= d; c++) {
            const uint64_t* w = round_msgs + ((size_t)round * (d + 1) + c) * 2;
            msg[c] = Ext2{gl::canon(w[0]), gl::canon(w[1])};
        }
        const gl::E2 sum = gl::e2_canon(gl::e2_add(gl::E2{msg[0].c0, msg[0].c1}, gl::E2{msg[1].c0, msg[1].c1}));
        if (sum.c0 != current.c0 || sum.c1 != current.c1) return MB_OK;
        for (int c = 0; c <= d; c++) t.append_ext2("round_message", msg[c]);
        const Ext2 r = t.challenge_ext2("challenge");
        if (challenges) {
            challenges[2 * round] = r.c0;
            challenges[2 * round + 1] = r.c1;
        }
        current = interpolate_and_evaluate(msg.data(), d + 1, r);
    }
    *ok = current.c0 == gl::canon(final_eval[0]) && current.c1 == gl::canon(final_eval[1]);
    return MB_OK;
}

// Whole sumcheck proof for d tables of 2^num_var elements that are already on
// the device (poly-major). base_field != 0: u64 tables; else (c0, c1) tables.
// The transcript starts as Transcript::new(label). Host outputs:
//   round_msgs[num_var][d+1][2], challenges[num_var][2], final_evals[d][2],
//   final_eval[2], transcript_state[8] (sponge words after the proof; may be NULL).
int gl_sumcheck_prove_device_ffi(const uint64_t* d_tables, int d, int num_var, int base_field,
                                 const uint8_t* label, size_t label_len, uint64_t* round_msgs,
                                 uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval,
                                 uint64_t* transcript_state) {
    mbhost::Transcript t(label, label_len);
    int rc = mbhost::prove_linear(d_tables, d, num_var, base_field != 0, t, round_msgs, challenges, final_evals,
                                  final_eval);
    if (rc == MB_OK && transcript_state) std::memcpy(transcript_state, t.state(), 64);
    return rc;
}

// Same proof from host tables: uploads them, proves, frees the device copy.
int gl_sumcheck_prove_host_ffi(const uint64_t* h_tables, int d, int num_var, int base_field,
                               const uint8_t* label, size_t label_len, uint64_t* round_msgs,
                               uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval,
                               uint64_t* transcript_state) {
    if (d < 1 || d > MAX_D || num_var < 0 || num_var > 40 || !h_tables) return MB_ERR_ARG;
    size_t words = ((size_t)1 << num_var) * (size_t)d * (base_field ? 1 : 2);
    uint64_t* d_tables = nullptr;
    MB_CUDA(pool_alloc((void**)&d_tables, words * sizeof(uint64_t)));
    int rc = MB_OK;
    if (cudaMemcpyAsync(d_tables, h_tables, words * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM) != cudaSuccess)
        rc = MB_ERR_CUDA;
    if (rc == MB_OK)
        rc = gl_sumcheck_prove_device_ffi(d_tables, d, num_var, base_field, label, label_len, round_msgs, challenges,
                                          final_evals, final_eval, transcript_state);
    pool_free(d_tables);
    return rc;
}

}  // extern "C"
