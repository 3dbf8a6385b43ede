// Host layer above the C-ABI for the almost-Goldilocks sumcheck: the prover loop
// and the verifier the reference keeps in Rust (zk-torch-4), written in C++
// because no Rust toolchain exists on the build machine.
//
//   GpuLinearSumcheckProver::new / prove / prove_ext2 / prove_gpu_resident
//                                     zk-torch-4/src/sumcheck/gpu_prover.rs:26-112
//   CpuLinearSumcheckProverExt2       zk-torch-4/src/sumcheck/cpu_ext2_prover.rs:21-100
//                                     (same transcript labels, interoperable proofs)
//   SumcheckVerifier::verify          zk-torch-4/src/sumcheck/verifier.rs:14-113
//
// The transcript is the caller's (Monolith width 12, rate 8): the proof continues
// it, as `prove(.., transcript)` does in the reference, so the layers above (an
// einsum block, a fold-tree node) keep one transcript across their sumchecks.
#include <vector>
#include "../agl_traits.cuh"
#include "linear_sumcheck_state.cuh"
#include "agl_transcript.hpp"

using namespace mb;
using namespace mb::sc;

namespace mbhost {

using AglSumcheckStateExt2 = LinearSumcheckState<AglBase, AglExt2>;
using AglTranscript = aglm::Transcript;

static const uint8_t L_NUM_VAR[] = "num_var", L_NUM_POLY[] = "num_poly", L_MSG[] = "round_message",
                     L_CHALLENGE[] = "challenge";

static Ext2 aext2_mul_host(Ext2 a, Ext2 b) {
    agl::E2 r = agl::e2_canon(agl::e2_mul(agl::E2{a.c0, a.c1}, agl::E2{b.c0, b.c1}));
    return Ext2{r.c0, r.c1};
}
static Ext2 aext2_add_host(Ext2 a, Ext2 b) {
    return Ext2{agl::canon(agl::add(a.c0, b.c0)), agl::canon(agl::add(a.c1, b.c1))};
}
static Ext2 aext2_sub_host(Ext2 a, Ext2 b) {
    return Ext2{agl::canon(agl::sub(a.c0, b.c0)), agl::canon(agl::sub(a.c1, b.c1))};
}
static Ext2 aext2_inv_host(Ext2 a) {
    agl::E2 r = agl::e2_canon(agl::e2_inv(agl::E2{a.c0, a.c1}));
    return Ext2{r.c0, r.c1};
}
static Ext2 challenge_ext2(AglTranscript& t) {
    uint64_t w[2];
    t.challenge_vector(L_CHALLENGE, sizeof(L_CHALLENGE) - 1, w, 2);  // label once, two squeezes (transcript.rs:120-125)
    return Ext2{w[0], w[1]};
}

static int prove_linear(const uint64_t* d_tables, int d, int num_var, bool base_field, AglTranscript& t,
                        uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval) {
    t.append_u64(L_NUM_VAR, sizeof(L_NUM_VAR) - 1, (uint64_t)num_var);
    t.append_u64(L_NUM_POLY, sizeof(L_NUM_POLY) - 1, (uint64_t)d);
    AglSumcheckStateExt2 st;
    int rc = st.init_device(d_tables, d, num_var, base_field);
    if (rc != MB_OK) return rc;
    std::vector<Ext2> msg;
    bool label_absorbed = false;   // the first label of a round goes in while the round's kernel runs
    for (int round = 0; round < num_var; round++) {
        rc = st.compute_round_message(msg);
        if (rc != MB_OK) return rc;
        for (int c = 0; c <= d; c++) {
            if (c > 0 || !label_absorbed) t.begin_append(L_MSG, sizeof(L_MSG) - 1);
            t.finish_append_ext2(msg[c].c0, msg[c].c1);
            round_msgs[((size_t)round * (d + 1) + c) * 2] = msg[c].c0;
            round_msgs[((size_t)round * (d + 1) + c) * 2 + 1] = msg[c].c1;
        }
        Ext2 r = challenge_ext2(t);
        if (challenges) {
            challenges[2 * round] = r.c0;
            challenges[2 * round + 1] = r.c1;
        }
        rc = st.fold(r);
        if (rc != MB_OK) return rc;
        label_absorbed = round + 1 < num_var;
        if (label_absorbed) t.begin_append(L_MSG, sizeof(L_MSG) - 1);
    }
    std::vector<Ext2> fe;
    rc = st.final_evaluations(fe);
    if (rc != MB_OK) return rc;
    Ext2 prod{1, 0};
    for (int i = 0; i < d; i++) {
        if (final_evals) {
            final_evals[2 * i] = fe[i].c0;
            final_evals[2 * i + 1] = fe[i].c1;
        }
        prod = aext2_mul_host(prod, fe[i]);
    }
    final_eval[0] = prod.c0;
    final_eval[1] = prod.c1;
    return MB_OK;
}

// Lagrange interpolation through x = 0..n-1, evaluated at x (verifier.rs:91-113).
static Ext2 interpolate_and_evaluate(const Ext2* evals, int n, Ext2 x) {
    Ext2 result{0, 0};
    for (int i = 0; i < n; i++) {
        Ext2 basis{1, 0};
        for (int j = 0; j < n; j++) {
            if (j == i) continue;
            Ext2 num = aext2_sub_host(x, Ext2{(uint64_t)j, 0});
            Ext2 den = aext2_sub_host(Ext2{(uint64_t)i, 0}, Ext2{(uint64_t)j, 0});
            basis = aext2_mul_host(basis, aext2_mul_host(num, aext2_inv_host(den)));
        }
        result = aext2_add_host(result, aext2_mul_host(basis, evals[i]));
    }
    return result;
}

}  // namespace mbhost

extern "C" {

// Whole sumcheck proof for d tables of 2^num_var elements already on the device
// (poly-major; base_field != 0: one word per element, else (c0, c1)). `transcript`
// is a handle from agl_transcript_create and is advanced by the proof. Host outputs:
// round_msgs[num_var][d+1][2], challenges[num_var][2] (may be NULL),
// final_evals[d][2] (may be NULL), final_eval[2] = product of the final evaluations.
int agl_sumcheck_prove_device_ffi(const uint64_t* d_tables, int d, int num_var, int base_field, void* transcript,
                                  uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals,
                                  uint64_t* final_eval) {
    if (!transcript || !round_msgs || !final_eval) return MB_ERR_ARG;
    return mbhost::prove_linear(d_tables, d, num_var, base_field != 0, *static_cast<mbhost::AglTranscript*>(transcript),
                                round_msgs, challenges, final_evals, final_eval);
}

// Same proof from host tables: uploads them, proves, frees the device copy.
int agl_sumcheck_prove_host_ffi(const uint64_t* h_tables, int d, int num_var, int base_field, void* transcript,
                                uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals,
                                uint64_t* final_eval) {
    if (d < 1 || d > MAX_D || num_var < 0 || num_var > 40 || !h_tables) return MB_ERR_ARG;
    size_t words = ((size_t)1 << num_var) * (size_t)d * (base_field ? 1 : 2);
    uint64_t* d_tables = nullptr;
    MB_CUDA(pool_alloc((void**)&d_tables, words * sizeof(uint64_t)));
    int rc = MB_OK;
    if (cudaMemcpyAsync(d_tables, h_tables, words * sizeof(uint64_t), cudaMemcpyHostToDevice, MB_STREAM) != cudaSuccess)
        rc = MB_ERR_CUDA;
    if (rc == MB_OK)
        rc = agl_sumcheck_prove_device_ffi(d_tables, d, num_var, base_field, transcript, round_msgs, challenges,
                                           final_evals, final_eval);
    pool_free(d_tables);
    return rc;
}

// SumcheckVerifier::verify on the host: *ok = 1 when every round's P(0) + P(1)
// equals the running claim and the last claim equals final_eval; the challenges
// (num_var pairs) are written when `challenges` is not NULL. The transcript is
// advanced exactly as the prover's, up to the round that fails.
int agl_sumcheck_verify_ffi(const uint64_t* round_msgs, const uint64_t* final_eval, const uint64_t* claimed_sum, int d,
                            int num_var, void* transcript, uint64_t* challenges, int* ok) {
    using namespace mbhost;
    if (!transcript || !ok || !final_eval || !claimed_sum || d < 1 || d > MAX_D || num_var < 0 || (num_var && !round_msgs))
        return MB_ERR_ARG;
    AglTranscript& t = *static_cast<AglTranscript*>(transcript);
    *ok = 0;
    t.append_u64(L_NUM_VAR, sizeof(L_NUM_VAR) - 1, (uint64_t)num_var);
    t.append_u64(L_NUM_POLY, sizeof(L_NUM_POLY) - 1, (uint64_t)d);
    Ext2 current{agl::canon(claimed_sum[0]), agl::canon(claimed_sum[1])};
    std::vector<Ext2> msg(d + 1);
    for (int round = 0; round < num_var; round++) {
        for (int c = 0; c <= d; c++) {
            const uint64_t* w = round_msgs + ((size_t)round * (d + 1) + c) * 2;
            msg[c] = Ext2{agl::canon(w[0]), agl::canon(w[1])};
        }
        Ext2 sum = aext2_add_host(msg[0], msg[1]);
        if (sum.c0 != current.c0 || sum.c1 != current.c1) return MB_OK;
        for (int c = 0; c <= d; c++) t.append_ext2(L_MSG, sizeof(L_MSG) - 1, msg[c].c0, msg[c].c1);
        Ext2 r = challenge_ext2(t);
        if (challenges) {
            challenges[2 * round] = r.c0;
            challenges[2 * round + 1] = r.c1;
        }
        current = interpolate_and_evaluate(msg.data(), d + 1, r);
    }
    *ok = current.c0 == agl::canon(final_eval[0]) && current.c1 == agl::canon(final_eval[1]);
    return MB_OK;
}

}  // extern "C"
