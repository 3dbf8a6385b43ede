// Same-point sumcheck over the almost-Goldilocks extension, whole protocol: the host loop the reference keeps
// in Rust (zk-torch-4/src/fold/same_point_sumcheck.rs), over this library's batched same-point kernels.
//
//   prove_same_point_gpu_batched           same_point_sumcheck.rs:1032-1063, 1334-1553 (uniform arity: header,
//                                          alpha, device eq tables, per-round combined message, fold, reveals)
//   GpuBatchedSamePointState               almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:468-760 (interleaved
//                                          layout: per leaf the eq table, then the f table)
//   verify_same_point                      same_point_sumcheck.rs:161-219
//
// M instances of the same arity k, each with its own claim point r_i, claim y_i = f_i(r_i) and witness f_i
// (binary packed, ternary single chunk, or an extension table); the sumcheck
//   sum_i alpha^i y_i = sum_x sum_i alpha^i eq(r_i, x) f_i(x)
// reduces them to one point R. Degree 2: three evaluations per round. The transcript is the caller's (Monolith
// width 12) and is advanced exactly as the reference's prover advances it, so proofs are interchangeable with
// the CPU prover's (heterogeneous arities stay on that path, as in the reference).
//
// Device side: two ping-pong buffers of M x (eq | f) tables; the eq tables of all leaves are built in two launches.
// A binary witness is never lifted: round 0 reads the packed bits, afterwards everything is an extension table.
// Per round: ONE pass over the tables (the fold on the challenge and the per-leaf sums of the next round in the
// same kernel; the reference folds, then reads the folded tables again), one small launch that adds the blocks'
// partial sums, a 48-byte-per-leaf read-back into page-locked memory, the host combination with the powers of
// alpha and the transcript. The header of the transcript (every claim point) is absorbed while the device builds
// the tables and the first message.
#include <vector>
#include "../agl_traits.cuh"
#include "../eq_kernels.cuh"
#include "agl_transcript.hpp"

using namespace mb;
using namespace mb::sc;

extern "C" {
int aext2_sumcheck_batched_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, size_t original_size, size_t half,
                                             int num_leaves, int num_blocks_x);
int aext2_sumcheck_batched_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0, uint64_t challenge_c1,
                                    size_t original_size, size_t half, int num_leaves);
int aext2_sumcheck_batched_round0_binary_msg_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_partial,
                                                 size_t original_size, size_t half, int num_leaves, int num_blocks_x,
                                                 size_t packed_size_u64);
int aext2_sumcheck_batched_round0_binary_fold_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_output,
                                                  uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size, size_t half,
                                                  int num_leaves, size_t packed_size_u64);
int aext2_sumcheck_batched_fold_message_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0, uint64_t challenge_c1,
                                            size_t original_size, size_t half, int num_leaves, int num_blocks_x, uint64_t* d_partial);
int aext2_sumcheck_batched_round0_binary_fold_message_ffi(const uint64_t* d_polys, const uint64_t* d_packed, uint64_t* d_output,
                                                          uint64_t challenge_c0, uint64_t challenge_c1, size_t original_size, size_t half,
                                                          int num_leaves, int num_blocks_x, size_t packed_size_u64, uint64_t* d_partial);
int aext2_batched_lift_ternary_single_ffi(const uint64_t* d_pos, const uint64_t* d_neg, uint64_t* d_polys, size_t original_size,
                                          int num_leaves, size_t packed_size_u64);
}

namespace mbhost {

using AglTranscript = aglm::Transcript;
using E2 = agl::E2;

namespace {

const uint8_t L_NUM_VAR[] = "sp_num_var", L_NUM_INST[] = "sp_num_inst", L_ARITY[] = "sp_arity_i", L_R[] = "sp_r_i",
              L_Y[] = "sp_y_i", L_ALPHA[] = "sp_alpha", L_MSG[] = "sp_round_msg", L_CH[] = "sp_round_challenge",
              L_FEVAL[] = "sp_f_eval";
#define SP_LABEL(l) l, sizeof(l) - 1

inline E2 e2c(E2 a) { return agl::e2_canon(a); }
inline E2 ld(const uint64_t* w) { return E2{agl::canon(w[0]), agl::canon(w[1])}; }
inline E2 challenge(AglTranscript& t, const uint8_t* l, size_t n) {
    uint64_t w[2];
    t.challenge_vector(l, n, w, 2);   // the label once, two squeezes (transcript.rs:120-125)
    return E2{w[0], w[1]};
}

// sums[leaf][c][2] = sum over the blocks of partial[block][leaf][c][2]: one thread per output word
__global__ void add_blocks_kernel(const uint64_t* __restrict__ partial, int blocks, int words, uint64_t* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= words) return;
    uint64_t s = 0;
    for (int b = 0; b < blocks; b++) s = agl::add(s, partial[(size_t)b * words + k]);
    out[k] = agl::canon(s);
}

// out[leaf][2] = element 0 of every leaf's f table
__global__ void first_f_kernel(const uint64_t* __restrict__ polys, size_t n, int leaves, uint64_t* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < 2 * leaves) out[k] = polys[(size_t)(k >> 1) * 4 * n + 2 * n + (k & 1)];
}

// dense witness: the caller's [leaf][n][2] tables into the f halves of the interleaved buffer
__global__ void place_dense_kernel(const uint64_t* __restrict__ src, uint64_t* __restrict__ polys, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    const uint64_t* s = src + (size_t)blockIdx.y * 2 * n;
    uint64_t* d = polys + (size_t)blockIdx.y * 4 * n + 2 * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        agl::e2_store(d + 2 * i, E2{agl::canon(s[2 * i]), agl::canon(s[2 * i + 1])});
}

void header(AglTranscript& t, int M, int arity, const uint64_t* pts, const uint64_t* vals) {   // same_point_sumcheck.rs:78-87
    t.append_u64(SP_LABEL(L_NUM_VAR), (uint64_t)arity);
    t.append_u64(SP_LABEL(L_NUM_INST), (uint64_t)M);
    for (int i = 0; i < M; i++) {
        t.append_u64(SP_LABEL(L_ARITY), (uint64_t)arity);
        for (int k = 0; k < arity; k++) {
            const uint64_t* p = pts + ((size_t)i * arity + k) * 2;
            t.append_ext2(SP_LABEL(L_R), p[0], p[1]);
        }
        t.append_ext2(SP_LABEL(L_Y), vals[2 * i], vals[2 * i + 1]);
    }
}

E2 eq_eval(const uint64_t* a, const E2* b, int n) {   // same_point_sumcheck.rs:907-921
    E2 acc{1, 0};
    const E2 one{1, 0};
    for (int i = 0; i < n; i++) {
        const E2 ai = ld(a + 2 * i);
        acc = e2c(agl::e2_mul(acc, agl::e2_add(agl::e2_mul(ai, b[i]), agl::e2_mul(agl::e2_sub(one, ai), agl::e2_sub(one, b[i])))));
    }
    return acc;
}

struct Buffers {
    uint64_t *a = nullptr, *b = nullptr, *partial = nullptr, *sums = nullptr, *pts = nullptr, *scratch = nullptr;
    ~Buffers() { pool_free(a); pool_free(b); pool_free(partial); pool_free(sums); pool_free(pts); pool_free(scratch); }
};

// Device state of M leaves of 2^arity points: eq tables from the claim points, and the f tables unless the
// witness is binary (round 0 reads the packed bits).
int setup(Buffers& buf, int M, int arity, const uint64_t* h_pts, int kind, const uint64_t* d_w0, const uint64_t* d_w1, bool two_buffers,
          int& blocks) {
    const size_t n = (size_t)1 << arity, words = arity >= 6 ? n >> 6 : 1;
    blocks = (int)(n / 2 >= (size_t)256 * 64 ? 64 : (n / 2 + 255) / 256 > 0 ? (n / 2 + 255) / 256 : 1);
    const int sum_words = 6 * M;
    MB_CUDA(pool_alloc((void**)&buf.a, sizeof(uint64_t) * 4 * n * (size_t)M));
    if (two_buffers) MB_CUDA(pool_alloc((void**)&buf.b, sizeof(uint64_t) * 4 * n * (size_t)M));
    MB_CUDA(pool_alloc((void**)&buf.partial, sizeof(uint64_t) * (size_t)blocks * sum_words));
    MB_CUDA(pool_alloc((void**)&buf.sums, sizeof(uint64_t) * sum_words));
    MB_CUDA(pool_alloc((void**)&buf.pts, sizeof(uint64_t) * 2 * (size_t)arity * M));
    MB_CUDA(pool_alloc((void**)&buf.scratch,
                       sizeof(uint64_t) * 2 * (size_t)M * (((size_t)1 << (arity / 2)) + ((size_t)1 << (arity - arity / 2)))));
    MB_CUDA(cudaMemcpyAsync(buf.pts, h_pts, sizeof(uint64_t) * 2 * (size_t)arity * M, cudaMemcpyHostToDevice, MB_STREAM));
    // eq tables from the claim points, on the device, into the eq halves: all leaves in two launches
    int rc = eq::build_batched<AglExt2>(buf.pts, 2 * (size_t)arity, buf.a, 4 * n, buf.scratch, arity, M, MB_STREAM);
    if (rc != MB_OK) return rc;
    if (kind == 1) {
        rc = aext2_batched_lift_ternary_single_ffi(d_w0, d_w1, buf.a, n, M, words);
    } else if (kind == 2) {
        MB_KERNEL("same_point_place");
        dim3 grid(grid_for(n, 256, 8), M);
        place_dense_kernel<<<grid, 256, 0, MB_STREAM>>>(d_w0, buf.a, n);
        rc = finish_async();
    }
    return rc;
}

// Page-locked landing zone of the calling thread for the per-leaf sums (grown on demand, kept between calls): a
// read-back into it is asynchronous, so the host can work while the device finishes the round.
uint64_t* pinned_words(size_t words) {
    struct Holder {
        uint64_t* p = nullptr;
        size_t cap = 0;
        ~Holder() { if (p) cudaFreeHost(p); }
    };
    static thread_local Holder h;
    if (h.cap < words) {
        if (h.p) cudaFreeHost(h.p);
        h.p = nullptr;
        h.cap = 0;
        if (cudaMallocHost(&h.p, words * sizeof(uint64_t)) != cudaSuccess) { h.p = nullptr; return nullptr; }
        h.cap = words;
    }
    return h.p;
}

inline int blocks_for(size_t pairs, int blocks) { return (int)((pairs + 255) / 256 < (size_t)blocks ? (pairs + 255) / 256 : blocks); }

// Adds the blocks' partial sums and queues the read-back of sums[leaf][3][2] into h_sums.
int queue_sums(Buffers& buf, int M, int bx, uint64_t* h_sums) {
    const int sum_words = 6 * M;
    {
        MB_KERNEL("same_point_add_blocks");
        add_blocks_kernel<<<(sum_words + 127) / 128, 128, 0, MB_STREAM>>>(buf.partial, bx, sum_words, buf.sums);
    }
    MB_CUDA(cudaMemcpyAsync(h_sums, buf.sums, sizeof(uint64_t) * sum_words, cudaMemcpyDeviceToHost, MB_STREAM));
    return MB_OK;
}

// Per-leaf T_i(0), T_i(1), T_i(2) of the current round into h_sums[leaf][3][2] (page-locked): launches and the
// read-back are queued; the caller synchronises the stream before it reads h_sums.
int leaf_messages(Buffers& buf, const uint64_t* cur, int M, size_t n, size_t half, int blocks, bool bits, const uint64_t* d_packed,
                  size_t words, uint64_t* h_sums) {
    const int bx = blocks_for(half, blocks);
    int rc = bits ? aext2_sumcheck_batched_round0_binary_msg_ffi(cur, d_packed, buf.partial, n, half, M, bx, words)
                  : aext2_sumcheck_batched_round_message_ffi(cur, buf.partial, n, half, M, bx);
    if (rc != MB_OK) return rc;
    return queue_sums(buf, M, bx, h_sums);
}

// The fold on r fused with the per-leaf sums of the next round (input half >= 2); h_sums as above.
int fold_and_next_messages(Buffers& buf, const uint64_t* cur, uint64_t* other, E2 r, int M, size_t n, size_t half, int blocks, bool bits,
                           const uint64_t* d_packed, size_t words, uint64_t* h_sums) {
    const int bx = blocks_for(half / 2, blocks);
    int rc = bits ? aext2_sumcheck_batched_round0_binary_fold_message_ffi(cur, d_packed, other, r.c0, r.c1, n, half, M, bx, words, buf.partial)
                  : aext2_sumcheck_batched_fold_message_ffi(cur, other, r.c0, r.c1, n, half, M, bx, buf.partial);
    if (rc != MB_OK) return rc;
    return queue_sums(buf, M, bx, h_sums);
}

}  // namespace

// y_i = f_i(r_i) for every leaf: the claims the protocol starts from (FoldData::evaluate_at_ext2,
// zk-torch-4/src/fold/mod.rs:107-110), as sum_x eq(r_i, x) f_i(x) = T_i(0) + T_i(1) of the first round.
int same_point_claims(int M, int arity, const uint64_t* h_pts, int kind, const uint64_t* d_w0, const uint64_t* d_w1, uint64_t* h_vals) {
    if (M < 1 || M > 4096 || arity < 1 || arity > 32 || !h_pts || !d_w0 || kind < 0 || kind > 2 || (kind == 1 && !d_w1) || !h_vals)
        return MB_ERR_ARG;
    const size_t n = (size_t)1 << arity, words = arity >= 6 ? n >> 6 : 1;
    Buffers buf;
    int blocks = 1;
    int rc = setup(buf, M, arity, h_pts, kind, d_w0, d_w1, false, blocks);
    if (rc != MB_OK) return rc;
    uint64_t* h_sums = pinned_words(6 * (size_t)M);
    if (!h_sums) return MB_ERR_CUDA;
    rc = leaf_messages(buf, buf.a, M, n, n / 2, blocks, kind == 0, d_w0, words, h_sums);
    if (rc != MB_OK) return rc;
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    for (int i = 0; i < M; i++) {
        const E2 y = e2c(agl::e2_add(ld(h_sums + 6 * (size_t)i), ld(h_sums + 6 * (size_t)i + 2)));
        h_vals[2 * i] = y.c0;
        h_vals[2 * i + 1] = y.c1;
    }
    return MB_OK;
}

// kind 0: d_w0 = packed bits [M][words]; 1: d_w0 / d_w1 = +1 / -1 masks [M][words]; 2: d_w0 = extension tables
// [M][2^arity][2]. words = max(1, 2^(arity - 6)).
int same_point_prove(int M, int arity, const uint64_t* h_pts, const uint64_t* h_vals, int kind, const uint64_t* d_w0,
                     const uint64_t* d_w1, AglTranscript& t, uint64_t* h_round_msgs, uint64_t* h_challenges, uint64_t* h_f_evals,
                     uint64_t* h_final_eval) {
    if (M < 1 || M > 4096 || arity < 1 || arity > 32 || !h_pts || !h_vals || !d_w0 || kind < 0 || kind > 2 || (kind == 1 && !d_w1) ||
        !h_round_msgs || !h_f_evals || !h_final_eval)
        return MB_ERR_ARG;
    const size_t n = (size_t)1 << arity, words = arity >= 6 ? n >> 6 : 1;
    Buffers buf;
    int blocks = 1;
    const int sum_words = 6 * M;
    uint64_t* h_sums = pinned_words(sum_words);
    if (!h_sums) return MB_ERR_CUDA;
    // the tables and the first round's per-leaf sums do not depend on alpha: they are queued first, and the
    // header of the transcript (every claim point, label by label: the longest host step of the proof) is
    // absorbed while the device works
    int rc = setup(buf, M, arity, h_pts, kind, d_w0, d_w1, true, blocks);
    if (rc != MB_OK) return rc;
    rc = leaf_messages(buf, buf.a, M, n, n / 2, blocks, kind == 0, d_w0, words, h_sums);
    if (rc != MB_OK) return rc;
    header(t, M, arity, h_pts, h_vals);
    const E2 alpha = challenge(t, SP_LABEL(L_ALPHA));
    std::vector<E2> alphas(M);
    E2 pw{1, 0};
    for (int i = 0; i < M; i++) { alphas[i] = pw; pw = e2c(agl::e2_mul(pw, alpha)); }

    std::vector<E2> R(arity);
    bool label_absorbed = false;
    uint64_t* cur = buf.a;
    uint64_t* other = buf.b;
    for (int round = 0; round < arity; round++) {
        const size_t half = n >> (round + 1);
        const bool bits = kind == 0 && round == 0;
        // this round's sums were queued with the setup (round 0) or by the fold of the round before
        MB_CUDA(cudaStreamSynchronize(MB_STREAM));
        E2 msg[3] = {{0, 0}, {0, 0}, {0, 0}};
        for (int i = 0; i < M; i++)
            for (int c = 0; c < 3; c++) msg[c] = agl::e2_add(msg[c], agl::e2_mul(alphas[i], ld(h_sums + (size_t)i * 6 + 2 * c)));
        for (int c = 0; c < 3; c++) {
            msg[c] = e2c(msg[c]);
            if (c > 0 || !label_absorbed) t.begin_append(SP_LABEL(L_MSG));
            t.finish_append_ext2(msg[c].c0, msg[c].c1);
            h_round_msgs[((size_t)round * 3 + c) * 2] = msg[c].c0;
            h_round_msgs[((size_t)round * 3 + c) * 2 + 1] = msg[c].c1;
        }
        const E2 r = challenge(t, SP_LABEL(L_CH));
        R[round] = r;
        if (h_challenges) { h_challenges[2 * round] = r.c0; h_challenges[2 * round + 1] = r.c1; }
        if (half >= 2)
            rc = fold_and_next_messages(buf, cur, other, r, M, n, half, blocks, bits, d_w0, words, h_sums);
        else
            rc = bits ? aext2_sumcheck_batched_round0_binary_fold_ffi(cur, d_w0, other, r.c0, r.c1, n, half, M, words)
                      : aext2_sumcheck_batched_fold_ffi(cur, other, r.c0, r.c1, n, half, M);
        if (rc != MB_OK) return rc;
        // the next message's first label is absorbed while the fold runs
        label_absorbed = round + 1 < arity;
        if (label_absorbed) t.begin_append(SP_LABEL(L_MSG));
        uint64_t* tmp = cur; cur = other; other = tmp;
    }
    // reveals f_i(R): element 0 of every leaf's f table
    std::vector<uint64_t> fe(2 * (size_t)M);
    {
        MB_KERNEL("same_point_reveals");
        first_f_kernel<<<(2 * M + 127) / 128, 128, 0, MB_STREAM>>>(cur, n, M, buf.sums);
    }
    MB_CUDA(cudaMemcpyAsync(fe.data(), buf.sums, sizeof(uint64_t) * 2 * (size_t)M, cudaMemcpyDeviceToHost, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    E2 fin{0, 0};
    for (int i = 0; i < M; i++) {
        t.append_ext2(SP_LABEL(L_FEVAL), fe[2 * i], fe[2 * i + 1]);
        h_f_evals[2 * i] = fe[2 * i];
        h_f_evals[2 * i + 1] = fe[2 * i + 1];
    }
    for (int i = 0; i < M; i++) {
        const E2 eq_i = eq_eval(h_pts + 2 * (size_t)arity * i, R.data(), arity);
        fin = agl::e2_add(fin, agl::e2_mul(alphas[i], e2c(agl::e2_mul(eq_i, ld(fe.data() + 2 * i)))));
    }
    fin = e2c(fin);
    h_final_eval[0] = fin.c0;
    h_final_eval[1] = fin.c1;
    return MB_OK;
}

// verify_same_point for instances of any arity <= num_vars: pts are concatenated (arity[i] pairs each).
int same_point_verify(int M, int N, const int* arity, const uint64_t* h_pts, const uint64_t* h_vals, const uint64_t* round_msgs,
                      const uint64_t* f_evals, const uint64_t* final_eval, AglTranscript& t, uint64_t* challenges, int* ok) {
    *ok = 0;
    if (M < 1 || N < 1 || N > 62) return MB_ERR_ARG;
    t.append_u64(SP_LABEL(L_NUM_VAR), (uint64_t)N);
    t.append_u64(SP_LABEL(L_NUM_INST), (uint64_t)M);
    std::vector<size_t> off(M);
    size_t o = 0;
    for (int i = 0; i < M; i++) {
        if (arity[i] < 0 || arity[i] > N) return MB_ERR_ARG;
        off[i] = o;
        t.append_u64(SP_LABEL(L_ARITY), (uint64_t)arity[i]);
        for (int k = 0; k < arity[i]; k++) t.append_ext2(SP_LABEL(L_R), h_pts[o + 2 * k], h_pts[o + 2 * k + 1]);
        t.append_ext2(SP_LABEL(L_Y), h_vals[2 * i], h_vals[2 * i + 1]);
        o += 2 * (size_t)arity[i];
    }
    const E2 alpha = challenge(t, SP_LABEL(L_ALPHA));
    std::vector<E2> alphas(M), R(N);
    E2 pw{1, 0}, current{0, 0};
    for (int i = 0; i < M; i++) {
        alphas[i] = pw;
        pw = e2c(agl::e2_mul(pw, alpha));
        const E2 weight{(uint64_t)1 << (N - arity[i]), 0};
        current = agl::e2_add(current, agl::e2_mul(alphas[i], e2c(agl::e2_mul(ld(h_vals + 2 * i), weight))));
    }
    current = e2c(current);
    const E2 inv2 = e2c(agl::e2_inv(E2{2, 0})), one{1, 0}, two{2, 0};
    for (int round = 0; round < N; round++) {
        E2 m[3];
        for (int c = 0; c < 3; c++) m[c] = ld(round_msgs + ((size_t)round * 3 + c) * 2);
        const E2 sum = e2c(agl::e2_add(m[0], m[1]));
        if (sum.c0 != current.c0 || sum.c1 != current.c1) return MB_OK;
        for (int c = 0; c < 3; c++) t.append_ext2(SP_LABEL(L_MSG), m[c].c0, m[c].c1);
        const E2 r = challenge(t, SP_LABEL(L_CH));
        R[round] = r;
        if (challenges) { challenges[2 * round] = r.c0; challenges[2 * round + 1] = r.c1; }
        // Lagrange through 0, 1, 2 (same_point_sumcheck.rs:886-904)
        const E2 xm1 = agl::e2_sub(r, one), xm2 = agl::e2_sub(r, two);
        const E2 l0 = agl::e2_mul(e2c(agl::e2_mul(xm1, xm2)), inv2);
        const E2 l1 = agl::e2_sub(E2{0, 0}, agl::e2_mul(r, xm2));
        const E2 l2 = agl::e2_mul(e2c(agl::e2_mul(r, xm1)), inv2);
        current = e2c(agl::e2_add(agl::e2_add(agl::e2_mul(e2c(l0), m[0]), agl::e2_mul(e2c(l1), m[1])), agl::e2_mul(e2c(l2), m[2])));
    }
    E2 expected{0, 0};
    for (int i = 0; i < M; i++) t.append_ext2(SP_LABEL(L_FEVAL), f_evals[2 * i], f_evals[2 * i + 1]);
    for (int i = 0; i < M; i++) {
        const E2 eq_i = eq_eval(h_pts + off[i], R.data(), arity[i]);
        expected = agl::e2_add(expected, agl::e2_mul(alphas[i], e2c(agl::e2_mul(eq_i, ld(f_evals + 2 * i)))));
    }
    expected = e2c(expected);
    const E2 fin = ld(final_eval);
    *ok = current.c0 == expected.c0 && current.c1 == expected.c1 && fin.c0 == expected.c0 && fin.c1 == expected.c1;
    return MB_OK;
}

}  // namespace mbhost

extern "C" {

// The whole same-point sumcheck for num_leaves instances of one arity (the reference's device path,
// same_point_sumcheck.rs:1334-1553). h_claim_pts[num_leaves][arity][2], h_claim_vals[num_leaves][2]; witness on the
// device: kind 0 binary packed (d_w0[num_leaves][words], words = max(1, 2^(arity - 6))), 1 ternary single chunk
// (d_w0 = +1 masks, d_w1 = -1 masks), 2 extension tables (d_w0[num_leaves][2^arity][2]). `transcript`: a handle
// from agl_transcript_create, advanced by the proof. Host outputs: round_msgs[arity][3][2], challenges[arity][2]
// (may be null), f_evals[num_leaves][2], final_eval[2]. Needs 2 x num_leaves x 2^arity x 32 bytes of device memory.
int agl_same_point_prove_device_ffi(int num_leaves, int arity, const uint64_t* h_claim_pts, const uint64_t* h_claim_vals, int kind,
                                    const uint64_t* d_w0, const uint64_t* d_w1, void* transcript, uint64_t* h_round_msgs,
                                    uint64_t* h_challenges, uint64_t* h_f_evals, uint64_t* h_final_eval) {
    if (!transcript) return MB_ERR_ARG;
    return mbhost::same_point_prove(num_leaves, arity, h_claim_pts, h_claim_vals, kind, d_w0, d_w1,
                                    *static_cast<mbhost::AglTranscript*>(transcript), h_round_msgs, h_challenges, h_f_evals,
                                    h_final_eval);
}

// The claims y_i = f_i(r_i) of the leaves (the witness' multilinear extension at its claim point), computed on the
// device with the kernels of the proof: h_claim_vals[num_leaves][2]. Arguments as agl_same_point_prove_device_ffi.
int agl_same_point_claims_device_ffi(int num_leaves, int arity, const uint64_t* h_claim_pts, int kind, const uint64_t* d_w0,
                                     const uint64_t* d_w1, uint64_t* h_claim_vals) {
    return mbhost::same_point_claims(num_leaves, arity, h_claim_pts, kind, d_w0, d_w1, h_claim_vals);
}

// verify_same_point on the host (same_point_sumcheck.rs:161-219); instances may have different arities
// (h_claim_pts holds arity[i] pairs per instance, back to back). *ok = 1 when the proof is accepted; the
// challenges (num_vars pairs) are written when `challenges` is not null.
int agl_same_point_verify_ffi(int num_instances, int num_vars, const int* arity, const uint64_t* h_claim_pts,
                              const uint64_t* h_claim_vals, const uint64_t* round_msgs, const uint64_t* f_evals,
                              const uint64_t* final_eval, void* transcript, uint64_t* challenges, int* ok) {
    if (!transcript || !ok || !arity || !h_claim_pts || !h_claim_vals || !round_msgs || !f_evals || !final_eval) return MB_ERR_ARG;
    return mbhost::same_point_verify(num_instances, num_vars, arity, h_claim_pts, h_claim_vals, round_msgs, f_evals, final_eval,
                                     *static_cast<mbhost::AglTranscript*>(transcript), challenges, ok);
}

}  // extern "C"
