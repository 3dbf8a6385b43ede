// The device sequence of one einsum block's proof in one call (Einsum::prove_gpu,
// zk-torch-4/src/basicblock/einsum.rs:1168-1310): per operand the partial evaluation at the output
// point's coordinates that belong to it alone (plain when those are its low variables, fused with the bit
// permutation of partial_eval.rs:283-321 otherwise), the eq table of the output variables two operands
// share, the tables tiled over the variables an operand does not depend on, and one linear sumcheck on the
// caller's transcript (gpu_prover.rs:26-112).
//
// The reference drives these steps from Rust, one synchronising FFI call each. Here the whole sequence is
// queued on the calling thread's stream: the small vectors (the point's coordinates per operand) go up in
// one copy from page-locked memory, nothing synchronises before the sumcheck's first round message, and the
// scratch comes from the stream-ordered pool. The per-operand plan (variable counts, index tables) is the
// caller's: it depends on the equation and the shapes only (matrix_b200/layer_trace.py builds it once).
#include <vector>
#include "../agl_traits.cuh"
#include "../eq_kernels.cuh"
#include "../fused_peval_kernels.cuh"
#include "../peval_kernels.cuh"

using namespace mb;
using namespace mb::sc;

extern "C" {

// One operand of the block. d_src: 2^n base-field words, index order as the equation names it. The first m
// variables of the operand's NEW order (given by the index tables; the identity when d_lut_lo is null) are fixed
// to point coordinates fixed_idx[0 .. m); the next n - m are table variables, the lowest n_mine... of the block's
// `rounds` variables; the table is tiled over the others.
typedef struct mb_einsum_operand {
    const uint64_t* d_src;
    const uint32_t* d_lut_lo;   // split index tables of the permutation (partial_eval.rs:283-321), or null
    const uint32_t* d_lut_hi;
    int n;                      // variables of the operand
    int m;                      // of which fixed to coordinates of the point
    int fixed_off;              // offset of this operand's m indices in fixed_idx
    int reserved;
} mb_einsum_operand;

int agl_sumcheck_prove_device_ffi(const uint64_t* d_tables, int d, int num_var, int base_field, void* transcript,
                                  uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval);
}

namespace {

__global__ void lift_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        agl::e2_store(out + 2 * i, agl::E2{agl::canon(in[i]), 0});
}
__global__ void ones_kernel(uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) agl::e2_store(out + 2 * i, agl::E2{1, 0});
}

struct Scratch {
    std::vector<void*> ptrs;
    ~Scratch() { for (void* p : ptrs) pool_free(p); }
    uint64_t* get(size_t words) {
        void* p = nullptr;
        if (pool_alloc(&p, sizeof(uint64_t) * (words ? words : 1)) != cudaSuccess) return nullptr;
        ptrs.push_back(p);
        return static_cast<uint64_t*>(p);
    }
};

// Page-locked staging of the calling thread for the point's coordinates (grown on demand).
uint64_t* staging(size_t words) {
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

// Repeat the first 2^have elements of an extension table up to 2^want (new high variables).
int tile(uint64_t* d_table, int have, int want) {
    for (int k = have; k < want; k++)
        MB_CUDA(cudaMemcpyAsync(d_table + ((size_t)2 << k), d_table, (size_t)16 << k, cudaMemcpyDeviceToDevice, MB_STREAM));
    return MB_OK;
}

}  // namespace

extern "C" {

// num_operands tables and the eq table of the shared output variables (or a table of ones when there are none)
// form a product of d = num_operands + 1 tables over `rounds` variables; the sum over the hypercube is proved on
// `transcript` (an agl_transcript handle). h_point: the output point, (c0, c1) per variable; fixed_idx / shared_idx
// index its variables. Host outputs as agl_sumcheck_prove_device_ffi: round_msgs[rounds][d + 1][2],
// challenges[rounds][2] (may be null), final_evals[d][2] (may be null), final_eval[2].
int agl_einsum_prove_device_ffi(int num_operands, const mb_einsum_operand* ops, const int* fixed_idx, int rounds, int num_shared,
                                const int* shared_idx, const uint64_t* h_point, int point_vars, void* transcript,
                                uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_evals, uint64_t* final_eval) {
    if (num_operands < 1 || num_operands > MAX_D - 1 || !ops || rounds < 0 || rounds > 30 || num_shared < 0 || num_shared > rounds ||
        (num_shared && !shared_idx) || (point_vars && !h_point) || !transcript || !round_msgs || !final_eval)
        return MB_ERR_ARG;
    const int d = num_operands + 1;
    const size_t size = (size_t)1 << rounds;
    // the small vectors: per operand its m coordinates, then the shared ones; one upload
    size_t small_words = 2 * (size_t)num_shared + 2;
    for (int k = 0; k < num_operands; k++) {
        const mb_einsum_operand& o = ops[k];
        if (!o.d_src || o.n < 0 || o.n > 30 || o.m < 0 || o.m > o.n || o.n - o.m > rounds || (o.m && !fixed_idx) ||
            ((o.d_lut_lo == nullptr) != (o.d_lut_hi == nullptr)))
            return MB_ERR_ARG;
        small_words += 2 * (size_t)o.m;
    }
    uint64_t* h_small = staging(small_words);
    if (!h_small) return MB_ERR_CUDA;
    std::vector<size_t> r_off(num_operands);
    size_t w = 0;
    for (int k = 0; k < num_operands; k++) {
        r_off[k] = w;
        for (int i = 0; i < ops[k].m; i++) {
            const int v = fixed_idx[ops[k].fixed_off + i];
            if (v < 0 || v >= point_vars) return MB_ERR_ARG;
            h_small[w++] = h_point[2 * v];
            h_small[w++] = h_point[2 * v + 1];
        }
    }
    const size_t shared_off = w;
    for (int i = 0; i < num_shared; i++) {
        const int v = shared_idx[i];
        if (v < 0 || v >= point_vars) return MB_ERR_ARG;
        h_small[w++] = h_point[2 * v];
        h_small[w++] = h_point[2 * v + 1];
    }
    const size_t one_off = w;
    h_small[w++] = 1;
    h_small[w++] = 0;

    Scratch sc;
    uint64_t* d_small = sc.get(small_words);
    uint64_t* tables = sc.get((size_t)d * size * 2);
    if (!d_small || !tables) return MB_ERR_CUDA;
    MB_CUDA(cudaMemcpyAsync(d_small, h_small, sizeof(uint64_t) * small_words, cudaMemcpyHostToDevice, MB_STREAM));

    for (int k = 0; k < num_operands; k++) {
        const mb_einsum_operand& o = ops[k];
        uint64_t* dst = tables + (size_t)k * size * 2;
        const int mine = o.n - o.m;
        int rc = MB_OK;
        if (!o.d_lut_lo && o.m == 0) {
            MB_KERNEL("einsum_lift");
            lift_kernel<<<grid_for((size_t)1 << o.n, 256, 8), 256, 0, MB_STREAM>>>(o.d_src, dst, (size_t)1 << o.n);
            rc = finish_async();
        } else if (!o.d_lut_lo) {
            // the fixed variables are the operand's low bits: a plain partial evaluation, then into place
            uint64_t* out = sc.get((size_t)2 << (o.n - 1));
            uint64_t* tmp = sc.get((size_t)2 << (o.n - 1));
            if (!out || !tmp) return MB_ERR_CUDA;
            rc = pe::partial_eval<AglBase, AglExt2>(o.d_src, out, tmp, d_small + r_off[k], o.n, o.m, MB_STREAM);
            if (rc == MB_OK && cudaMemcpyAsync(dst, out, (size_t)16 << mine, cudaMemcpyDeviceToDevice, MB_STREAM) != cudaSuccess)
                rc = MB_ERR_CUDA;
        } else {
            const uint64_t* eq_ptr = d_small + one_off;
            if (o.m) {
                uint64_t* eqt = sc.get((size_t)2 << o.m);
                uint64_t* eqs = sc.get(2 * (((size_t)1 << (o.m / 2)) + ((size_t)1 << (o.m - o.m / 2))));
                if (!eqt || !eqs) return MB_ERR_CUDA;
                rc = eq::build<AglExt2>(d_small + r_off[k], eqt, eqs, o.m, MB_STREAM);
                eq_ptr = eqt;
            }
            if (rc == MB_OK)
                rc = fp::launch<AglBase, AglExt2>(o.d_src, dst, eq_ptr, o.d_lut_lo, o.d_lut_hi, o.n, o.m, o.n / 2, 1 << mine, MB_STREAM);
        }
        if (rc != MB_OK) return rc;
        rc = tile(dst, mine, rounds);
        if (rc != MB_OK) return rc;
    }
    uint64_t* last = tables + (size_t)(d - 1) * size * 2;
    if (num_shared) {
        uint64_t* eqs = sc.get(2 * (((size_t)1 << (num_shared / 2)) + ((size_t)1 << (num_shared - num_shared / 2))));
        if (!eqs) return MB_ERR_CUDA;
        int rc = eq::build<AglExt2>(d_small + shared_off, last, eqs, num_shared, MB_STREAM);
        if (rc != MB_OK) return rc;
        rc = tile(last, num_shared, rounds);
        if (rc != MB_OK) return rc;
    } else {
        MB_KERNEL("einsum_ones");
        ones_kernel<<<grid_for(size, 256, 8), 256, 0, MB_STREAM>>>(last, size);
        int rc = finish_async();
        if (rc != MB_OK) return rc;
    }
    return agl_sumcheck_prove_device_ffi(tables, d, rounds, 0, transcript, round_msgs, challenges, final_evals, final_eval);
}

}  // extern "C"
