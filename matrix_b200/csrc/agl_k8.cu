// C-ABI: the K = F_q[Theta]/(Theta^8 - 3) product sumcheck and its table helpers
// (reference: almost-goldilocks-cuda-rs/src/ffi.rs:65-75, definitions
// almost-goldilocks-cuda-rs/cuda/wrapper.cu:3815-3905; Rust callers
// zk-torch-4/src/morpheus/piop/gpu.rs). Tables are device arrays of 64-byte
// elements; challenges, points and sums are host arrays of 8 words per element.
// The sums come back through one pinned copy; everything runs on the caller's
// per-thread stream.
#include <cstring>
#include "agl_k8.cuh"

using namespace mb;
using namespace mb::k8;

namespace {

struct Scratch {
    uint64_t* partial = nullptr;  // [grid][MAXTAB + 1][8]
    uint64_t* sums = nullptr;     // [(MAXTAB + 1) * 8]
    unsigned int* counter = nullptr;
    int grid_cap = 0;
    ~Scratch() {}
};

// Per host thread and device: partial rows for the largest grid, the sums and the ticket counter.
int scratch_for(int grid, Scratch** out) {
    static thread_local Scratch s[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MB_ERR_CUDA;
    Scratch& sc = s[dev];
    if (grid > sc.grid_cap) {
        // allocate into temporaries: the thread's scratch changes only when everything succeeded, so a failed
        // allocation leaves the old (smaller, still valid) buffers or none, never a dangling pointer
        const int cap = sm_count() * 8;
        const int want = grid > cap ? grid : cap;
        const size_t row = (size_t)(MAXTAB + 1) * 8;
        uint64_t *partial = nullptr, *sums = nullptr;
        if (pool_alloc((void**)&partial, sizeof(uint64_t) * row * want) != cudaSuccess) return MB_ERR_CUDA;
        if (pool_alloc((void**)&sums, sizeof(uint64_t) * (row + 2)) != cudaSuccess) {
            pool_free(partial);
            return MB_ERR_CUDA;
        }
        if (cudaMemsetAsync(sums + row, 0, 2 * sizeof(uint64_t), MB_STREAM) != cudaSuccess) {
            pool_free(partial);
            pool_free(sums);
            return MB_ERR_CUDA;
        }
        if (sc.partial) { pool_free(sc.partial); pool_free(sc.sums); }
        sc.partial = partial;
        sc.sums = sums;
        sc.counter = reinterpret_cast<unsigned int*>(sums + row);
        sc.grid_cap = want;
    }
    *out = &sc;
    return MB_OK;
}

int fetch_sums(Scratch* sc, int d, uint64_t* h_out) {
    uint64_t* h = pinned_scratch();  // 64 words; (d + 1) * 8 <= 56
    if (!h) return MB_ERR_CUDA;
    MB_CUDA(cudaMemcpyAsync(h, sc->sums, sizeof(uint64_t) * (size_t)(d + 1) * 8, cudaMemcpyDeviceToHost, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    std::memcpy(h_out, h, sizeof(uint64_t) * (size_t)(d + 1) * 8);
    return MB_OK;
}

Elem elem_from(const uint64_t* h) {
    Elem e;
    for (int i = 0; i < 8; i++) e.c[i] = h[i];
    return e;
}

}  // namespace

extern "C" {

// h_out[(d + 1) * 8]: s[t] = sum_k prod_j (T_j[2k] + t (T_j[2k+1] - T_j[2k])), t = 0..d. -3: too many tables / degree.
int agl_mpiop_sc_round(const uint64_t* const* h_tabs, int ntab, uint64_t len, int d, uint64_t* h_out) {
    if (!h_tabs || !h_out || ntab < 1 || d < 0 || len < 2 || (len & 1)) return MB_ERR_ARG;
    if (ntab > MAXTAB || d > MAXTAB) return -3;
    Tabs T;
    T.ntab = ntab;
    for (int j = 0; j < MAXTAB; j++) T.t[j] = j < ntab ? h_tabs[j] : nullptr;
    const uint64_t npairs = len / 2;
    const int grid = grid_for(npairs * 8, 256, 4);
    Scratch* sc;
    int rc = scratch_for(grid, &sc);
    if (rc != MB_OK) return rc;
    {
        MB_KERNEL("k8_sc_round");
        sc_round_kernel<<<grid, 256, 0, MB_STREAM>>>(T, npairs, d, sc->partial, sc->counter, sc->sums);
    }
    if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
    return fetch_sums(sc, d, h_out);
}

// d_out[k] = d_in[2k] + r (d_in[2k+1] - d_in[2k]), k < len / 2.
int agl_mpiop_sc_fold(const uint64_t* d_in, uint64_t* d_out, uint64_t len, const uint64_t* h_r) {
    if (!d_in || !d_out || !h_r || len < 2 || (len & 1)) return MB_ERR_ARG;
    const uint64_t nout = len / 2;
    {
        MB_KERNEL("k8_sc_fold");
        sc_fold_kernel<<<grid_for(nout * 8, 256, 4), 256, 0, MB_STREAM>>>(d_in, d_out, nout, elem_from(h_r));
    }
    return finish_async();
}

// Folds the ntab tables (length len) with r into h_outs (length len / 2) and returns the d + 1 sums of the
// next round over the folded tables.
int agl_mpiop_sc_fold_round(const uint64_t* const* h_tabs, uint64_t* const* h_outs, int ntab, uint64_t len,
                            const uint64_t* h_r, int d, uint64_t* h_out) {
    if (!h_tabs || !h_outs || !h_r || !h_out || ntab < 1 || d < 0) return MB_ERR_ARG;
    if (ntab > MAXTAB || d > MAXTAB || len < 4 || (len & 3)) return -3;
    Tabs T;
    OutTabs O;
    T.ntab = ntab;
    for (int j = 0; j < MAXTAB; j++) {
        T.t[j] = j < ntab ? h_tabs[j] : nullptr;
        O.t[j] = j < ntab ? h_outs[j] : nullptr;
    }
    const uint64_t nquads = len / 4;
    const int grid = grid_for(nquads * 8, 256, 4);
    Scratch* sc;
    int rc = scratch_for(grid, &sc);
    if (rc != MB_OK) return rc;
    {
        MB_KERNEL("k8_sc_fold_round");
        sc_fold_round_kernel<<<grid, 256, 0, MB_STREAM>>>(T, O, nquads, elem_from(h_r), d, sc->partial, sc->counter, sc->sums);
    }
    if (cudaGetLastError() != cudaSuccess) return MB_ERR_CUDA;
    return fetch_sums(sc, d, h_out);
}

// d_out[2^n] = eq(x, point), bit j of the index matching point[j] (field8.rs:160-182).
int agl_mpiop_eq(const uint64_t* h_point, int n, uint64_t* d_out) {
    if (!d_out || n < 0 || n > 30 || (n > 0 && !h_point)) return MB_ERR_ARG;
    const uint64_t one[8] = {1, 0, 0, 0, 0, 0, 0, 0};
    uint64_t* tmp = nullptr;
    if (n > 0 && pool_alloc((void**)&tmp, ((size_t)1 << n) * 64) != cudaSuccess) return MB_ERR_CUDA;
    uint64_t* bufs[2] = {d_out, tmp};
    int cur = (n % 2 == 0) ? 0 : 1;  // the last step lands in d_out
    int rc = MB_OK;
    if (cudaMemcpyAsync(bufs[cur], one, 64, cudaMemcpyHostToDevice, MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
    if (cudaStreamSynchronize(MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;  // `one` is on this stack frame
    uint64_t half = 1;
    for (int j = n - 1; j >= 0 && rc == MB_OK; j--) {
        MB_KERNEL("k8_eq_double");
        eq_double_kernel<<<grid_for(half * 8, 256, 4), 256, 0, MB_STREAM>>>(bufs[cur], bufs[cur ^ 1], half, elem_from(h_point + 8 * j));
        cur ^= 1;
        half <<= 1;
    }
    if (rc == MB_OK) rc = finish_async();
    pool_free(tmp);
    return rc;
}

int agl_mpiop_eq_outer(const uint64_t* d_lo, int nlo, const uint64_t* d_hi, int nhi, uint64_t* d_out) {
    if (!d_lo || !d_hi || !d_out || nlo < 0 || nhi < 0 || nlo + nhi > 30) return MB_ERR_ARG;
    const uint64_t n = (uint64_t)1 << (nlo + nhi);
    MB_KERNEL("k8_eq_outer");
    eq_outer_kernel<<<grid_for(n * 8, 256, 4), 256, 0, MB_STREAM>>>(d_lo, nlo, d_hi, n, d_out);
    return finish_async();
}

// d_out[x] += c * d_in[x]
int agl_mpiop_axpy(uint64_t* d_out, const uint64_t* d_in, uint64_t n, const uint64_t* h_c) {
    if (!d_out || !d_in || !h_c) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("k8_axpy");
    axpy_kernel<<<grid_for(n * 8, 256, 4), 256, 0, MB_STREAM>>>(d_out, d_in, n, elem_from(h_c));
    return finish_async();
}

int agl_mpiop_lift(const uint64_t* d_in, uint64_t n, uint64_t* d_out) {
    if (!d_in || !d_out) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("k8_lift");
    lift_kernel<<<grid_for(n * 8, 256, 8), 256, 0, MB_STREAM>>>(d_in, n, d_out);
    return finish_async();
}

// ---- helpers over base-field tables (wrapper.cu:3753-3837) ----
namespace {
VarMap make_map(const int* pos, int n) {
    VarMap m;
    m.n = n;
    for (int j = 0; j < MAXV; j++) m.pos[j] = j < n ? pos[j] : 0;
    return m;
}
// out (device, nrest elements) = partial evaluation; `e` is a device K table of 2^nfix_v elements
int run_pe(const uint64_t* d_vals, const VarMap& rest, const VarMap& fix, const uint64_t* d_e, uint64_t* d_out) {
    const uint64_t nrest = (uint64_t)1 << rest.n, nfix = (uint64_t)1 << fix.n;
    uint64_t want = (uint64_t)sm_count() * 8;
    uint64_t gx = nrest < want ? nrest : want;
    uint64_t gy = (want + gx - 1) / gx;
    const uint64_t max_gy = (nfix + 31) / 32;
    if (gy > max_gy) gy = max_gy;
    if (gy > 65535) gy = 65535;
    if (gy < 1) gy = 1;
    uint64_t* partial = nullptr;
    MB_CUDA(pool_alloc((void**)&partial, sizeof(uint64_t) * 8 * nrest * gy));
    {
        MB_KERNEL("k8_pe");
        dim3 grid((unsigned)gx, (unsigned)gy);
        pe_kernel<<<grid, 256, 0, MB_STREAM>>>(d_vals, rest, fix, d_e, nrest, nfix, partial);
    }
    {
        MB_KERNEL("k8_sum_rows");
        sum_rows_kernel<<<grid_for(nrest * 8, 256, 4), 256, 0, MB_STREAM>>>(partial, nrest, (int)gy, d_out);
    }
    int rc = finish_async();
    pool_free(partial);
    return rc;
}
}  // namespace

// d_out[r] = sum_f d_vals[deposit(r, rest_pos) | deposit(f, fix_pos)] d_e[f]; rest_pos / fix_pos are host arrays of bit positions.
int agl_mpiop_pe(const uint64_t* d_vals, const int* rest_pos, int nrest_v, const int* fix_pos, int nfix_v, const uint64_t* d_e,
                 uint64_t* d_out) {
    if (!d_vals || !d_e || !d_out || nrest_v < 0 || nfix_v < 0 || nrest_v > MAXV || nfix_v > MAXV || nrest_v + nfix_v > 40 ||
        (nrest_v && !rest_pos) || (nfix_v && !fix_pos))
        return MB_ERR_ARG;
    return run_pe(d_vals, make_map(rest_pos, nrest_v), make_map(fix_pos, nfix_v), d_e, d_out);
}

// h_out[8] = sum_x d_vals[x] eq(x, h_point): the multilinear extension of a base-field table at a K point.
// The point is split in two: T[h] = sum_l eq_lo[l] vals[h 2^nlo + l], then sum_h eq_hi[h] T[h].
int agl_mpiop_mle(const uint64_t* d_vals, const uint64_t* h_point, int n, uint64_t* h_out) {
    if (!d_vals || !h_out || n < 0 || n > 40 || (n && !h_point)) return MB_ERR_ARG;
    const int nlo = n / 2, nhi = n - nlo;
    uint64_t *e_lo = nullptr, *e_hi = nullptr, *T = nullptr, *partial = nullptr;
    MB_CUDA(pool_alloc((void**)&e_lo, (size_t)64 << nlo));
    int rc = MB_OK;
    if (pool_alloc((void**)&e_hi, (size_t)64 << nhi) != cudaSuccess) rc = MB_ERR_CUDA;
    if (rc == MB_OK && pool_alloc((void**)&T, (size_t)64 << nhi) != cudaSuccess) rc = MB_ERR_CUDA;
    const uint64_t nh = (uint64_t)1 << nhi;
    const int grid = grid_for(nh * 8, 256, 4);
    if (rc == MB_OK && pool_alloc((void**)&partial, sizeof(uint64_t) * 8 * (size_t)(grid + 1)) != cudaSuccess) rc = MB_ERR_CUDA;
    if (rc == MB_OK) rc = agl_mpiop_eq(h_point, nlo, e_lo);
    if (rc == MB_OK) rc = agl_mpiop_eq(h_point ? h_point + 8 * nlo : nullptr, nhi, e_hi);
    if (rc == MB_OK) {
        int lo_pos[MAXV], hi_pos[MAXV];
        for (int j = 0; j < nlo; j++) lo_pos[j] = j;
        for (int j = 0; j < nhi; j++) hi_pos[j] = nlo + j;
        rc = run_pe(d_vals, make_map(hi_pos, nhi), make_map(lo_pos, nlo), e_lo, T);
    }
    if (rc == MB_OK) {
        {
            MB_KERNEL("k8_dot");
            dot_kernel<<<grid, 256, 0, MB_STREAM>>>(e_hi, T, nh, partial);
        }
        {
            MB_KERNEL("k8_sum_rows");
            sum_rows_kernel<<<1, 32, 0, MB_STREAM>>>(partial, 1, grid, partial + 8 * (size_t)grid);
        }
        uint64_t* h = pinned_scratch();
        if (!h || cudaMemcpyAsync(h, partial + 8 * (size_t)grid, 64, cudaMemcpyDeviceToHost, MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
        if (rc == MB_OK) rc = finish_sync();
        if (rc == MB_OK) std::memcpy(h_out, h, 64);
    }
    pool_free(e_lo); pool_free(e_hi); pool_free(T); pool_free(partial);
    return rc;
}

// d_out[x] = d_in[sum_j ((x >> pos[j]) & 1) << j], x < n; pos is a host array of nv bit positions.
int agl_mpiop_gather(const uint64_t* d_in, const int* pos, int nv, uint64_t n, uint64_t* d_out) {
    if (!d_in || !d_out || nv < 0 || nv > MAXV || (nv && !pos)) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("k8_gather");
    gather_kernel<<<grid_for(n * 8, 256, 8), 256, 0, MB_STREAM>>>(d_in, make_map(pos, nv), n, d_out);
    return finish_async();
}

// d_out[i] = d_table[(d_sel[i] >> shift) & mask]
int agl_mpiop_sel_lookup(const uint64_t* d_sel, uint64_t n, int shift, uint64_t mask, const uint64_t* d_table, uint64_t* d_out) {
    if (!d_sel || !d_table || !d_out || shift < 0 || shift > 63) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("k8_sel_lookup");
    sel_lookup_kernel<<<grid_for(n * 8, 256, 8), 256, 0, MB_STREAM>>>(d_sel, n, shift, mask, d_table, d_out);
    return finish_async();
}

}  // extern "C"
