// C-ABI: sparse boolean-check sumcheck over the almost-Goldilocks extension (reference declarations
// almost-goldilocks-cuda-rs/src/ffi.rs:140-158, definitions almost-goldilocks-cuda-rs/cuda/wrapper.cu:2650-2981,
// Rust state almost-goldilocks-cuda-rs/src/sumcheck_prover.rs:2186-2340).
//
//     sum_t w_t sum_x eq(x) v_t(x) (v_t(x) - 1)
//
// over sparse tables v_t given as sorted (position, value) lists, one slice of the entry arrays per term
// (term_off). A round binds the LOW position bit: entries 2r and 2r + 1 of one term merge into entry r.
//   flags[i] = 1 when entry i opens a group (the first of its term, or not the odd partner of its predecessor)
//   gid      = exclusive prefix sum of flags over all entries; total = number of groups
//   message  = sum over groups of w_t a_c (a_c - 1) e_c at c = 0..3, a_c = v0 + c (v1 - v0), e_c likewise
//              from eq[2r], eq[2r + 1]
//   fold     = out[gid] = (r, v0 + ch (v1 - v0)); new term offsets = gid at the old offsets
//
// Launch structure: the entry array is cut into tiles of 2048 entries regardless of the terms (a thread
// finds its term by a binary search of the offsets held in shared memory), so the grid does not depend on
// how the entries are spread over the terms, and one kernel marks, counts and forms the message; a single
// small block scans the tile counts and adds the tile partial sums on the device (the message is one
// 72-byte read-back); a third pass writes gid. The caller's d_partial and d_scan_scratch are not needed.
#include "agl_field.cuh"
#include "common.cuh"
#include "prof.cuh"

using namespace mb;

namespace {

using agl::E2;
constexpr int TILE = 2048, THREADS = 256, PER_THREAD = TILE / THREADS, OFF_CACHE = 4096;

__device__ __forceinline__ E2 ld(const uint64_t* p, uint64_t i) { return agl::e2_load(p + 2 * i); }
__device__ __forceinline__ void st(uint64_t* p, uint64_t i, E2 v) { agl::e2_store(p + 2 * i, agl::e2_canon(v)); }
__device__ __forceinline__ E2 zero() { return E2{0, 0}; }

// Exact sums of extension products a b (three 160-bit integer sums), reduced once: at most 64 products.
struct LazyE2 {
    gl::Acc s00, s11, s01;
};
__device__ __forceinline__ LazyE2 lazy_zero() { return LazyE2{gl::acc_zero(), gl::acc_zero(), gl::acc_zero()}; }
__device__ __forceinline__ void lazy_mul(LazyE2& q, E2 a, E2 b) {
    gl::acc_mul(q.s00, a.c0, b.c0);
    gl::acc_mul(q.s11, a.c1, b.c1);
    gl::acc_mul(q.s01, a.c0, b.c1);
    gl::acc_mul(q.s01, a.c1, b.c0);
}
__device__ __forceinline__ E2 lazy_reduce(const LazyE2& q) {
    return E2{agl::add(agl::acc_reduce(q.s00), agl::mul_small(agl::acc_reduce(q.s11), 3)), agl::acc_reduce(q.s01)};
}

// Largest t in [0, n_terms) with off[t] <= i (the term whose slice holds entry i; empty terms are skipped).
__device__ __forceinline__ int find_term(const uint32_t* off, int n_terms, uint32_t i) {
    int lo = 0, hi = n_terms - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (off[mid] <= i) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ E2 warp_sum(E2 v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const E2 u{__shfl_down_sync(0xffffffffu, v.c0, o), __shfl_down_sync(0xffffffffu, v.c1, o)};
        v = agl::e2_add(v, u);
    }
    return v;
}

// One tile per block: flags, the tile's group count and its share of the message.
__global__ void __launch_bounds__(THREADS, 2) bool_mark_msg_kernel(const uint32_t* __restrict__ idx, const uint64_t* __restrict__ val,
                                                                const uint32_t* __restrict__ term_off, const uint64_t* __restrict__ w,
                                                                const uint64_t* __restrict__ eq, int n_terms, uint32_t n,
                                                                uint32_t* __restrict__ flags, uint32_t* __restrict__ tile_count,
                                                                uint64_t* __restrict__ tile_part) {
    __shared__ uint32_t soff[OFF_CACHE];
    __shared__ uint64_t sh[THREADS / 32][8];
    __shared__ uint32_t shc[THREADS / 32];
    const int tid = threadIdx.x;
    const bool cached = n_terms + 1 <= OFF_CACHE;
    if (cached)
        for (int t = tid; t <= n_terms; t += THREADS) soff[t] = term_off[t];
    __syncthreads();
    const uint32_t* off = cached ? soff : term_off;
    const uint32_t covered = off[n_terms];   // entries past the last term belong to no group

    // The weight of a term is applied once per run of entries of that term: S[c] collects a_c (a_c - 1) e_c as exact
    // sums (a thread has at most eight entries), acc[c] += w_t S[c] when the term changes and at the end.
    E2 acc[4];
    LazyE2 S[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        acc[k] = zero();
        S[k] = lazy_zero();
    }
    int cur_t = -1;
    auto flush = [&]() {
        if (cur_t < 0) return;
        const E2 wt = ld(w, cur_t);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            acc[k] = agl::e2_add(acc[k], agl::e2_mul_lazy(wt, lazy_reduce(S[k])));
            S[k] = lazy_zero();
        }
    };
    uint32_t count = 0;
    const uint32_t base = blockIdx.x * (uint32_t)TILE;
#pragma unroll 1
    for (int j = 0; j < PER_THREAD; j++) {
        const uint32_t i = base + j * THREADS + tid;
        if (i >= n) break;
        if (i >= covered) {
            flags[i] = 0;
            continue;
        }
        const int t = find_term(off, n_terms, i);
        const uint32_t s = off[t], e = off[t + 1];
        const uint32_t pos = idx[i];
        const bool leader = (i == s) || !((pos & 1u) && idx[i - 1] == pos - 1u);
        flags[i] = leader ? 1u : 0u;
        if (!leader) continue;
        count++;
        const uint32_t rest = pos >> 1;
        E2 v0 = zero(), v1 = zero();
        if ((pos & 1u) == 0u) {
            v0 = ld(val, i);
            if (i + 1 < e && idx[i + 1] == pos + 1u) v1 = ld(val, i + 1);
        } else {
            v1 = ld(val, i);
        }
        const E2 e0 = ld(eq, 2 * (uint64_t)rest), e1 = ld(eq, 2 * (uint64_t)rest + 1);
        if (t != cur_t) {
            flush();
            cur_t = t;
        }
        const E2 one{1, 0};
        const E2 vd = agl::e2_sub(v1, v0), ed = agl::e2_sub(e1, e0);
        E2 a = v0, ec = e0;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            lazy_mul(S[c], agl::e2_mul_lazy(a, agl::e2_sub(a, one)), ec);
            a = agl::e2_add(a, vd);
            ec = agl::e2_add(ec, ed);
        }
    }
    flush();
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const E2 v = warp_sum(acc[k]);
        if ((tid & 31) == 0) {
            sh[tid >> 5][2 * k] = v.c0;
            sh[tid >> 5][2 * k + 1] = v.c1;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) count += __shfl_down_sync(0xffffffffu, count, o);
    if ((tid & 31) == 0) shc[tid >> 5] = count;
    __syncthreads();
    if (tid < 4) {
        E2 v = zero();
        for (int wp = 0; wp < THREADS / 32; wp++) v = agl::e2_add(v, E2{sh[wp][2 * tid], sh[wp][2 * tid + 1]});
        st(tile_part, (uint64_t)blockIdx.x * 4 + tid, v);
    }
    if (tid == 0) {
        uint32_t c = 0;
        for (int wp = 0; wp < THREADS / 32; wp++) c += shc[wp];
        tile_count[blockIdx.x] = c;
    }
}

// One block: tile_count becomes its exclusive prefix sum; result = [message (8 words), total].
__global__ void __launch_bounds__(1024) bool_scan_reduce_kernel(uint32_t* __restrict__ tile_count, const uint64_t* __restrict__ tile_part,
                                                                uint32_t n_tiles, uint64_t* __restrict__ result) {
    __shared__ uint32_t sc[1024];
    __shared__ uint64_t sh[32][8];
    const int tid = threadIdx.x;
    const uint32_t per = (n_tiles + 1023) / 1024;
    const uint32_t lo = min(n_tiles, tid * per), hi = min(n_tiles, lo + per);
    uint32_t sum = 0;
    E2 acc[4];
#pragma unroll
    for (int k = 0; k < 4; k++) acc[k] = zero();
    for (uint32_t b = lo; b < hi; b++) {
        sum += tile_count[b];
#pragma unroll
        for (int k = 0; k < 4; k++) acc[k] = agl::e2_add(acc[k], ld(tile_part, (uint64_t)b * 4 + k));
    }
    sc[tid] = sum;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {   // inclusive scan of the per-thread sums
        const uint32_t add = tid >= o ? sc[tid - o] : 0u;
        __syncthreads();
        sc[tid] += add;
        __syncthreads();
    }
    uint32_t run = sc[tid] - sum;
    for (uint32_t b = lo; b < hi; b++) {
        const uint32_t c = tile_count[b];
        tile_count[b] = run;
        run += c;
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const E2 v = warp_sum(acc[k]);
        if ((tid & 31) == 0) {
            sh[tid >> 5][2 * k] = v.c0;
            sh[tid >> 5][2 * k + 1] = v.c1;
        }
    }
    __syncthreads();
    if (tid < 4) {
        E2 v = zero();
        for (int wp = 0; wp < 32; wp++) v = agl::e2_add(v, E2{sh[wp][2 * tid], sh[wp][2 * tid + 1]});
        st(result, tid, v);
    }
    if (tid == 1023) result[8] = sc[1023];
}

// gid[i] = tile offset + exclusive prefix of the flags inside the tile; a thread owns eight consecutive entries.
__global__ void __launch_bounds__(THREADS) bool_gid_kernel(const uint32_t* __restrict__ flags, const uint32_t* __restrict__ tile_off,
                                                           uint32_t n, uint32_t* __restrict__ gid) {
    __shared__ uint32_t sw[THREADS / 32];
    const int tid = threadIdx.x;
    const uint32_t first = blockIdx.x * (uint32_t)TILE + tid * PER_THREAD;
    uint32_t f[PER_THREAD], sum = 0;
#pragma unroll
    for (int j = 0; j < PER_THREAD; j++) {
        f[j] = first + j < n ? flags[first + j] : 0u;
        sum += f[j];
    }
    uint32_t inc = sum;   // inclusive scan over the warp, then over the eight warps
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o);
        if ((tid & 31) >= o) inc += u;
    }
    if ((tid & 31) == 31) sw[tid >> 5] = inc;
    __syncthreads();
    uint32_t before = tile_off[blockIdx.x];
    for (int wp = 0; wp < (tid >> 5); wp++) before += sw[wp];
    uint32_t run = before + inc - sum;
#pragma unroll
    for (int j = 0; j < PER_THREAD; j++) {
        if (first + j < n) gid[first + j] = run;
        run += f[j];
    }
}

__global__ void bool_fold_kernel(const uint32_t* __restrict__ idx, const uint64_t* __restrict__ val, const uint32_t* __restrict__ flags,
                                 const uint32_t* __restrict__ gid, uint32_t n, E2 ch, uint32_t* __restrict__ out_idx,
                                 uint64_t* __restrict__ out_val) {
    const agl::E2Pre rp = agl::e2_pre(ch);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        if (!flags[i]) continue;
        const uint32_t pos = idx[i];
        E2 v0 = zero(), v1 = zero();
        if ((pos & 1u) == 0u) {
            v0 = ld(val, i);
            if (i + 1 < n && !flags[i + 1]) v1 = ld(val, i + 1);   // a cleared flag marks the odd partner of this entry
        } else {
            v1 = ld(val, i);
        }
        const uint32_t g = gid[i];
        out_idx[g] = pos >> 1;
        st(out_val, g, agl::e2_fma_pre(rp, agl::e2_sub(v1, v0), v0));
    }
}

__global__ void bool_newoff_kernel(const uint32_t* __restrict__ gid, const uint32_t* __restrict__ term_off, int n_terms, uint32_t n,
                                   uint32_t total, uint32_t* __restrict__ new_off) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > n_terms) return;
    const uint32_t s = term_off[t];
    new_off[t] = (t == n_terms || s >= n) ? total : gid[s];
}

__global__ void bool_finish_kernel(const uint32_t* __restrict__ idx, const uint64_t* __restrict__ val, const uint32_t* __restrict__ term_off,
                                   int n_terms, uint32_t n, uint64_t* __restrict__ out) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_terms) return;
    const uint32_t s = term_off[t], e = term_off[t + 1];
    E2 v = zero();
    if (s < e && s < n && idx[s] == 0u) v = ld(val, s);
    st(out, t, v);
}

__global__ void bool_init_val_kernel(uint64_t* __restrict__ val, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        agl::e2_store(val + 2 * i, E2{1, 0});
}

}  // namespace

extern "C" {

// Every selection entry starts at (1, 0).
int agl_bool_init_val_ffi(uint64_t* d_val, size_t n) {
    if (n == 0) return MB_OK;
    if (!d_val) return MB_ERR_ARG;
    MB_KERNEL("bool_init_val");
    bool_init_val_kernel<<<grid_for(n, 256, 8), 256, 0, MB_STREAM>>>(d_val, n);
    return finish_sync();
}

// One round: fills d_flags and d_gid (n entries each), h_msg = the 4 evaluations (8 canonical words),
// *h_total = number of groups. d_partial, grid_x and the scan scratch of the reference's interface are unused.
int agl_bool_round_msg_ffi(const uint32_t* d_idx, const uint64_t* d_val, const uint32_t* d_term_off, const uint64_t* d_w, const uint64_t* d_eq,
                           int n_terms, size_t n, uint32_t* d_flags, uint32_t* d_gid, uint64_t* d_partial, int grid_x,
                           uint32_t* d_scan_scratch, size_t scan_scratch_len, uint64_t* h_msg, uint32_t* h_total) {
    (void)d_partial; (void)grid_x; (void)d_scan_scratch; (void)scan_scratch_len;
    if (!h_msg || !h_total) return MB_ERR_ARG;
    if (n == 0) {
        for (int k = 0; k < 8; k++) h_msg[k] = 0;
        *h_total = 0;
        return MB_OK;
    }
    if (!d_idx || !d_val || !d_term_off || !d_w || !d_eq || !d_flags || !d_gid || n_terms < 1 || n > 0xffffefffULL) return MB_ERR_ARG;
    const uint32_t n_tiles = (uint32_t)((n + TILE - 1) / TILE);
    uint32_t* tile_count = nullptr;
    uint64_t *tile_part = nullptr, *result = nullptr;
    uint64_t* pin = pinned_scratch();
    if (!pin) return MB_ERR_CUDA;
    MB_CUDA(pool_alloc((void**)&tile_count, (size_t)n_tiles * 4));
    if (pool_alloc((void**)&tile_part, (size_t)n_tiles * 64) != cudaSuccess || pool_alloc((void**)&result, 9 * 8) != cudaSuccess) {
        pool_free(tile_count);
        pool_free(tile_part);
        return MB_ERR_CUDA;
    }
    {
        MB_KERNEL("bool_mark_msg");
        bool_mark_msg_kernel<<<n_tiles, THREADS, 0, MB_STREAM>>>(d_idx, d_val, d_term_off, d_w, d_eq, n_terms, (uint32_t)n, d_flags, tile_count,
                                                                tile_part);
    }
    {
        MB_KERNEL("bool_scan_reduce");
        bool_scan_reduce_kernel<<<1, 1024, 0, MB_STREAM>>>(tile_count, tile_part, n_tiles, result);
    }
    {
        MB_KERNEL("bool_gid");
        bool_gid_kernel<<<n_tiles, THREADS, 0, MB_STREAM>>>(d_flags, tile_count, (uint32_t)n, d_gid);
    }
    int rc = cudaMemcpyAsync(pin, result, 9 * 8, cudaMemcpyDeviceToHost, MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    if (rc == MB_OK) rc = finish_sync();
    pool_free(tile_count);
    pool_free(tile_part);
    pool_free(result);
    if (rc != MB_OK) return rc;
    for (int k = 0; k < 8; k++) h_msg[k] = pin[k];
    *h_total = (uint32_t)pin[8];
    return MB_OK;
}

// Fold by the challenge with the flags / gid / total of the preceding round message: `total` entries out and
// n_terms + 1 new offsets.
int agl_bool_fold_ffi(const uint32_t* d_idx, const uint64_t* d_val, const uint32_t* d_flags, const uint32_t* d_gid, const uint32_t* d_term_off,
                      int n_terms, size_t n, uint64_t r0, uint64_t r1, uint32_t total, int grid_x, uint32_t* d_out_idx, uint64_t* d_out_val,
                      uint32_t* d_new_off) {
    (void)grid_x;
    if (n == 0) return MB_OK;
    if (!d_idx || !d_val || !d_flags || !d_gid || !d_term_off || !d_out_idx || !d_out_val || !d_new_off || n_terms < 1 || n > 0xffffefffULL)
        return MB_ERR_ARG;
    {
        MB_KERNEL("bool_fold");
        bool_fold_kernel<<<grid_for(n, 256, 8), 256, 0, MB_STREAM>>>(d_idx, d_val, d_flags, d_gid, (uint32_t)n, E2{r0, r1}, d_out_idx, d_out_val);
    }
    {
        MB_KERNEL("bool_newoff");
        bool_newoff_kernel<<<(n_terms + 256) / 256, 256, 0, MB_STREAM>>>(d_gid, d_term_off, n_terms, (uint32_t)n, total, d_new_off);
    }
    return finish_sync();
}

// d_out[t] = the value of term t at position 0 (zero when the term has none).
int agl_bool_finish_ffi(const uint32_t* d_idx, const uint64_t* d_val, const uint32_t* d_term_off, int n_terms, size_t n, uint64_t* d_out) {
    if (n_terms <= 0) return MB_OK;
    if (!d_idx || !d_val || !d_term_off || !d_out) return MB_ERR_ARG;
    MB_KERNEL("bool_finish");
    bool_finish_kernel<<<(n_terms + 255) / 256, 256, 0, MB_STREAM>>>(d_idx, d_val, d_term_off, n_terms, (uint32_t)n, d_out);
    return finish_sync();
}

}  // extern "C"
