// C-ABI: exact module commitment over F_q[Y]/(Y^4096 + 1) with key caches in the
// transform domain (reference declarations almost-goldilocks-cuda-rs/src/ffi.rs:18-21,
// definitions almost-goldilocks-cuda-rs/cuda/wrapper.cu:3076-3229; Rust caller
// zk-torch-4/src/morpheus/commit_gpu.rs:27-97).
#include <cstring>
#include <mutex>

#include "agl_mcommit.cuh"
#include "common.cuh"
#include "prof.cuh"

using namespace mb;

namespace {

constexpr int MAX_DEV = 64;
constexpr int MAX_V = 8;

uint64_t powmod(uint64_t b, uint64_t e, uint64_t p) {
    uint64_t r = 1;
    b %= p;
    for (; e; e >>= 1) {
        if (e & 1) r = (unsigned __int128)r * b % p;
        b = (unsigned __int128)b * b % p;
    }
    return r;
}
uint32_t shoup(uint64_t w, uint64_t p) { return (uint32_t)((w << 32) / p); }

struct HostTables {
    mcm::Consts c;
    uint2 tw[mcm::MAXP][mcm::N], itw[mcm::MAXP][mcm::N];
};

// Everything derived from the primes and roots, computed once per process.
const HostTables* host_tables() {
    static HostTables* T = [] {
        HostTables* h = new HostTables();
        std::memset(h, 0, sizeof(HostTables));
        for (int i = 0; i < mcm::MAXP; i++) {
            const uint64_t p = mcm::PRIMES[i], psi = mcm::PSI[i], psi_inv = powmod(psi, p - 2, p);
            h->c.p[i] = (uint32_t)p;
            h->c.delta[i] = (uint32_t)((1ULL << 32) % p);
            const uint64_t ni = powmod(mcm::N, p - 2, p);
            h->c.ninv[i] = (uint32_t)ni;
            h->c.ninv_sh[i] = shoup(ni, p);
            for (int j = 0; j < mcm::N; j++) {
                int br = 0;
                for (int b = 0; b < 12; b++) br |= ((j >> b) & 1) << (11 - b);
                const uint64_t z = powmod(psi, br, p), zi = powmod(psi_inv, br, p);
                h->tw[i][j] = make_uint2((uint32_t)z, shoup(z, p));
                h->itw[i][j] = make_uint2((uint32_t)zi, shoup(zi, p));
            }
            for (int j = 0; j < i; j++) {
                const uint64_t g = powmod(mcm::PRIMES[j] % p, p - 2, p);
                h->c.ginv[i][j] = (uint32_t)g;
                h->c.ginv_sh[i][j] = shoup(g, p);
            }
        }
        for (int k = 1; k <= mcm::MAXP; k++) {
            // P_k - 1 has every mixed-radix digit at its maximum; halve it digit by digit from the top.
            uint64_t rem = 0;
            for (int i = k - 1; i >= 0; i--) {
                const uint64_t cur = rem * mcm::PRIMES[i] + (mcm::PRIMES[i] - 1);
                h->c.half[k - 1][i] = (uint32_t)(cur / 2);
                rem = cur & 1;
            }
            unsigned __int128 pm = 1;
            for (int i = 0; i < k; i++) pm = pm * mcm::PRIMES[i] % mcm::Q;
            h->c.pmodq[k - 1] = (uint64_t)pm;
        }
        return h;
    }();
    return T;
}

// Uploads the tables to the current device on first use there.
int ensure_tables() {
    static std::mutex mx;
    static bool ready[MAX_DEV] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return MB_ERR_CUDA;
    std::lock_guard<std::mutex> lk(mx);
    if (ready[dev]) return MB_OK;
    const HostTables* h = host_tables();
    MB_CUDA(cudaMemcpyToSymbolAsync(mcm::c_mc, &h->c, sizeof(mcm::Consts), 0, cudaMemcpyHostToDevice, MB_STREAM));
    MB_CUDA(cudaMemcpyToSymbolAsync(mcm::g_tw, h->tw, sizeof(h->tw), 0, cudaMemcpyHostToDevice, MB_STREAM));
    MB_CUDA(cudaMemcpyToSymbolAsync(mcm::g_itw, h->itw, sizeof(h->itw), 0, cudaMemcpyHostToDevice, MB_STREAM));
    MB_CUDA(cudaStreamSynchronize(MB_STREAM));
    ready[dev] = true;
    return MB_OK;
}

// CTAs of the streaming kernel that fit the device at once (its grid is sized to one full wave).
template <int V, int R>
int mac_slots(int rows) {
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, mcm::mac_kernel<V, R>, 128 * ((rows + R - 1) / R), 0) != cudaSuccess || occ < 1)
        occ = 1;
    return occ * sm_count();
}
template <int V, int R>
void launch_mac(const uint32_t* key, int kcols, int rows, const uint32_t* xh, const uint32_t* colidx, int C, int k, int chunk_cols,
                int chunks, uint32_t* part) {
    dim3 grid((unsigned)(k * mcm::N / 128), (unsigned)chunks), block(128, (unsigned)((rows + R - 1) / R));
    mcm::mac_kernel<V, R><<<grid, block, 0, MB_STREAM>>>(key, kcols, rows, xh, colidx, C, k, chunk_cols, part);
}
// Rows per thread for V vectors per pass: V * R accumulators stay in registers.
#define MCM_DISPATCH_V(V, CALL)              \
    switch (V) {                             \
        case 1: { CALL(1, 16); break; }      \
        case 2: { CALL(2, 16); break; }      \
        case 3: { CALL(3, 8); break; }       \
        case 4: { CALL(4, 8); break; }       \
        case 5: { CALL(5, 4); break; }       \
        case 6: { CALL(6, 4); break; }       \
        case 7: { CALL(7, 4); break; }       \
        default: { CALL(8, 4); break; }      \
    }

}  // namespace

extern "C" {

// d_key[k][ncols][rows][4096] (u32): transform-domain cache of key elements (kind, row, col0 + c).
int agl_mcommit_keygen(const uint32_t* h_seed, uint32_t kind, int rows, uint64_t col0, int ncols, int k, uint32_t* d_key) {
    if (!h_seed || rows < 1 || rows > mcm::MAXROWS || k < 1 || k > mcm::MAXP || ncols < 0 || (ncols && !d_key)) return MB_ERR_ARG;
    if ((size_t)ncols * rows > 0x7fffffffULL) return MB_ERR_ARG;
    if (ncols == 0) return MB_OK;
    int rc = ensure_tables();
    if (rc != MB_OK) return rc;
    uint32_t* d_seed = nullptr;
    MB_CUDA(pool_alloc((void**)&d_seed, 32));
    rc = cudaMemcpyAsync(d_seed, h_seed, 32, cudaMemcpyHostToDevice, MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    if (rc == MB_OK) rc = cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;   // h_seed is the caller's
    if (rc == MB_OK) {
        MB_KERNEL("mcommit_keygen_ntt");
        mcm::keygen_ntt_kernel<<<(unsigned)(ncols * rows), mcm::NT, 0, MB_STREAM>>>(d_seed, kind, rows, col0, ncols, k, d_key);
        rc = finish_sync();
    }
    pool_free(d_seed);
    return rc;
}

// d_acc[V][k][rows][4096] = sum over the C input columns of key[.][colidx[c]][row] * transform(x[v][c]).
// x_bytes 1 (int8) or 8 (int64); vector v starts at element v * x_vstride (0: packed, C * 4096);
// d_colidx may be null (identity); the key cache has kcols columns and `rows` rows.
int agl_mcommit_partial(const uint32_t* d_key, int kcols, int rows, int k, const void* d_x, int x_bytes, int V, int C,
                        uint64_t x_vstride, const uint32_t* d_colidx, uint32_t* d_acc) {
    if (rows < 1 || rows > mcm::MAXROWS || k < 1 || k > mcm::MAXP || V < 1 || V > MAX_V || C < 0 || !d_acc || (x_bytes != 1 && x_bytes != 8))
        return MB_ERR_ARG;
    const size_t stride = (size_t)V * k * rows * mcm::N;
    if (C == 0) {
        MB_CUDA(cudaMemsetAsync(d_acc, 0, stride * 4, MB_STREAM));
        return finish_sync();
    }
    if (!d_key || !d_x || kcols < 1 || (size_t)V * C > 0x7fffffffULL) return MB_ERR_ARG;
    int rc = ensure_tables();
    if (rc != MB_OK) return rc;
    // Column chunks: one full wave of CTAs (a second, partial wave would run at a fraction of the
    // bandwidth), chunk lengths a multiple of the three columns between folds.
    const int xblocks = k * mcm::N / 128;
    int slots = 0;
#define MCM_SLOTS(VV, RR) slots = mac_slots<VV, RR>(rows)
    MCM_DISPATCH_V(V, MCM_SLOTS)
#undef MCM_SLOTS
    int chunks = slots / xblocks;
    if (chunks > (C + 2) / 3) chunks = (C + 2) / 3;
    if (chunks < 1) chunks = 1;
    int chunk_cols = (C + chunks - 1) / chunks;
    chunk_cols = (chunk_cols + 2) / 3 * 3;
    chunks = (C + chunk_cols - 1) / chunk_cols;
    uint32_t *xh = nullptr, *part = nullptr;
    MB_CUDA(pool_alloc((void**)&xh, (size_t)V * k * C * mcm::N * 4));
    if (chunks > 1 && pool_alloc((void**)&part, (size_t)chunks * stride * 4) != cudaSuccess) {
        pool_free(xh);
        return MB_ERR_CUDA;
    }
    const size_t vs = x_vstride ? (size_t)x_vstride : (size_t)C * mcm::N;
    {
        MB_KERNEL("mcommit_input_ntt");
        if (x_bytes == 1) mcm::input_ntt_kernel<int8_t><<<(unsigned)(V * C), mcm::NT, 0, MB_STREAM>>>((const int8_t*)d_x, vs, C, k, xh);
        else mcm::input_ntt_kernel<int64_t><<<(unsigned)(V * C), mcm::NT, 0, MB_STREAM>>>((const int64_t*)d_x, vs, C, k, xh);
    }
    uint32_t* dst = chunks > 1 ? part : d_acc;
    {
        MB_KERNEL("mcommit_mac");
#define MCM_LAUNCH(VV, RR) launch_mac<VV, RR>(d_key, kcols, rows, xh, d_colidx, C, k, chunk_cols, chunks, dst)
        MCM_DISPATCH_V(V, MCM_LAUNCH)
#undef MCM_LAUNCH
    }
    if (chunks > 1) {
        MB_KERNEL("mcommit_sum_parts");
        mcm::sum_parts_kernel<<<grid_for(stride, 256, 8), 256, 0, MB_STREAM>>>(part, chunks, stride, k, rows, d_acc);
    }
    rc = finish_sync();
    pool_free(xh);
    if (part) pool_free(part);
    return rc;
}

// d_dst += d_src (accumulators of the same shape), mod p per prime.
int agl_mcommit_add(uint32_t* d_dst, const uint32_t* d_src, int V, int k, int rows) {
    if (!d_dst || !d_src || V < 1 || k < 1 || k > mcm::MAXP || rows < 1 || rows > mcm::MAXROWS) return MB_ERR_ARG;
    int rc = ensure_tables();
    if (rc != MB_OK) return rc;
    const size_t n = (size_t)V * k * rows * mcm::N;
    MB_KERNEL("mcommit_add");
    mcm::add_kernel<<<grid_for(n, 256, 8), 256, 0, MB_STREAM>>>(d_dst, d_src, n, k, rows);
    return finish_sync();
}

// d_out[V][rows][4096] = CRT(inverse transform(d_acc)) mod q (+ d_err[V][rows][4096], may be null), canonical.
// d_acc is left unchanged (the reference transforms it in place).
int agl_mcommit_finish(uint32_t* d_acc, int V, int k, int rows, const int64_t* d_err, uint64_t* d_out) {
    if (!d_acc || !d_out || V < 1 || k < 1 || k > mcm::MAXP || rows < 1 || rows > mcm::MAXROWS) return MB_ERR_ARG;
    int rc = ensure_tables();
    if (rc != MB_OK) return rc;
    MB_KERNEL("mcommit_finish");
    mcm::finish_kernel<<<(unsigned)(V * rows), mcm::NT, 0, MB_STREAM>>>(d_acc, k, rows, d_err, d_out);
    return finish_sync();
}

}  // extern "C"
