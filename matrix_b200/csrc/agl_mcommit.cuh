// Module commitment over R = F_q[Y]/(Y^4096 + 1), q = 2^64 - 2^32 - 31, computed
// exactly (reference kernels cuda_almost_goldilocks/morpheus_commit.cuh:61-334,
// CPU definition zk-torch-4/src/morpheus/ring.rs and commit.rs:48-83):
//
//     C[v][row] = sum_c key[row][col(c)] * x[v][c]      (+ identity error)
//
// where the key elements are the centred representatives of SHAKE256-expanded
// residues (zk-torch-4/src/morpheus/keys.rs:48-83) and the products are integer
// negacyclic convolutions: formed modulo the first k of five 31-bit primes
// p = 1 mod 8192 by a length-4096 negacyclic transform, accumulated pointwise,
// transformed back, recombined by Garner's mixed-radix CRT to the centred
// integer and only then reduced mod q.
//
// Layouts (u32 residues; the order inside a transformed vector is this file's
// own, callers only pass the buffers between the entry points):
//     key cache   key[prime][column][row][4096]
//     accumulator acc[vector][prime][row][4096]
//
// Kernels
//   keygen_ntt   one CTA per key element: 512 threads expand one SHAKE block of
//                8 coefficients each, then per prime residues -> transform -> store
//                (the element never leaves the chip between expansion and cache).
//   input_ntt    one CTA per (vector, column): the column is read once, all k
//                transforms are formed from registers.
//   mac          streaming pointwise multiply-accumulate, HBM bound on the key
//                cache (16 KB per prime, column and row); lazy 64-bit sums folded
//                with 2^32 = delta (mod p), delta < 2^20.
//   finish       one CTA per (vector, row): k inverse transforms kept in
//                registers, Garner digits, Horner mod q, centring, error.
//
// Transform: 512 threads x 8 values, four radix-8 passes in registers (three
// butterfly layers each) with one padded shared-memory exchange between passes:
// three barriers per transform instead of twelve. Twiddles carry their Shoup
// companions floor(w 2^32 / p), so a modular product is mulhi, two mullo, min.
#pragma once
#include <cstdint>

#include "agl_field.cuh"

namespace mcm {

constexpr int N = 4096;
constexpr int MAXP = 5;
constexpr int MAXROWS = 16;
constexpr int NT = 512;                   // threads per transform, 8 values each
constexpr int SPAD = N + (N >> 6) * 8;    // padded exchange buffer (words)
constexpr uint64_t Q = 0xFFFFFFFEFFFFFFE1ULL;

// p_i and a primitive 8192-th root psi_i (psi^4096 = -1), zk-torch-4/src/morpheus/ring.rs:26-32.
constexpr uint32_t PRIMES[MAXP] = {2147377153u, 2147352577u, 2147295233u, 2147205121u, 2147196929u};
constexpr uint32_t PSI[MAXP] = {1202012506u, 760495213u, 920713129u, 2061834542u, 1321772815u};

struct Consts {
    uint32_t p[MAXP];
    uint32_t delta[MAXP];                  // 2^32 mod p
    uint32_t ninv[MAXP], ninv_sh[MAXP];    // 4096^{-1} mod p and its Shoup companion
    uint32_t ginv[MAXP][MAXP];             // ginv[i][j] = p_j^{-1} mod p_i, j < i
    uint32_t ginv_sh[MAXP][MAXP];
    uint32_t half[MAXP][MAXP];             // half[k-1][i]: mixed-radix digits of floor(P_k / 2)
    uint64_t pmodq[MAXP];                  // P_k mod q
};

#ifdef __CUDACC__
__constant__ Consts c_mc;
__device__ uint2 g_tw[MAXP][N];    // (psi^bitrev(i), Shoup companion)
__device__ uint2 g_itw[MAXP][N];   // the same for psi^{-1}

// ------------------------------------------------------------------ arithmetic mod p (p < 2^31)
__device__ __forceinline__ uint32_t mul_shoup(uint32_t a, uint32_t w, uint32_t wsh, uint32_t p) {
    const uint32_t q = __umulhi(a, wsh);
    const uint32_t r = a * w - q * p;   // in [0, 2p)
    return min(r, r - p);
}
__device__ __forceinline__ uint32_t addp(uint32_t a, uint32_t b, uint32_t p) {
    const uint32_t s = a + b;
    return min(s, s - p);
}
__device__ __forceinline__ uint32_t subp(uint32_t a, uint32_t b, uint32_t p) {
    const uint32_t d = a - b;
    return min(d, d + p);
}
// x -> lo + hi * delta, congruent mod p; delta < 2^20 maps [0, 2^64) into [0, 2^32 + 2^52).
__device__ __forceinline__ uint64_t foldp(uint64_t x, uint32_t delta) {
    return (uint64_t)(uint32_t)x + (uint64_t)(uint32_t)(x >> 32) * delta;
}
__device__ __forceinline__ uint32_t reduce_u64(uint64_t x, uint32_t p, uint32_t delta) {
    x = foldp(foldp(foldp(x, delta), delta), delta);   // < 2^32 + 2^29 < 3p
    if (x >= p) x -= p;
    if (x >= p) x -= p;
    return (uint32_t)x;
}
__device__ __forceinline__ uint32_t residue_i64(int64_t x, uint32_t p, uint32_t delta) {
    const bool neg = x < 0;
    const uint64_t m = neg ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
    const uint32_t r = reduce_u64(m, p, delta);
    return (neg && r) ? p - r : r;
}

__device__ __forceinline__ int spad(int i) { return i + ((i >> 6) << 3); }

// Cooley-Tukey layer on a pair: (a, b) -> (a + w b, a - w b).
__device__ __forceinline__ void ct(uint32_t& a, uint32_t& b, uint2 w, uint32_t p) {
    const uint32_t t = mul_shoup(b, w.x, w.y, p);
    b = subp(a, t, p);
    a = addp(a, t, p);
}
// Gentleman-Sande layer on a pair: (a, b) -> (a + b, (a - b) w).
__device__ __forceinline__ void gs(uint32_t& a, uint32_t& b, uint2 w, uint32_t p) {
    const uint32_t d = subp(a, b, p);
    a = addp(a, b, p);
    b = mul_shoup(d, w.x, w.y, p);
}

// Three forward layers on eight values spaced by one stride; `G` is the index of
// the group of 8 strides among the groups of layer `s0`.
__device__ __forceinline__ void radix8_fwd(uint32_t x[8], const uint2* tw, int s0, int G, uint32_t p) {
    const uint2 wa = tw[(1 << s0) + G];
#pragma unroll
    for (int i = 0; i < 4; i++) ct(x[i], x[i + 4], wa, p);
    const uint2 wb0 = tw[(2 << s0) + 2 * G], wb1 = tw[(2 << s0) + 2 * G + 1];
    ct(x[0], x[2], wb0, p);
    ct(x[1], x[3], wb0, p);
    ct(x[4], x[6], wb1, p);
    ct(x[5], x[7], wb1, p);
#pragma unroll
    for (int i = 0; i < 4; i++) ct(x[2 * i], x[2 * i + 1], tw[(4 << s0) + 4 * G + i], p);
}
__device__ __forceinline__ void radix8_inv(uint32_t x[8], const uint2* tw, int s0, int G, uint32_t p) {
#pragma unroll
    for (int i = 0; i < 4; i++) gs(x[2 * i], x[2 * i + 1], tw[(4 << s0) + 4 * G + i], p);
    const uint2 wb0 = tw[(2 << s0) + 2 * G], wb1 = tw[(2 << s0) + 2 * G + 1];
    gs(x[0], x[2], wb0, p);
    gs(x[1], x[3], wb0, p);
    gs(x[4], x[6], wb1, p);
    gs(x[5], x[7], wb1, p);
    const uint2 wa = tw[(1 << s0) + G];
#pragma unroll
    for (int i = 0; i < 4; i++) gs(x[i], x[i + 4], wa, p);
}

// Forward transform. In: x[i] = a[t + 512 i], residues in [0, p). Out: x[i] = value at
// position 8 t + i of the transformed vector. `s` is SPAD words of shared memory;
// ends without a barrier after its last shared-memory read.
__device__ __forceinline__ void ntt_forward(uint32_t x[8], uint32_t* s, const uint2* tw, uint32_t p, int t) {
    radix8_fwd(x, tw, 0, 0, p);
#pragma unroll
    for (int i = 0; i < 8; i++) s[spad(t + 512 * i)] = x[i];
    __syncthreads();
    {
        const int base = (t >> 6) * 512 + (t & 63);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = s[spad(base + 64 * i)];
        radix8_fwd(x, tw, 3, t >> 6, p);
#pragma unroll
        for (int i = 0; i < 8; i++) s[spad(base + 64 * i)] = x[i];
    }
    __syncthreads();
    {
        const int base = (t >> 3) * 64 + (t & 7);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = s[spad(base + 8 * i)];
        radix8_fwd(x, tw, 6, t >> 3, p);
#pragma unroll
        for (int i = 0; i < 8; i++) s[spad(base + 8 * i)] = x[i];
    }
    __syncthreads();
    {
        const uint4* v = reinterpret_cast<const uint4*>(s + spad(8 * t));
        const uint4 lo = v[0], hi = v[1];
        x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
        x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
        radix8_fwd(x, tw, 9, t, p);
    }
}

// Inverse transform including the factor 4096^{-1}. In: x[i] = value at position
// 8 t + i. Out: x[i] = a[t + 512 i]. Starts with shared-memory writes: the caller
// puts a barrier between an earlier use of `s` and this call.
__device__ __forceinline__ void ntt_inverse(uint32_t x[8], uint32_t* s, const uint2* tw, uint32_t p, uint32_t ninv,
                                            uint32_t ninv_sh, int t) {
    radix8_inv(x, tw, 9, t, p);
    {
        uint4* v = reinterpret_cast<uint4*>(s + spad(8 * t));
        v[0] = make_uint4(x[0], x[1], x[2], x[3]);
        v[1] = make_uint4(x[4], x[5], x[6], x[7]);
    }
    __syncthreads();
    {
        const int base = (t >> 3) * 64 + (t & 7);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = s[spad(base + 8 * i)];
        radix8_inv(x, tw, 6, t >> 3, p);
#pragma unroll
        for (int i = 0; i < 8; i++) s[spad(base + 8 * i)] = x[i];
    }
    __syncthreads();
    {
        const int base = (t >> 6) * 512 + (t & 63);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = s[spad(base + 64 * i)];
        radix8_inv(x, tw, 3, t >> 6, p);
#pragma unroll
        for (int i = 0; i < 8; i++) s[spad(base + 64 * i)] = x[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = s[spad(t + 512 * i)];
    radix8_inv(x, tw, 0, 0, p);
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = mul_shoup(x[i], ninv, ninv_sh, p);
}

__device__ __forceinline__ void store8(uint32_t* g, int t, const uint32_t x[8]) {
    uint4* v = reinterpret_cast<uint4*>(g + 8 * t);
    v[0] = make_uint4(x[0], x[1], x[2], x[3]);
    v[1] = make_uint4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void load8(const uint32_t* g, int t, uint32_t x[8]) {
    const uint4* v = reinterpret_cast<const uint4*>(g + 8 * t);
    const uint4 lo = v[0], hi = v[1];
    x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
    x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
}
#endif  // __CUDACC__

// ------------------------------------------------------------------ SHAKE256 key blocks
// Keccak-f[1600] (FIPS 202), host and device.
#ifdef __CUDACC__
#define MCM_HD __host__ __device__ __forceinline__
#else
#define MCM_HD inline
#endif

MCM_HD uint64_t rotl64(uint64_t x, int s) { return s ? (x << s) | (x >> (64 - s)) : x; }

#define MCM_KECCAK_RC                                                                                                   \
    {0x0000000000000001ULL, 0x0000000000008082ULL, 0x800000000000808aULL, 0x8000000080008000ULL, 0x000000000000808bULL, \
     0x0000000080000001ULL, 0x8000000080008081ULL, 0x8000000000008009ULL, 0x000000000000008aULL, 0x0000000000000088ULL, \
     0x0000000080008009ULL, 0x000000008000000aULL, 0x000000008000808bULL, 0x800000000000008bULL, 0x8000000000008089ULL, \
     0x8000000000008003ULL, 0x8000000000008002ULL, 0x8000000000000080ULL, 0x000000000000800aULL, 0x800000008000000aULL, \
     0x8000000080008081ULL, 0x8000000000008080ULL, 0x0000000080000001ULL, 0x8000000080008008ULL}
#ifdef __CUDACC__
static __constant__ uint64_t c_keccak_rc[24] = MCM_KECCAK_RC;
#endif
static const uint64_t h_keccak_rc[24] = MCM_KECCAK_RC;

MCM_HD void keccak_f1600(uint64_t a[25]) {
    // rotation offsets r[x + 5 y]
    constexpr int RHO[25] = {0, 1, 62, 28, 27, 36, 44, 6, 55, 20, 3, 10, 43, 25, 39, 41, 45, 15, 21, 8, 18, 2, 61, 56, 14};
#ifdef __CUDA_ARCH__
#pragma unroll 1
#endif
    for (int r = 0; r < 24; r++) {
        uint64_t c[5], b[25];
#pragma unroll
        for (int x = 0; x < 5; x++) c[x] = a[x] ^ a[x + 5] ^ a[x + 10] ^ a[x + 15] ^ a[x + 20];
#pragma unroll
        for (int x = 0; x < 5; x++) {
            const uint64_t d = c[(x + 4) % 5] ^ rotl64(c[(x + 1) % 5], 1);
#pragma unroll
            for (int y = 0; y < 5; y++) a[x + 5 * y] ^= d;
        }
        // rho and pi: lane (x, y) moves to (y, 2x + 3y)
#pragma unroll
        for (int y = 0; y < 5; y++)
#pragma unroll
            for (int x = 0; x < 5; x++) b[y + 5 * ((2 * x + 3 * y) % 5)] = rotl64(a[x + 5 * y], RHO[x + 5 * y]);
#pragma unroll
        for (int y = 0; y < 5; y++)
#pragma unroll
            for (int x = 0; x < 5; x++) a[x + 5 * y] = b[x + 5 * y] ^ (~b[(x + 1) % 5 + 5 * y] & b[(x + 2) % 5 + 5 * y]);
#ifdef __CUDA_ARCH__
        a[0] ^= c_keccak_rc[r];
#else
        a[0] ^= h_keccak_rc[r];
#endif
    }
}

// First 64 bytes of SHAKE256("MORPHEUS/KEY/SHAKE256/v2\0" || seed[8] || counter || nonce[3]),
// words little-endian (zk-torch-4/src/morpheus/keys.rs:48-59): a 73-byte message, one block.
MCM_HD void shake_key_block(const uint32_t seed[8], uint32_t counter, const uint32_t nonce[3], uint32_t out[16]) {
    // The 25-byte tag as little-endian 64-bit lanes; byte 24 (the terminator) is zero.
    uint64_t st[25];
#pragma unroll
    for (int i = 0; i < 25; i++) st[i] = 0;
    st[0] = 0x5355454850524f4dULL;   // "MORPHEUS"
    st[1] = 0x4148532f59454b2fULL;   // "/KEY/SHA"
    st[2] = 0x32762f363532454bULL;   // "KE256/v2"
    // words follow from byte 25: word w sits at bytes 25 + 4w .. 28 + 4w
    uint32_t w[12];
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = seed[i];
    w[8] = counter;
    w[9] = nonce[0];
    w[10] = nonce[1];
    w[11] = nonce[2];
#pragma unroll
    for (int i = 0; i < 12; i++) {
        const int off = 25 + 4 * i;            // byte offset, off % 8 in {1, 5}
        const int lane = off / 8, sh = 8 * (off % 8);
        st[lane] ^= (uint64_t)w[i] << sh;
        if (sh > 32) st[lane + 1] ^= (uint64_t)w[i] >> (64 - sh);
    }
    st[73 / 8] ^= 0x1fULL << (8 * (73 % 8));   // SHAKE suffix after 73 message bytes
    st[16] ^= 0x8000000000000000ULL;           // last byte of the 136-byte rate
    keccak_f1600(st);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        out[2 * i] = (uint32_t)st[i];
        out[2 * i + 1] = (uint32_t)(st[i] >> 32);
    }
}

// Eight canonical coefficients of block b of key element (kind, row, col): 64-bit words
// below q are accepted in order, up to 16 blocks (counters b + 512 retry), zero fill
// (zk-torch-4/src/morpheus/keys.rs:62-83).
MCM_HD void key_block8(const uint32_t seed[8], uint32_t kind, uint32_t row, uint64_t col, uint32_t b, uint64_t vals[8]) {
    const uint32_t nonce[3] = {(kind << 16) | row, (uint32_t)col, (uint32_t)(col >> 32)};
    int written = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) vals[i] = 0;
    for (uint32_t retry = 0; retry < 16 && written < 8; retry++) {
        uint32_t w[16];
        shake_key_block(seed, b + 512u * retry, nonce, w);
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const uint64_t v = (uint64_t)w[2 * t] | ((uint64_t)w[2 * t + 1] << 32);
            if (v < Q && written < 8) {
                // written is uniform over t only when nothing was rejected; select by compare to stay in registers
#pragma unroll
                for (int s = 0; s < 8; s++)
                    if (s == written) vals[s] = v;
                written++;
            }
        }
    }
}

#ifdef __CUDACC__
// ------------------------------------------------------------------ kernels
// Key cache for columns [col0, col0 + ncols): grid = ncols * rows CTAs of 512 threads.
__global__ void __launch_bounds__(NT) keygen_ntt_kernel(const uint32_t* __restrict__ seed, uint32_t kind, int rows, uint64_t col0,
                                                        int ncols, int k, uint32_t* __restrict__ key) {
    __shared__ __align__(16) uint32_t s[SPAD];
    const int t = threadIdx.x;
    const int row = blockIdx.x % rows, c = blockIdx.x / rows;
    uint32_t sd[8];
#pragma unroll
    for (int i = 0; i < 8; i++) sd[i] = seed[i];
    uint64_t vals[8];
    key_block8(sd, kind, (uint32_t)row, col0 + (uint64_t)c, (uint32_t)t, vals);
    int64_t cen[8];
#pragma unroll
    for (int i = 0; i < 8; i++) cen[i] = vals[i] > (Q - 1) / 2 ? -(int64_t)(Q - vals[i]) : (int64_t)vals[i];
    for (int pi = 0; pi < k; pi++) {
        const uint32_t p = c_mc.p[pi], delta = c_mc.delta[pi];
        uint32_t x[8];
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = residue_i64(cen[i], p, delta);
        // thread t made coefficients 8t .. 8t+7; the transform wants t + 512 i
        __syncthreads();
        {
            uint4* v = reinterpret_cast<uint4*>(s + spad(8 * t));
            v[0] = make_uint4(x[0], x[1], x[2], x[3]);
            v[1] = make_uint4(x[4], x[5], x[6], x[7]);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = s[spad(t + 512 * i)];   // the words this thread rewrites first
        ntt_forward(x, s, g_tw[pi], p, t);
        store8(key + (((size_t)pi * ncols + c) * rows + row) * N, t, x);
    }
}

// xh[v][prime][c][4096] = transform of column c of vector v (int8 or int64 coefficients).
template <typename TX>
__global__ void __launch_bounds__(NT, sizeof(TX) == 1 ? 3 : 2) input_ntt_kernel(const TX* __restrict__ x, size_t vstride, int C, int k, uint32_t* __restrict__ xh) {
    __shared__ __align__(16) uint32_t s[SPAD];
    const int t = threadIdx.x;
    const int c = blockIdx.x % C, v = blockIdx.x / C;
    const TX* col = x + (size_t)v * vstride + (size_t)c * N;
    int64_t in[8];
#pragma unroll
    for (int i = 0; i < 8; i++) in[i] = (int64_t)col[t + 512 * i];
    for (int pi = 0; pi < k; pi++) {
        const uint32_t p = c_mc.p[pi], delta = c_mc.delta[pi];
        uint32_t r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (sizeof(TX) == 1) r[i] = in[i] < 0 ? p - (uint32_t)(-in[i]) : (uint32_t)in[i];
            else r[i] = residue_i64(in[i], p, delta);
        }
        if (pi) __syncthreads();
        ntt_forward(r, s, g_tw[pi], p, t);
        store8(xh + (((size_t)v * k + pi) * C + c) * N, t, r);
    }
}

// part[chunk][v][prime][row][j] = sum over the chunk's columns of key[prime][col(c)][row][j] * xh[v][prime][c][j].
// Thread = (prime, j, group of R rows); block (128, rows / R); grid (k * 4096 / 128, chunks).
template <int V, int R>
__global__ void __launch_bounds__(128 * (MAXROWS / R), V == 1 ? 6 : V == 2 ? 5 : V <= 4 ? 2 : 1) mac_kernel(const uint32_t* __restrict__ key, int kcols, int rows,
                                                                  const uint32_t* __restrict__ xh, const uint32_t* __restrict__ colidx,
                                                                  int C, int k, int chunk_cols, uint32_t* __restrict__ part) {
    const int j = blockIdx.x * 128 + threadIdx.x;
    const int pi = j / N, jj = j % N;
    const int r0 = threadIdx.y * R;
    const uint32_t p = c_mc.p[pi], delta = c_mc.delta[pi];
    const int c0 = blockIdx.y * chunk_cols, c1 = min(C, c0 + chunk_cols);
    uint64_t acc[V][R];
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int r = 0; r < R; r++) acc[v][r] = 0;
    // The loads of column c + 1 are issued before the products of column c, so every warp keeps
    // R + V loads in flight; three columns between folds: 2^53 + 3 * 2^62 < 2^64.
    uint32_t an[R], xn[V];
    auto fetch = [&](int c) {
        const int kc = colidx ? (int)colidx[c] : c;
        const uint32_t* kp = key + (((size_t)pi * kcols + kc) * rows + r0) * N + jj;
#pragma unroll
        for (int r = 0; r < R; r++) an[r] = (r0 + r < rows) ? __ldcs(kp + (size_t)r * N) : 0u;
#pragma unroll
        for (int v = 0; v < V; v++) xn[v] = __ldg(xh + (((size_t)v * k + pi) * C + c) * N + jj);
    };
    if (c0 < c1) fetch(c0);
    for (int cb = c0; cb < c1; cb += 3) {
#pragma unroll
        for (int u = 0; u < 3; u++) {
            const int c = cb + u;
            if (c < c1) {
                uint32_t a[R], xv[V];
#pragma unroll
                for (int r = 0; r < R; r++) a[r] = an[r];
#pragma unroll
                for (int v = 0; v < V; v++) xv[v] = xn[v];
                if (c + 1 < c1) fetch(c + 1);
#pragma unroll
                for (int v = 0; v < V; v++)
#pragma unroll
                    for (int r = 0; r < R; r++) acc[v][r] += (uint64_t)a[r] * xv[v];
            }
        }
#pragma unroll
        for (int v = 0; v < V; v++)
#pragma unroll
            for (int r = 0; r < R; r++) acc[v][r] = foldp(acc[v][r], delta);
    }
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int r = 0; r < R; r++)
            if (r0 + r < rows)
                part[((((size_t)blockIdx.y * V + v) * k + pi) * rows + r0 + r) * N + jj] = reduce_u64(acc[v][r], p, delta);
}

// acc[id] = sum over `parts` blocks of part[b * stride + id] mod p; id over [v][prime][row][4096].
__global__ void sum_parts_kernel(const uint32_t* __restrict__ part, int parts, size_t stride, int k, int rows, uint32_t* __restrict__ acc) {
    for (size_t id = blockIdx.x * (size_t)blockDim.x + threadIdx.x; id < stride; id += (size_t)gridDim.x * blockDim.x) {
        const int pi = (int)((id / ((size_t)rows * N)) % k);
        uint64_t s = 0;
        for (int b = 0; b < parts; b++) s += part[(size_t)b * stride + id];   // parts < 2^32
        acc[id] = reduce_u64(s, c_mc.p[pi], c_mc.delta[pi]);
    }
}

__global__ void add_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, size_t n, int k, int rows) {
    for (size_t id = blockIdx.x * (size_t)blockDim.x + threadIdx.x; id < n; id += (size_t)gridDim.x * blockDim.x) {
        const int pi = (int)((id / ((size_t)rows * N)) % k);
        dst[id] = addp(dst[id], src[id], c_mc.p[pi]);
    }
}

// out[v][row][4096] = centred CRT of the inverse transforms of acc[v][*][row], mod q, plus err.
// grid = V * rows CTAs of 512 threads.
__global__ void __launch_bounds__(NT) finish_kernel(const uint32_t* __restrict__ acc, int k, int rows, const int64_t* __restrict__ err,
                                                    uint64_t* __restrict__ out) {
    __shared__ __align__(16) uint32_t s[SPAD];
    const int t = threadIdx.x;
    const int row = blockIdx.x % rows, v = blockIdx.x / rows;
    uint32_t d[MAXP][8];
#pragma unroll
    for (int pi = 0; pi < MAXP; pi++) {
        if (pi < k) {
            const uint32_t p = c_mc.p[pi];
            uint32_t x[8];
            load8(acc + (((size_t)v * k + pi) * rows + row) * N, t, x);
            if (pi) __syncthreads();
            ntt_inverse(x, s, g_itw[pi], p, c_mc.ninv[pi], c_mc.ninv_sh[pi], t);
#pragma unroll
            for (int i = 0; i < 8; i++) d[pi][i] = x[i];
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        // Garner: d[a] becomes the mixed-radix digit a
#pragma unroll
        for (int a = 1; a < MAXP; a++) {
            if (a < k) {
                const uint32_t p = c_mc.p[a];
                uint32_t x = d[a][i];
#pragma unroll
                for (int b = 0; b < a; b++) {
                    const uint32_t db = min(d[b][i], d[b][i] - p);   // digit b < p_b < 2 p_a
                    x = mul_shoup(subp(x, db, p), c_mc.ginv[a][b], c_mc.ginv_sh[a][b], p);
                }
                d[a][i] = x;
            }
        }
        uint64_t x = 0;
        bool greater = false, decided = false;
#pragma unroll
        for (int a = MAXP - 1; a >= 0; a--) {
            if (a < k) {
                x = agl::add(agl::mul(x, (uint64_t)c_mc.p[a]), (uint64_t)d[a][i]);
                const uint32_t h = c_mc.half[k - 1][a];
                if (!decided && d[a][i] != h) {
                    decided = true;
                    greater = d[a][i] > h;
                }
            }
        }
        if (greater) x = agl::sub(x, c_mc.pmodq[k - 1]);
        const size_t o = ((size_t)v * rows + row) * N + t + 512 * i;
        if (err) {
            const int64_t e = err[o];
            x = e >= 0 ? agl::add(x, (uint64_t)e) : agl::sub(x, (uint64_t)0 - (uint64_t)e);
        }
        out[o] = agl::canon(x);
    }
}
#endif  // __CUDACC__

}  // namespace mcm
