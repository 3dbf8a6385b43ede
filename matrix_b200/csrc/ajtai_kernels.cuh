// Ajtai ring commitment over almost-Goldilocks: c_i = sum_j M[i][j] * z_j in
// R = F_q[X]/(X^64 + 1), i < KAPPA = 42 (reference: cuda_almost_goldilocks/ajtai.cuh:29-30,
// 94-161, 215-275; matrix generator ajtai_chacha8.cuh:60-178; CPU twin
// ajtai_cpu_reference.cuh:165-186).
//
// M[i][j] is never stored: its 64 coefficients are 8 ChaCha8 blocks keyed by
// (row i, column j), rejection-sampled below q. This file holds the generator
// and the scalar commit path (exact integer accumulation per column, one
// modular reduction per output and column). The tensor-core path for small
// signed digits lives in ajtai_tc.cuh.
#pragma once
#include "agl_field.cuh"
#include "common.cuh"

namespace mb {
namespace aj {

constexpr int D = 64;
constexpr int KAPPA = 42;
constexpr int BLOCKS_PER_COL = KAPPA * D / 8;  // 336 ChaCha8 blocks per column

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int n) { return __funnelshift_l(x, x, n); }

#define MB_AJ_QR(a, b, c, d)          \
    a += b; d ^= a; d = rotl32(d, 16); \
    c += d; b ^= c; b = rotl32(b, 12); \
    a += b; d ^= a; d = rotl32(d, 8);  \
    c += d; b ^= c; b = rotl32(b, 7);

// One ChaCha8 block (4 double rounds), 16 output words.
__device__ __forceinline__ void chacha8_block(const uint32_t (&key)[8], uint32_t counter, uint32_t n0, uint32_t n1,
                                              uint32_t n2, uint32_t (&out)[16]) {
    uint32_t s[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, key[0], key[1], key[2], key[3],
                      key[4], key[5], key[6], key[7], counter, n0, n1, n2};
    uint32_t x[16];
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = s[i];
#pragma unroll
    for (int dr = 0; dr < 4; dr++) {
        MB_AJ_QR(x[0], x[4], x[8], x[12]) MB_AJ_QR(x[1], x[5], x[9], x[13])
        MB_AJ_QR(x[2], x[6], x[10], x[14]) MB_AJ_QR(x[3], x[7], x[11], x[15])
        MB_AJ_QR(x[0], x[5], x[10], x[15]) MB_AJ_QR(x[1], x[6], x[11], x[12])
        MB_AJ_QR(x[2], x[7], x[8], x[13]) MB_AJ_QR(x[3], x[4], x[9], x[14])
    }
#pragma unroll
    for (int i = 0; i < 16; i++) out[i] = x[i] + s[i];
}

// The first column round touches the nonce words one column at a time: columns 0, 1 and 3 of the state see only
// the constants, the key, the block counter, the row and the high word of the column index. A thread that
// generates the same (row, counter) for a run of matrix columns computes those three quarter rounds once.
struct ChaChaColumns {
    uint32_t q[12];     // state words (0, 4, 8, 12), (1, 5, 9, 13), (3, 7, 11, 15) after the first column round
    uint32_t n2;        // the high word of the column index they were made for
};
__device__ __forceinline__ void chacha8_columns(const uint32_t (&key)[8], uint32_t counter, uint32_t n0, uint32_t n2,
                                                ChaChaColumns& pre) {
    uint32_t a0 = 0x61707865u, b0 = key[0], c0 = key[4], d0 = counter;
    uint32_t a1 = 0x3320646eu, b1 = key[1], c1 = key[5], d1 = n0;
    uint32_t a3 = 0x6b206574u, b3 = key[3], c3 = key[7], d3 = n2;
    MB_AJ_QR(a0, b0, c0, d0) MB_AJ_QR(a1, b1, c1, d1) MB_AJ_QR(a3, b3, c3, d3)
    pre.q[0] = a0; pre.q[1] = b0; pre.q[2] = c0; pre.q[3] = d0;
    pre.q[4] = a1; pre.q[5] = b1; pre.q[6] = c1; pre.q[7] = d1;
    pre.q[8] = a3; pre.q[9] = b3; pre.q[10] = c3; pre.q[11] = d3;
    pre.n2 = n2;
}
// chacha8_block(key, counter, n0, n1, pre.n2) with the three quarter rounds taken from `pre`.
__device__ __forceinline__ void chacha8_block_pre(const uint32_t (&key)[8], const ChaChaColumns& pre, uint32_t counter,
                                                  uint32_t n0, uint32_t n1, uint32_t (&out)[16]) {
    uint32_t x[16];
    x[0] = pre.q[0]; x[4] = pre.q[1]; x[8] = pre.q[2]; x[12] = pre.q[3];
    x[1] = pre.q[4]; x[5] = pre.q[5]; x[9] = pre.q[6]; x[13] = pre.q[7];
    x[3] = pre.q[8]; x[7] = pre.q[9]; x[11] = pre.q[10]; x[15] = pre.q[11];
    x[2] = 0x79622d32u; x[6] = key[2]; x[10] = key[6]; x[14] = n1;
    MB_AJ_QR(x[2], x[6], x[10], x[14])
    MB_AJ_QR(x[0], x[5], x[10], x[15]) MB_AJ_QR(x[1], x[6], x[11], x[12])
    MB_AJ_QR(x[2], x[7], x[8], x[13]) MB_AJ_QR(x[3], x[4], x[9], x[14])
#pragma unroll
    for (int dr = 1; dr < 4; dr++) {
        MB_AJ_QR(x[0], x[4], x[8], x[12]) MB_AJ_QR(x[1], x[5], x[9], x[13])
        MB_AJ_QR(x[2], x[6], x[10], x[14]) MB_AJ_QR(x[3], x[7], x[11], x[15])
        MB_AJ_QR(x[0], x[5], x[10], x[15]) MB_AJ_QR(x[1], x[6], x[11], x[12])
        MB_AJ_QR(x[2], x[7], x[8], x[13]) MB_AJ_QR(x[3], x[4], x[9], x[14])
    }
    const uint32_t s[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, key[0], key[1], key[2], key[3],
                            key[4], key[5], key[6], key[7], counter, n0, n1, pre.n2};
#pragma unroll
    for (int i = 0; i < 16; i++) out[i] = x[i] + s[i];
}

// Coefficients 8*block_idx .. 8*block_idx+7 of M[row][j]: the words of blocks
// counter = block_idx, block_idx + 8, ... that are below q, first eight kept
// (at most 16 blocks; a word is rejected with probability about 2^-31).
__device__ __forceinline__ void prg_ring_block(const uint32_t (&key)[8], uint32_t row, uint64_t j, uint32_t block_idx,
                                               uint64_t (&out)[8]) {
    uint32_t buf[16];
    chacha8_block(key, block_idx, row, (uint32_t)j, (uint32_t)(j >> 32), buf);
    bool ok = true;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        out[k] = ((uint64_t)buf[2 * k + 1] << 32) | buf[2 * k];
        ok = ok && (out[k] < agl::P);
    }
    if (ok) return;
    // rare path: restart and keep accepted words in order
    uint64_t tmp[8];
#pragma unroll
    for (int k = 0; k < 8; k++) tmp[k] = 0;
    int written = 0;
    for (uint32_t retry = 0; retry < 16 && written < 8; retry++) {
        chacha8_block(key, block_idx + 8u * retry, row, (uint32_t)j, (uint32_t)(j >> 32), buf);
        for (int k = 0; k < 8 && written < 8; k++) {
            uint64_t v = ((uint64_t)buf[2 * k + 1] << 32) | buf[2 * k];
            if (v < agl::P) {
                // static-index write keeps tmp in registers
#pragma unroll
                for (int w = 0; w < 8; w++)
                    if (w == written) tmp[w] = v;
                written++;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 8; k++) out[k] = tmp[k];
}

// prg_ring_block for a thread that keeps `pre` = chacha8_columns(key, block_idx, row, high word of j) across
// columns. A coefficient is rejected only when its high word is 0xFFFFFFFE or 0xFFFFFFFF (q = 2^64 - 2^32 - 31),
// so one comparison per coefficient decides whether the exact path has to look.
__device__ __forceinline__ void prg_ring_block_pre(const uint32_t (&key)[8], ChaChaColumns& pre, uint32_t row, uint64_t j,
                                                   uint32_t block_idx, uint64_t (&out)[8]) {
    if ((uint32_t)(j >> 32) != pre.n2) chacha8_columns(key, block_idx, row, (uint32_t)(j >> 32), pre);
    uint32_t buf[16];
    chacha8_block_pre(key, pre, block_idx, row, (uint32_t)j, buf);
    bool ok = true;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        out[k] = ((uint64_t)buf[2 * k + 1] << 32) | buf[2 * k];
        ok = ok && (buf[2 * k + 1] < 0xFFFFFFFEu);
    }
    if (ok) return;
    prg_ring_block(key, row, j, block_idx, out);
}

enum Kind { KIND_BITS = 0, KIND_S8 = 1, KIND_WIDE = 2 };

// ---- scalar commit -----------------------------------------------------------------
// grid = (column chunks, planes); block = 384 threads. Per column the block
// fills M (42 x 64 coefficients) in shared memory, then thread t accumulates
// outputs (i, r) = t, t + 384, ... (7 per thread):
//   bits / s8:  exact 128-bit sums of the wrapped (negative) and unwrapped
//               (positive) terms, one reduction of each per column;
//   wide:       a modular multiply-add per term.
// partial[(chunk * planes + p) * 2688 + i * 64 + r] = canonical chunk sum.
template <int KIND>
__global__ void __launch_bounds__(384)
commit_scalar_kernel(const uint32_t* __restrict__ d_key, const void* __restrict__ z, uint64_t N, uint64_t col_offset,
                     uint64_t cols_per_chunk, uint64_t* __restrict__ partial, const uint64_t* __restrict__ premat = nullptr) {
    __shared__ uint64_t M_sh[KAPPA * D];
    __shared__ uint64_t zw_sh[D];   // wide coefficients / bit mask in [0]
    __shared__ int8_t zd_sh[D];
    uint32_t key[8];
#pragma unroll
    for (int k = 0; k < 8; k++) key[k] = premat ? 0u : d_key[k];
    const int t = threadIdx.x, p = blockIdx.y;
    const uint64_t j0 = (uint64_t)blockIdx.x * cols_per_chunk;
    const uint64_t j1 = j0 + cols_per_chunk < N ? j0 + cols_per_chunk : N;
    uint64_t acc[7];
#pragma unroll
    for (int q = 0; q < 7; q++) acc[q] = 0;
    for (uint64_t j = j0; j < j1; j++) {
        __syncthreads();
        if (premat) {  // a matrix materialised earlier: [column][row][coefficient]
#pragma unroll
            for (int q = 0; q < 7; q++) M_sh[t + 384 * q] = agl::canon(premat[(col_offset + j) * (uint64_t)(KAPPA * D) + t + 384 * q]);
        } else if (t < BLOCKS_PER_COL) {
            uint64_t c[8];
            prg_ring_block(key, (uint32_t)(t >> 3), col_offset + j, (uint32_t)(t & 7), c);
#pragma unroll
            for (int k = 0; k < 8; k++) M_sh[(t >> 3) * D + (t & 7) * 8 + k] = c[k];
        }
        if (KIND == KIND_BITS) {
            if (t == 0) zw_sh[0] = static_cast<const uint64_t*>(z)[(size_t)p * N + j];
        } else if (KIND == KIND_S8) {
            if (t < D) zd_sh[t] = static_cast<const int8_t*>(z)[((size_t)p * N + j) * D + t];
        } else {
            if (t < D) zw_sh[t] = agl::canon(static_cast<const uint64_t*>(z)[((size_t)p * N + j) * D + t]);
        }
        __syncthreads();
        if (KIND == KIND_BITS && zw_sh[0] == 0) continue;
#pragma unroll
        for (int q = 0; q < 7; q++) {
            const int o = t + 384 * q, i = o >> 6, r = o & 63;
            const uint64_t* m = M_sh + i * D;
            if (KIND == KIND_WIDE) {
                uint64_t a = acc[q];
                for (int l = 0; l < D; l++) {
                    uint64_t prod = agl::mul(m[(r - l) & 63], zw_sh[l]);
                    a = l <= r ? agl::add(a, prod) : agl::sub(a, prod);
                }
                acc[q] = a;
            } else {
                // exact sums: positive terms (l <= r) and wrapped terms (l > r), 128 bits each,
                // with signed digits split by sign
                uint64_t plo = 0, phi = 0, nlo = 0, nhi = 0;
                const uint64_t bits = KIND == KIND_BITS ? zw_sh[0] : 0;
                for (int l = 0; l < D; l++) {
                    int d = KIND == KIND_BITS ? (int)((bits >> l) & 1) : (int)zd_sh[l];
                    if (d == 0) continue;
                    uint64_t mv = m[(r - l) & 63];
                    uint32_t ad = (uint32_t)(d < 0 ? -d : d);
                    uint64_t lo = mv * ad, hi = __umul64hi(mv, (uint64_t)ad);
                    bool positive = (l <= r) == (d > 0);
                    if (positive) {
                        plo += lo;
                        phi += hi + (plo < lo);
                    } else {
                        nlo += lo;
                        nhi += hi + (nlo < lo);
                    }
                }
                acc[q] = agl::add(acc[q], agl::sub(agl::reduce128(plo, phi), agl::reduce128(nlo, nhi)));
            }
        }
    }
#pragma unroll
    for (int q = 0; q < 7; q++)
        partial[((size_t)blockIdx.x * gridDim.y + p) * (KAPPA * D) + t + 384 * q] = agl::canon(acc[q]);
}

// out[k] = sum over chunks of partial[chunk][k], k < planes * 2688.
static __global__ void reduce_chunks_kernel(const uint64_t* __restrict__ partial, size_t chunks, size_t width,
                                            uint64_t* __restrict__ out) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < width; k += step) {
        uint64_t a = 0;
        for (size_t c = 0; c < chunks; c++) a = agl::add(a, partial[c * width + k]);
        out[k] = agl::canon(a);
    }
}

// Ternary planes to signed digits: digits[(p * N + j) * 64 + l] = +1 / -1 / 0 from the bit
// masks pos[p * N + j], neg[p * N + j] (disjoint; cuda_almost_goldilocks/ajtai.cuh:1262-1270).
static __global__ void ternary_expand_kernel(const uint64_t* __restrict__ pos, const uint64_t* __restrict__ neg,
                                             size_t words, int8_t* __restrict__ digits) {
    const size_t total = words * 4, step = (size_t)gridDim.x * blockDim.x;  // 16 digits per thread and step
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
        const size_t w = t >> 2;
        const int part = (int)(t & 3);
        const uint32_t pm = (uint32_t)(pos[w] >> (16 * part)) & 0xFFFFu, nm = (uint32_t)(neg[w] >> (16 * part)) & 0xFFFFu;
        uint32_t v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int l = 4 * q + b;
                const uint32_t d = ((pm >> l) & 1u) ? 1u : (((nm >> l) & 1u) ? 0xFFu : 0u);
                word |= d << (8 * b);
            }
            v[q] = word;
        }
        *reinterpret_cast<uint4*>(digits + w * 64 + 16 * part) = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// Signed 16-bit coefficients to ternary bit planes: plane i holds bit i of |v|, in pos when v >= 0,
// in neg otherwise; |v| >= 2^k_chunks raises *err (almost_sumcheck_prover.cuh:447-478).
static __global__ void wide_to_ternary_kernel(const int16_t* __restrict__ wide, uint64_t* __restrict__ pos,
                                              uint64_t* __restrict__ neg, int* err, size_t n_ring, int k_chunks) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_ring; j += step) {
        uint64_t p[16], n[16];
#pragma unroll
        for (int i = 0; i < 16; i++) p[i] = n[i] = 0;
        bool bad = false;
        for (int k = 0; k < 64; k++) {
            const int v = wide[j * 64 + k];
            const uint32_t a = (uint32_t)(v < 0 ? -v : v);
            bad |= (a >> k_chunks) != 0;
            const uint64_t bit = 1ULL << k;
#pragma unroll
            for (int i = 0; i < 16; i++)
                if (i < k_chunks && ((a >> i) & 1u)) {
                    if (v < 0) n[i] |= bit; else p[i] |= bit;
                }
        }
        if (bad) atomicExch(err, 1);
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (i < k_chunks) {
                pos[(size_t)i * n_ring + j] = p[i];
                neg[(size_t)i * n_ring + j] = n[i];
            }
    }
}

// Sparse commit: c_i = sum over positions p of X^(p mod 64) M[i][p / 64] (ajtai_cpu_reference.cuh:192-219).
// One block per chunk of positions; the column's 42 ring elements are regenerated only when the column
// changes, so sorted position lists cost one generation per distinct column. partial[chunk][42 * 64].
static __global__ void __launch_bounds__(384)
commit_sparse_kernel(const uint32_t* __restrict__ d_key, const uint64_t* __restrict__ positions, uint64_t K,
                     uint64_t per_chunk, uint64_t* __restrict__ partial) {
    __shared__ uint64_t M_sh[KAPPA * D];
    uint32_t key[8];
#pragma unroll
    for (int k = 0; k < 8; k++) key[k] = d_key[k];
    const int t = threadIdx.x;
    const uint64_t k0 = (uint64_t)blockIdx.x * per_chunk, k1 = k0 + per_chunk < K ? k0 + per_chunk : K;
    uint64_t acc[7];
#pragma unroll
    for (int q = 0; q < 7; q++) acc[q] = 0;
    uint64_t have = ~0ULL;
    for (uint64_t k = k0; k < k1; k++) {
        const uint64_t pidx = positions[k], j = pidx >> 6;
        const int ell = (int)(pidx & 63);
        if (j != have) {
            __syncthreads();
            if (t < BLOCKS_PER_COL) {
                uint64_t c[8];
                prg_ring_block(key, (uint32_t)(t >> 3), j, (uint32_t)(t & 7), c);
#pragma unroll
                for (int q = 0; q < 8; q++) M_sh[(t >> 3) * D + (t & 7) * 8 + q] = c[q];
            }
            __syncthreads();
            have = j;
        }
#pragma unroll
        for (int q = 0; q < 7; q++) {
            const int o = t + 384 * q, i = o >> 6, r = o & 63;
            const uint64_t mv = M_sh[i * D + ((r - ell) & 63)];
            acc[q] = r >= ell ? agl::add(acc[q], mv) : agl::sub(acc[q], mv);
        }
    }
#pragma unroll
    for (int q = 0; q < 7; q++) partial[(size_t)blockIdx.x * (KAPPA * D) + t + 384 * q] = agl::canon(acc[q]);
}

// M[j][i][k] for j < N (the layout of ajtai_materialize_m_ffi, cuda_almost_goldilocks/ajtai_premat.cuh:41-84).
static __global__ void materialize_kernel(const uint32_t* __restrict__ d_key, uint64_t* __restrict__ M, uint64_t N,
                                          uint64_t col_offset) {
    uint32_t key[8];
#pragma unroll
    for (int k = 0; k < 8; k++) key[k] = d_key[k];
    const uint64_t total = N * BLOCKS_PER_COL;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += step) {
        uint64_t j = g / BLOCKS_PER_COL;
        uint32_t b = (uint32_t)(g % BLOCKS_PER_COL);
        uint64_t c[8];
        prg_ring_block(key, b >> 3, col_offset + j, b & 7, c);
        ulonglong2* dst = reinterpret_cast<ulonglong2*>(M + g * 8);
#pragma unroll
        for (int k = 0; k < 4; k++) dst[k] = make_ulonglong2(c[2 * k], c[2 * k + 1]);
    }
}

}  // namespace aj
}  // namespace mb
