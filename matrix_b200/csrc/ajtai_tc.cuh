// Ajtai commitment of small signed digits on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory).
//
// c[p][i][r] = sum_j sum_k M[i][j][k] * T_{p,j}[k][r],   T[k][r] = z[r-k] (k <= r), -z[r-k+64] (k > r)
// is a GEMM with exact integer arithmetic once the 64-bit matrix coefficients
// are split into eight unsigned byte planes (the decomposition of the reference's
// mma.sync kernel, cuda_almost_goldilocks/ajtai.cuh:1506-1668):
//   A[(i, b)][(j, k)] = byte b of M[i][j][k]            u8, rows = 14 matrix rows x 8 planes (+16 zero rows)
//   B[(p, r)][(j, k)] = T_{p,j}[k][r]                    s8, negacyclic Toeplitz expansion of the digits
//   D[(i, b)][(p, r)] = sum over (j, k)                  s32 in tensor memory
// and c = sum_b 2^(8b) D[(i, b)] mod q. With |digit| <= 127 a sum over 512
// columns (K = 32768) stays below 255 * 127 * 32768 < 2^31, so the accumulators
// are drained every 512 columns.
//
// One CTA owns a chunk of columns and one of three groups of 14 matrix rows, so
// no ChaCha8 block is generated twice. Per stage of four columns its 256 threads
// generate the A bytes (the dominant cost: 112 ChaCha8 blocks per column) and
// expand the digits into B, both in the no-swizzle K-major core-matrix layout
// (8 rows x 16 bytes, cores contiguous along K), then one thread issues eight
// K = 32 MMAs and commits them to an mbarrier that gates the reuse of the
// buffers. Every wait is bounded and reports through an error word instead of
// spinning forever.
#pragma once
#include "ajtai_kernels.cuh"

namespace mb {
namespace aj {

constexpr int TC_ROWS = 14;             // matrix rows per CTA (3 groups cover 42)
constexpr int TC_STAGE_COLS = 4;        // columns per MMA stage
constexpr int TC_STAGE_K = TC_STAGE_COLS * D;   // 256 bytes of K per stage
constexpr int TC_CHUNK_COLS = 512;      // columns per accumulation (s32 exactness)
constexpr int TC_MAX_PLANES = 4;        // digit planes per CTA: N = 64 * planes <= 256
constexpr int TC_THREADS = 256;
constexpr uint32_t TC_CORE = 128;       // bytes of one 8 x 16 core matrix
constexpr uint32_t TC_SBO = (TC_STAGE_K / 16) * TC_CORE;  // 2048: next 8-row group
constexpr uint32_t TC_A_BYTES = 16 * TC_SBO;              // 128 rows
constexpr int TC_V_STRIDE = 144;        // bytes per reversed digit window (128 + padding, 16-byte multiple)

enum TcError { TC_OK = 0, TC_ERR_DIGIT_RANGE = 1, TC_ERR_TIMEOUT = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, K-major, no swizzle: start address, byte
// distance between core matrices along K (leading), along M/N (stride).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ULL << 46);
}

// kind::i8 instruction descriptor: D = s32, A = u8, B = s8, both K-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int n) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// Bounded wait for an mbarrier phase; false on timeout.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 20); it++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// grid = (column chunks, 3 row groups); block = 256 threads; dynamic shared memory.
// d_digits: [planes][N][64] s8 (this CTA uses planes p0 .. p0 + np - 1).
// partial[((chunk * 3 + group) * np + p) * 14 * 64 + i_local * 64 + r] = canonical chunk sum.
static __global__ void __launch_bounds__(TC_THREADS)
commit_tc_kernel(const uint32_t* __restrict__ d_key, const int8_t* __restrict__ d_digits, uint64_t N, int p0, int np,
                 uint64_t col_offset, uint64_t* __restrict__ partial, int* __restrict__ d_error) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int n_cols = 64 * np;                       // UMMA N
    uint8_t* A_sh = smem;                             // 32 KB
    uint8_t* B_sh = smem + TC_A_BYTES;                // (n_cols / 8) * 2048
    uint8_t* V_sh = B_sh + (size_t)(n_cols / 8) * TC_SBO;  // [4 cols][np][144]
    int8_t* Z_sh = reinterpret_cast<int8_t*>(V_sh + TC_STAGE_COLS * TC_MAX_PLANES * TC_V_STRIDE);  // [4][np][64]
    __shared__ __align__(8) uint64_t mbar;
    __shared__ uint32_t tmem_base_sh;

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int group = blockIdx.y;
    const uint64_t j0 = (uint64_t)blockIdx.x * TC_CHUNK_COLS;
    const uint64_t j1 = j0 + TC_CHUNK_COLS < N ? j0 + TC_CHUNK_COLS : N;
    uint32_t key[8];
#pragma unroll
    for (int k = 0; k < 8; k++) key[k] = d_key[k];

    // zero the padding rows 112..127 of A (row groups 14, 15) once
    for (int x = t; x < (int)(2 * TC_SBO / 16); x += TC_THREADS)
        reinterpret_cast<uint4*>(A_sh + 14 * TC_SBO)[x] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar)));
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(256u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;");
    const uint32_t tmem = tmem_base_sh;
    const uint32_t bar = smem_u32(&mbar);
    const uint32_t idesc = umma_idesc_i8(n_cols);
    uint32_t phase = 0;
    bool first = true, failed = false;
    int bad_digit = 0;

    for (uint64_t js = j0; js < j1 && !failed; js += TC_STAGE_COLS) {
        // the previous stage's MMAs must have read A and B before they are overwritten
        if (!first) {
            if (!mbar_wait(bar, phase)) failed = true;
            phase ^= 1;
            if (__syncthreads_or(failed)) { failed = true; break; }
        }
        // ---- digits of this stage (zero beyond the last column) ----
        for (int x = t; x < TC_STAGE_COLS * np * D; x += TC_THREADS) {
            int jj = x / (np * D), rem = x % (np * D), p = rem / D, l = rem % D;
            int8_t dgt = 0;
            if (js + jj < j1) dgt = d_digits[((size_t)(p0 + p) * N + js + jj) * D + l];
            if (dgt == -128) bad_digit = 1;
            Z_sh[x] = dgt;
        }
        // ---- A: byte planes of the generated matrix coefficients ----
        for (int job = t; job < TC_STAGE_COLS * TC_ROWS * 8; job += TC_THREADS) {
            int jj = job / (TC_ROWS * 8), rem = job % (TC_ROWS * 8), il = rem >> 3, blk = rem & 7;
            uint64_t c[8];
            prg_ring_block(key, (uint32_t)(group * TC_ROWS + il), col_offset + js + jj, (uint32_t)blk, c);
            uint32_t kk = (uint32_t)(jj * D + 8 * blk);
            uint8_t* dst = A_sh + il * TC_SBO + (kk >> 4) * TC_CORE + (kk & 15);
            // Two lanes fill one 128-byte core (8 plane rows x 16 bytes). The plane order is rotated by the
            // lane pair so that the lanes of a store instruction spread over the rows (banks) instead of
            // all writing the same row of different cores.
            const int rot = (t >> 1) & 3;
#pragma unroll
            for (int b = 0; b < 8; b++) {
                const int bp = (b & 4) | ((b + rot) & 3);
                uint32_t w[8];
#pragma unroll
                for (int x = 0; x < 8; x++) w[x] = b < 4 ? (uint32_t)c[x] : (uint32_t)(c[x] >> 32);
                const uint32_t sel = (uint32_t)(bp & 3) | ((4u + (uint32_t)(bp & 3)) << 4);
                uint32_t lo = __byte_perm(__byte_perm(w[0], w[1], sel), __byte_perm(w[2], w[3], sel), 0x5410);
                uint32_t hi = __byte_perm(__byte_perm(w[4], w[5], sel), __byte_perm(w[6], w[7], sel), 0x5410);
                *reinterpret_cast<uint2*>(dst + bp * 16) = make_uint2(lo, hi);
            }
        }
        __syncthreads();
        // ---- w: the reversed, sign-wrapped digit window of every (column, plane): w[i] = z[63 - i] for i < 64,
        // -z[127 - i] for 64 <= i < 128, one word (four digits) per thread and step; word 32 is padding ----
        for (int x = t; x < TC_STAGE_COLS * np * 33; x += TC_THREADS) {
            const int cp = x / 33, q = x % 33;  // cp = jj * np + p
            const uint32_t* zw = reinterpret_cast<const uint32_t*>(Z_sh + cp * D);
            uint32_t v = 0;
            if (q < 16) v = __byte_perm(zw[15 - q], 0, 0x0123);
            else if (q < 32) v = __vneg4(__byte_perm(zw[31 - q], 0, 0x0123));
            reinterpret_cast<uint32_t*>(V_sh + cp * TC_V_STRIDE)[q] = v;
        }
        __syncthreads();
        // ---- B[(p, r)][(jj, k)] = w[63 - r + k], 16-byte chunks along k cut out of w at any byte offset
        // (five aligned words, funnel shifts). Consecutive lanes take consecutive rows of one core (16 bytes
        // apart): a store instruction covers whole 128-byte cores. ----
        for (int x = t; x < n_cols * 16; x += TC_THREADS) {
            int n = ((x >> 7) << 3) | (x & 7), kc = (x >> 3) & 15, p = n >> 6, r = n & 63, jj = kc >> 2, cq = kc & 3;
            const int s0 = 63 - r + 16 * cq, sh = 8 * (s0 & 3);
            const uint32_t* src = reinterpret_cast<const uint32_t*>(V_sh + (jj * np + p) * TC_V_STRIDE) + (s0 >> 2);
            const uint32_t w0 = src[0], w1 = src[1], w2 = src[2], w3 = src[3], w4 = src[4];
            uint4 v = make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh),
                                 __funnelshift_r(w3, w4, sh));
            *reinterpret_cast<uint4*>(B_sh + (n >> 3) * TC_SBO + kc * TC_CORE + (n & 7) * 16) = v;
        }
        // generic-proxy writes -> visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (t == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;");
            const uint32_t a_addr = smem_u32(A_sh), b_addr = smem_u32(B_sh);
#pragma unroll 1
            for (int ks = 0; ks < TC_STAGE_K / 32; ks++) {
                uint64_t da = umma_desc(a_addr + ks * 2 * TC_CORE, TC_CORE, TC_SBO);
                uint64_t db = umma_desc(b_addr + ks * 2 * TC_CORE, TC_CORE, TC_SBO);
                uint32_t acc = (first && ks == 0) ? 0u : 1u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
        }
        first = false;
    }
    // ---- all MMAs of the chunk done ----
    if (!first && !failed) {
        if (!mbar_wait(bar, phase)) failed = true;
    }
    if (__syncthreads_or(failed)) failed = true;
    asm volatile("tcgen05.fence::after_thread_sync;");

    if (!failed && !first) {
        // Drain: warp w reads TMEM lanes 32 (w & 3) ..+31 (row m = lane), warps 0-3 the first
        // half of the columns, warps 4-7 the second. Row m = 8 i_local + b: the eight byte
        // planes of one matrix row sit in eight consecutive lanes and are combined with a
        // three-step butterfly of field additions after scaling by 2^(8b).
        const int q = warp & 3, half = warp >> 2;
        const int m = 32 * q + lane, b = m & 7, il = m >> 3;
        const uint64_t scale = 1ULL << (8 * b);  // < 2^56, canonical
        const int c_lo = half * (n_cols / 2), c_hi = c_lo + n_cols / 2;
        for (int c0 = c_lo; c0 < c_hi; c0 += 8) {
            uint32_t v[8];
            uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)c0;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                         : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 8; e++) {
                int32_t sv = (int32_t)v[e];
                uint64_t f = sv >= 0 ? (uint64_t)sv : agl::P - (uint64_t)(-(int64_t)sv);
                f = agl::mul(f, scale);
#pragma unroll
                for (int off = 1; off < 8; off <<= 1) f = agl::add(f, __shfl_xor_sync(0xffffffffu, f, off));
                if (b == 0 && il < TC_ROWS) {
                    int n = c0 + e, p = n >> 6, r = n & 63;
                    partial[(((size_t)blockIdx.x * 3 + group) * np + p) * (TC_ROWS * D) + il * D + r] = agl::canon(f);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u));
    if (failed && t == 0) atomicMax(d_error, (int)TC_ERR_TIMEOUT);
    if (bad_digit) atomicMax(d_error, (int)TC_ERR_DIGIT_RANGE);
}

// out[p][i][r] = sum over chunks of partial[chunk][group = i / 14][p][i % 14][r]
static __global__ void reduce_tc_partials_kernel(const uint64_t* __restrict__ partial, size_t chunks, int np,
                                                 uint64_t* __restrict__ out) {
    const size_t width = (size_t)np * KAPPA * D;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < width; k += step) {
        int p = (int)(k / (KAPPA * D)), i = (int)((k / D) % KAPPA), r = (int)(k % D);
        int g = i / TC_ROWS, il = i % TC_ROWS;
        uint64_t a = 0;
        for (size_t c = 0; c < chunks; c++)
            a = agl::add(a, partial[((c * 3 + g) * np + p) * (TC_ROWS * D) + il * D + r]);
        out[k] = agl::canon(a);
    }
}

inline size_t tc_smem_bytes(int np) {
    return TC_A_BYTES + (size_t)(64 * np / 8) * TC_SBO + TC_STAGE_COLS * TC_MAX_PLANES * TC_V_STRIDE +
           TC_STAGE_COLS * TC_MAX_PLANES * D;
}

}  // namespace aj
}  // namespace mb
