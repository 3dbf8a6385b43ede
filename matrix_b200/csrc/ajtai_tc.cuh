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
// One CTA owns a chunk of at most 512 columns and one of three groups of 14 matrix rows, so no ChaCha8 block
// is generated twice. It works in stages of four columns (K = 256): eight K = 32 MMAs per stage, committed to
// the mbarrier of the stage's operand buffer; a buffer is rewritten only after that commit has landed. Operands
// use the no-swizzle K-major core-matrix layout (8 rows x 16 bytes, cores contiguous along K). Every wait is
// bounded and reports through an error word instead of spinning forever. Two kernels follow: commit_tc_pipe
// (all threads build a stage, one of them issues it; kept for the mode that writes the matrix images out) and
// commit_tc_ws (builder warps and an issuing warp, the commit path).
//
// B (the Toeplitz expansion) is never written out as 64 x 64 bytes per (column, plane). With the rows taken in
// reverse (MMA column n = 63 - r) entry (n, k) is w[n + k], w the reversed, sign-wrapped digit window of the
// (column, plane) (128 bytes), so the 8 x 16 core matrix at row group g and K block c holds rows
// w[8 (g + 2 c) + i .. + 15], i = 0..7: it depends on g + 2 c only. The operand is therefore stored as 112
// consecutive 16-byte rows, row o = w[o .. o + 15] (1792 bytes instead of 4096), and addressed with a stride of
// 128 bytes between row groups and 256 bytes between K blocks, so that the core matrices of the descriptor
// overlap in shared memory. In commit_tc_pipe every plane has its own image and its own MMA of N = 64;
// commit_tc_ws interleaves the planes of a column by core matrix (strides 128 and 256 x planes), which puts all
// planes behind one descriptor and one MMA of N = 64 x planes.
//
// Where the matrix comes from (TcSource): the ChaCha8 stream; d_M[j][i][k] as 64-bit coefficients (split into
// byte planes here); or d_T, the byte planes already in operand order: per stage of four columns and row group
// the 28 KB image of the A buffer, [stage][group][14 x 2048] (written by this kernel in its materialise mode),
// which is copied as is.
#pragma once
#include "ajtai_kernels.cuh"

namespace mb {
namespace aj {

constexpr int TC_ROWS = 14;             // matrix rows per CTA (3 groups cover 42)
constexpr int TC_STAGE_COLS = 4;        // columns per MMA stage
constexpr int TC_STAGE_K = TC_STAGE_COLS * D;   // 256 bytes of K per stage
constexpr int TC_CHUNK_COLS = 512;      // most columns per accumulation (s32 exactness)
constexpr int TC_CHUNK_MIN = 32;        // fewest columns per CTA: below that the set-up and the epilogue dominate
constexpr int TC_MAX_PLANES = 4;        // digit planes per CTA: N = 64 * planes <= 256
constexpr uint32_t TC_CORE = 128;       // bytes of one 8 x 16 core matrix
constexpr uint32_t TC_SBO = (TC_STAGE_K / 16) * TC_CORE;  // 2048: next 8-row group
constexpr uint32_t TC_A_BYTES = 16 * TC_SBO;              // 128 rows
constexpr int TC_V_STRIDE = 144;        // bytes per reversed digit window (128 + padding, 16-byte multiple)
constexpr int TC_B_ROWS = 112;          // sliding 16-byte rows of one (column, plane): offsets 0 .. 111
constexpr uint32_t TC_B_IMAGE = TC_B_ROWS * 16;   // 1792 bytes per (column, plane)

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

constexpr int TCP_THREADS = 512;                    // sixteen warps hide the latencies of the build
enum TcSource { TC_SRC_CHACHA = 0, TC_SRC_COEFFS = 1, TC_SRC_TILED = 2 };
constexpr uint32_t TCP_A_IMAGE = 14 * TC_SBO;       // 28672 bytes: the rows of the A buffer that hold data

// grid = (column chunks of chunk_cols columns, a multiple of 4 and at most 512; 3 row groups); dynamic shared memory tc_pipe_smem_bytes(np).
// d_digits: [planes][N][64] s8 (this CTA uses planes p0 .. p0 + np - 1, np <= 4: N = 64 np columns of one MMA).
// partial[((chunk * 3 + group) * np + p) * 14 * 64 + i_local * 64 + r] = canonical chunk sum.
// materialize != nullptr: no digits, no MMAs; the A images of this CTA's stages are written there instead.
// The number of planes of the pass is a template parameter: the index arithmetic of the build (which column,
// plane, row a task works on) folds to shifts and constants.
template <int SRC, int NP>
static __global__ void __launch_bounds__(TCP_THREADS, 1)
commit_tc_pipe_kernel(const uint32_t* __restrict__ d_key, const uint64_t* __restrict__ d_M, const uint8_t* __restrict__ d_T,
                      const int8_t* __restrict__ d_digits, uint64_t N, int p0, uint64_t col_offset, uint64_t* __restrict__ partial,
                      int* __restrict__ d_error, uint8_t* __restrict__ materialize, int chunk_cols) {
    constexpr int np = NP;
    constexpr bool PREMAT = SRC == TC_SRC_COEFFS;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int n_cols = 64 * np;
    const size_t b_bytes = (size_t)TC_STAGE_COLS * np * TC_B_IMAGE, buf_bytes = TC_A_BYTES + b_bytes;
    uint8_t* V_sh = smem + 2 * buf_bytes;
    __shared__ __align__(8) uint64_t mbar[2];
    __shared__ uint32_t tmem_base_sh;

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int group = blockIdx.y;
    const uint64_t j0 = (uint64_t)blockIdx.x * (uint64_t)chunk_cols;
    const uint64_t j1 = j0 + (uint64_t)chunk_cols < N ? j0 + (uint64_t)chunk_cols : N;
    uint32_t key[8];
#pragma unroll
    for (int k = 0; k < 8; k++) key[k] = SRC == TC_SRC_CHACHA ? d_key[k] : 0u;
    const uint32_t tmem_cols = 256u;

    for (int x = t; x < TC_STAGE_COLS * TC_MAX_PLANES * TC_V_STRIDE / 4; x += TCP_THREADS) reinterpret_cast<uint32_t*>(V_sh)[x] = 0;
    for (int b = 0; b < 2; b++)   // zero padding rows 112..127 of both A buffers
        for (int x = t; x < (int)(2 * TC_SBO / 16); x += TCP_THREADS)
            reinterpret_cast<uint4*>(smem + b * buf_bytes + 14 * TC_SBO)[x] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;");
    const uint32_t tmem = tmem_base_sh;
    const uint32_t idesc = umma_idesc_i8(64);   // one plane per MMA
    bool failed = false;
    int bad_digit = 0;

    // what one thread fetches for a stage: four digits, and the 8 coefficients of up to two (column, row, block) jobs
    constexpr int JOBS = TC_STAGE_COLS * TC_ROWS * 8;   // 448
    uint32_t zreg = 0;
    ulonglong2 creg[4];
    uint4 treg[4];   // TILED: 1792 16-byte pieces of the A image over 512 threads
    auto fetch = [&](uint64_t js) {
        const int x4 = 4 * t;   // digits x4 .. x4 + 3 of the stage's [col][plane][64] block
        zreg = 0;
        if (!materialize && x4 < TC_STAGE_COLS * np * D) {
            const int jj = x4 / (np * D), rem = x4 % (np * D), p = rem / D, l = rem % D;
            if (js + jj < j1) zreg = *reinterpret_cast<const uint32_t*>(d_digits + ((size_t)(p0 + p) * N + js + jj) * D + l);
        }
        if (SRC == TC_SRC_TILED) {
            const uint4* src = reinterpret_cast<const uint4*>(d_T + ((js / TC_STAGE_COLS) * 3 + (uint64_t)group) * TCP_A_IMAGE);
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const int piece = t + x * TCP_THREADS;
                treg[x] = piece < (int)(TCP_A_IMAGE / 16) ? __ldcs(src + piece) : make_uint4(0, 0, 0, 0);
            }
        }
        if (PREMAT) {
            const int job = t;
            const int jj = job / (TC_ROWS * 8), rem = job % (TC_ROWS * 8), il = rem >> 3, blk = rem & 7;
            const bool on = job < JOBS && js + jj < j1;
            const ulonglong2* src = reinterpret_cast<const ulonglong2*>(
                d_M + ((js + jj) * (uint64_t)KAPPA + (uint64_t)(group * TC_ROWS + il)) * D + 8 * blk);
#pragma unroll
            for (int x = 0; x < 4; x++) creg[x] = on ? __ldcs(src + x) : make_ulonglong2(0, 0);
        }
    };
    const int n_stages = (int)((j1 - j0 + TC_STAGE_COLS - 1) / TC_STAGE_COLS);
    if (n_stages > 0) fetch(j0);

    for (int sidx = 0; sidx < n_stages && !failed; sidx++) {
        const uint64_t js = j0 + (uint64_t)sidx * TC_STAGE_COLS;
        const int buf = sidx & 1;
        uint8_t* A_sh = smem + buf * buf_bytes;
        uint8_t* B_sh = A_sh + TC_A_BYTES;
        // ---- reversed, sign-wrapped digit windows straight from the prefetched digits: the z word zi of a
        // (column, plane) is window word 15 - zi reversed, and word 31 - zi reversed and negated ----
        if (4 * t < TC_STAGE_COLS * np * D) {
            if (((zreg & 0xffu) == 0x80u) | ((zreg & 0xff00u) == 0x8000u) | ((zreg & 0xff0000u) == 0x800000u) | ((zreg >> 24) == 0x80u))
                bad_digit = 1;
            uint32_t* win = reinterpret_cast<uint32_t*>(V_sh + (t >> 4) * TC_V_STRIDE);
            const uint32_t rev = __byte_perm(zreg, 0, 0x0123);
            win[15 - (t & 15)] = rev;
            win[31 - (t & 15)] = __vneg4(rev);
        }
        // the MMAs that last read this buffer must be done before it is rewritten
        if (sidx >= 2 && !materialize) {
            if (!mbar_wait(smem_u32(&mbar[buf]), (uint32_t)(((sidx >> 1) - 1) & 1))) failed = true;
        }
        if (__syncthreads_or(failed)) { failed = true; break; }
        // ---- A: byte planes of the matrix coefficients ----
        if (SRC == TC_SRC_TILED) {
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const int piece = t + x * TCP_THREADS;
                if (piece < (int)(TCP_A_IMAGE / 16)) reinterpret_cast<uint4*>(A_sh)[piece] = treg[x];
            }
        } else {
            const int job = t;   // 448 jobs, one per thread
            if (job < JOBS) {
                const int jj = job / (TC_ROWS * 8), rem = job % (TC_ROWS * 8), il = rem >> 3, blk = rem & 7;
                uint64_t c[8];
                if (PREMAT) {
#pragma unroll
                    for (int x = 0; x < 4; x++) {
                        c[2 * x] = creg[x].x;
                        c[2 * x + 1] = creg[x].y;
                    }
                } else {
                    prg_ring_block(key, (uint32_t)(group * TC_ROWS + il), col_offset + js + jj, (uint32_t)blk, c);
                }
                const uint32_t kk = (uint32_t)(jj * D + 8 * blk);
                uint8_t* dst = A_sh + il * TC_SBO + (kk >> 4) * TC_CORE + (kk & 15);
                const int rot = (t >> 1) & 3;
#pragma unroll
                for (int b = 0; b < 8; b++) {
                    const int bp = (b & 4) | ((b + rot) & 3);
                    uint32_t w[8];
#pragma unroll
                    for (int x = 0; x < 8; x++) w[x] = b < 4 ? (uint32_t)c[x] : (uint32_t)(c[x] >> 32);
                    const uint32_t sel = (uint32_t)(bp & 3) | ((4u + (uint32_t)(bp & 3)) << 4);
                    const uint32_t lo = __byte_perm(__byte_perm(w[0], w[1], sel), __byte_perm(w[2], w[3], sel), 0x5410);
                    const uint32_t hi = __byte_perm(__byte_perm(w[4], w[5], sel), __byte_perm(w[6], w[7], sel), 0x5410);
                    *reinterpret_cast<uint2*>(dst + bp * 16) = make_uint2(lo, hi);
                }
            }
        }
        if (materialize) {
            __syncthreads();
            uint4* out = reinterpret_cast<uint4*>(materialize + ((js / TC_STAGE_COLS) * 3 + (uint64_t)group) * TCP_A_IMAGE);
            for (int piece = t; piece < (int)(TCP_A_IMAGE / 16); piece += TCP_THREADS) out[piece] = reinterpret_cast<const uint4*>(A_sh)[piece];
            __syncthreads();
            continue;
        }
        // ---- the next stage's global reads are in flight while this one is built ----
        if (sidx + 1 < n_stages) fetch(js + TC_STAGE_COLS);
        // ---- B: the 112 sliding rows of every (column, plane) of the stage; row o = window bytes o .. o + 15 ----
        for (int x = t; x < TC_STAGE_COLS * np * TC_B_ROWS; x += TCP_THREADS) {
            const int cp = x / TC_B_ROWS, o = x - cp * TC_B_ROWS;
            const uint32_t* W = reinterpret_cast<const uint32_t*>(V_sh + cp * TC_V_STRIDE) + (o >> 2);
            const int sh = 8 * (o & 3);
            const uint32_t w0 = W[0], w1 = W[1], w2 = W[2], w3 = W[3], w4 = W[4];
            *reinterpret_cast<uint4*>(B_sh + (size_t)cp * TC_B_IMAGE + 16 * o) =
                make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh),
                           __funnelshift_r(w3, w4, sh));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (t == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;");
            const uint32_t a_addr = smem_u32(A_sh), b_addr = smem_u32(B_sh);
            // the descriptors advance by adding to their address field (bytes / 16, no carry out of its 14 bits)
            const uint64_t da0 = umma_desc(a_addr, TC_CORE, TC_SBO);
            // B: K blocks 256 bytes apart, row groups 128 bytes apart (overlapping core matrices, see the header)
            const uint64_t db0 = umma_desc(b_addr, 2 * TC_CORE, TC_CORE);
#pragma unroll
            for (int ks = 0; ks < TC_STAGE_K / 32; ks++) {
                const uint64_t da = da0 + (uint64_t)(ks * 2 * TC_CORE / 16);
                const int jj = ks >> 1, h = ks & 1;   // column of the stage, half of its 64 coefficients
#pragma unroll
                for (int p = 0; p < np; p++) {
                    const uint64_t db = db0 + (uint64_t)(((jj * np + p) * TC_B_IMAGE + h * 4 * TC_CORE) / 16);
                    const uint32_t acc = (sidx == 0 && ks == 0) ? 0u : 1u;
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                                 ::"r"(tmem + (uint32_t)(64 * p)), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mbar[buf])) : "memory");
        }
    }
    // ---- the last commit covers every MMA issued before it ----
    if (!failed && n_stages > 0 && !materialize) {
        const int last = n_stages - 1;
        if (!mbar_wait(smem_u32(&mbar[last & 1]), (uint32_t)((last >> 1) & 1))) failed = true;
    }
    if (__syncthreads_or(failed)) failed = true;
    asm volatile("tcgen05.fence::after_thread_sync;");

    if (!failed && n_stages > 0 && !materialize) {
        const int q = warp & 3, part = warp >> 2;   // four warps per quarter of the columns
        const int m = 32 * q + lane, b = m & 7, il = m >> 3;
        const uint64_t scale = 1ULL << (8 * b);
        const int c_lo = part * (n_cols / 4), c_hi = c_lo + n_cols / 4;
        for (int c0 = c_lo; c0 < c_hi; c0 += 8) {
            uint32_t v[8];
            const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)c0;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                         : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int32_t sv = (int32_t)v[e];
                uint64_t f = sv >= 0 ? (uint64_t)sv : agl::P - (uint64_t)(-(int64_t)sv);
                f = agl::mul(f, scale);
#pragma unroll
                for (int off = 1; off < 8; off <<= 1) f = agl::add(f, __shfl_xor_sync(0xffffffffu, f, off));
                if (b == 0 && il < TC_ROWS) {
                    const int n = c0 + e, p = n >> 6, r = 63 - (n & 63);   // the rows of B run in reverse
                    partial[(((size_t)blockIdx.x * 3 + group) * np + p) * (TC_ROWS * D) + il * D + r] = agl::canon(f);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols));
    if (failed && t == 0) atomicMax(d_error, (int)TC_ERR_TIMEOUT);
    if (bad_digit) atomicMax(d_error, (int)TC_ERR_DIGIT_RANGE);
}

// ---- the commit kernel: builder warps and an issuing warp ------------------------------------------------
// Fifteen warps build operands, the sixteenth issues MMAs; they meet only at mbarriers, so a builder never
// waits for the issue of a stage and the issuer never waits for a block-wide barrier.
// A stage uses buffer b = s mod WS_NB (three buffers: the round trip builder -> issuer -> tensor pipe -> builder
// is longer than a stage, two buffers left the pipe waiting).
//   full[b]   (count 15)  every builder warp has finished buffer b of this stage (lane 0 arrives after a
//                         proxy fence and a warp barrier)
//   empty[b]  (count 1)   the MMAs that read buffer b have completed (tcgen05.commit)
//   tma[q]    (tiled)     the 28 KB image of stage s has landed in slot q = s mod ws_a_slots(NP) of the A ring
// Work needs no other synchronisation: a (column, plane) pair's digits are fetched (asynchronous copies into a
// ring, three stages ahead), reversed and expanded into its rows of B by one warp (pair w of the stage, and
// w + the number of builder warps where there are more pairs than warps), and every matrix job (one ChaCha8
// block or eight coefficients -> one 8 x 8 byte tile of A) belongs to one thread.
// B is the overlapping sliding-row image described at the top of this file (1792 bytes per pair), with the
// planes of a column interleaved by core matrix: row group o / 8 of plane p sits at group (o / 8) np + p of the
// column's image. With a row-group stride of 128 bytes and a K-block stride of 256 np bytes one descriptor then
// walks all planes (MMA column 8 (g' np + p) + i = row 8 g' + i of plane p), so a K step is ONE MMA of
// N = 64 np instead of np MMAs of N = 64. That matters because an i8 MMA of M = 128, K = 32 occupies the tensor
// pipe for about 90 cycles whatever its width up to N = 128 (and 136 cycles at N = 256): per-plane MMAs cap the
// kernel at 37 % of the pipe's rate.
// The small B leaves room for a deeper ring of A images, which is what the copies from HBM need.
// TILED: the A image is not touched by threads at all: thread 0 issues one bulk copy per stage into a ring of
// ws_a_slots(NP) slots, ws_a_slots(NP) - 2 stages ahead of the builders (the copy issued at stage s reuses the
// slot of stage s - 2, whose MMAs the thread has just seen complete); rows 112..127 of the M = 128 operand are whatever follows the slot in shared
// memory: they only feed accumulator rows that nobody reads.
// Every wait is bounded; a warp that gives up records TC_ERR_TIMEOUT and leaves the loop, the others then run
// out of their own waits, and all threads meet at the barrier before the epilogue.
// Warps: 15 builders and the issuer (512 threads) when threads generate or split the matrix (the ChaCha8 build
// needs 120 registers). Tiled source: 16 builders (one (column, plane) pair each at four planes: with 15 the warp
// that owned two pairs set the pace of every stage), the issuer, and a warp whose first lane issues the bulk
// copies of the A images into their own ring, as far ahead as the ring is deep (the issuer commits every stage
// to the B buffer's barrier and to the A slot's).
__host__ __device__ constexpr int ws_build_warps(int src) { return src == TC_SRC_TILED ? 16 : 15; }
__host__ __device__ constexpr int ws_threads(int src) { return src == TC_SRC_TILED ? 576 : 512; }
constexpr int WS_NB = 3;                             // operand buffers in flight (a round trip builder -> issuer ->
                                                     // tensor pipe -> builder takes about two stage times)
constexpr int WS_A_SLOTS_MAX = 6;
constexpr int WS_DIGIT_DEPTH = 4;                    // ring of digit stages: copies run three stages ahead
__host__ __device__ constexpr int ws_nb(int src) { return src == TC_SRC_TILED ? 2 : WS_NB; }   // tiled: room for the A ring
__host__ __device__ constexpr int ws_a_slots(int np) { return np <= 3 ? 6 : 5; }

template <int SRC, int NP>
static __global__ void __launch_bounds__(ws_threads(SRC), 1)
commit_tc_ws_kernel(const uint32_t* __restrict__ d_key, const uint64_t* __restrict__ d_M, const uint8_t* __restrict__ d_T,
                    const int8_t* __restrict__ d_digits, uint64_t N, int p0, uint64_t col_offset, uint64_t* __restrict__ partial,
                    int* __restrict__ d_error, int chunk_cols) {
    constexpr int np = NP;
    constexpr bool TILED = SRC == TC_SRC_TILED, PREMAT = SRC == TC_SRC_COEFFS;
    constexpr int PAIRS = TC_STAGE_COLS * np;                       // (column, plane) pairs per stage
    constexpr int WS_BUILD_WARPS = ws_build_warps(SRC), WS_THREADS = ws_threads(SRC);
    constexpr int PAIRS_PER_WARP = (PAIRS + WS_BUILD_WARPS - 1) / WS_BUILD_WARPS;
    constexpr uint32_t A_SLOT = TILED ? TCP_A_IMAGE : TC_A_BYTES;
    constexpr int NB = ws_nb(SRC);
    constexpr int A_SLOTS = TILED ? ws_a_slots(NP) : NB;
    constexpr uint32_t B_BYTES = PAIRS * TC_B_IMAGE;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* A_base = smem;
    uint8_t* B_base = smem + A_SLOTS * A_SLOT;
    uint8_t* DG_base = B_base + NB * B_BYTES;                        // WS_DIGIT_DEPTH stages of digits, 64 bytes per pair
    __shared__ __align__(8) uint64_t bar_full[WS_NB], bar_empty[WS_NB], bar_tma[WS_A_SLOTS_MAX], bar_afree[WS_A_SLOTS_MAX];
    __shared__ uint32_t tmem_base_sh;

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int group = blockIdx.y;
    const int n_cols = 64 * np;
    const uint64_t j0 = (uint64_t)blockIdx.x * (uint64_t)chunk_cols;
    const uint64_t j1 = j0 + (uint64_t)chunk_cols < N ? j0 + (uint64_t)chunk_cols : N;
    const int n_stages = (int)((j1 - j0 + TC_STAGE_COLS - 1) / TC_STAGE_COLS);
    const uint32_t tmem_cols = 256u;

    if (!TILED) {   // rows 112..127 of the A buffers stay zero
        for (int b = 0; b < NB; b++)
            for (int x = t; x < (int)(2 * TC_SBO / 16); x += WS_THREADS)
                reinterpret_cast<uint4*>(A_base + b * A_SLOT + 14 * TC_SBO)[x] = make_uint4(0, 0, 0, 0);
    }
    if (t == 0) {
        for (int b = 0; b < NB; b++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar_full[b])), "r"(WS_BUILD_WARPS));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_empty[b])));
        }
        for (int q = 0; q < WS_A_SLOTS_MAX; q++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_tma[q])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_afree[q])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;");
    const uint32_t tmem = tmem_base_sh;
    bool failed = false;
    int bad_digit = 0;
    int copies_issued = 0;   // copy warp: stages whose bulk copy has gone out

    auto tma_issue = [&](int stage) {   // one thread: the A image of `stage` into its ring slot
        const uint32_t bar = smem_u32(&bar_tma[stage % A_SLOTS]);
        const uint32_t dst = smem_u32(A_base + (stage % A_SLOTS) * A_SLOT);
        const uint8_t* src = d_T + (((j0 / TC_STAGE_COLS) + (uint64_t)stage) * 3 + (uint64_t)group) * TCP_A_IMAGE;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)TCP_A_IMAGE) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(src), "r"((uint32_t)TCP_A_IMAGE), "r"(bar) : "memory");
    };

    if (warp < WS_BUILD_WARPS) {
        // ================= builders =================
        uint32_t key[8];
#pragma unroll
        for (int k = 0; k < 8; k++) key[k] = SRC == TC_SRC_CHACHA ? d_key[k] : 0u;
        constexpr int JOBS = TC_STAGE_COLS * TC_ROWS * 8;   // 448 matrix jobs per stage, one per thread
        ulonglong2 creg[4];
        // The digits of stage `stage` go into slot stage mod WS_DIGIT_DEPTH of a ring in shared memory by
        // asynchronous copies (16 bytes per lane, four lanes per pair), WS_DIGIT_DEPTH - 1 stages ahead of their
        // use: a global load consumed one stage later leaves every stage waiting for a full memory latency.
        // One group is committed per stage, empty or not, so that the group count says which stage has landed.
        auto fetch_digits = [&](int stage) {
            const uint64_t js = j0 + (uint64_t)stage * TC_STAGE_COLS;
            uint8_t* slot = DG_base + (stage % WS_DIGIT_DEPTH) * (PAIRS * D);
#pragma unroll
            for (int q = 0; q < PAIRS_PER_WARP; q++) {
                const int cp = warp + WS_BUILD_WARPS * q;
                if (cp < PAIRS && lane < 4) {
                    const int jj = cp / np, p = cp % np;
                    const bool on = stage < n_stages && js + jj < j1;
                    const int8_t* src = d_digits + ((size_t)(p0 + p) * N + (on ? js + jj : j0)) * D + 16 * lane;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                                 ::"r"(smem_u32(slot + cp * D + 16 * lane)), "l"(src), "r"(on ? 16 : 0) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto fetch = [&](uint64_t js) {
            if (PREMAT) {
                const int jj = t / (TC_ROWS * 8), rem = t % (TC_ROWS * 8), il = rem >> 3, blk = rem & 7;
                const bool on = t < JOBS && js + jj < j1;
                const ulonglong2* src = reinterpret_cast<const ulonglong2*>(
                    d_M + ((js + jj) * (uint64_t)KAPPA + (uint64_t)(group * TC_ROWS + il)) * D + 8 * blk);
#pragma unroll
                for (int x = 0; x < 4; x++) creg[x] = on ? __ldcs(src + x) : make_ulonglong2(0, 0);
            }
        };
        if (n_stages > 0) fetch(j0);
        for (int st = 0; st < WS_DIGIT_DEPTH - 1; st++) fetch_digits(st);
        // this thread's matrix job has the same row and block in every stage: the quarter rounds of the first
        // column round that do not see the column index are computed once
        ChaChaColumns cols_pre;
        cols_pre.n2 = 0;
        if (SRC == TC_SRC_CHACHA && t < JOBS) {
            const int rem = t % (TC_ROWS * 8);
            chacha8_columns(key, (uint32_t)(rem & 7), (uint32_t)(group * TC_ROWS + (rem >> 3)), (uint32_t)((col_offset + j0) >> 32), cols_pre);
        }
        for (int sidx = 0; sidx < n_stages; sidx++) {
            const uint64_t js = j0 + (uint64_t)sidx * TC_STAGE_COLS;
            const int buf = sidx % NB, use = sidx / NB;   // buffer and how many times it has been used before
            uint8_t* A_sh = A_base + buf * A_SLOT;     // not used when TILED
            uint8_t* B_sh = B_base + buf * B_BYTES;
            // the MMAs that last read this buffer (stage sidx - NB) must be done before it is rewritten
            if (sidx >= NB) {
                uint32_t ok = 1;
                if (lane == 0) ok = mbar_wait(smem_u32(&bar_empty[buf]), (uint32_t)((use - 1) & 1)) ? 1u : 0u;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { failed = true; break; }
            }
            // the copies of stage sidx + WS_DIGIT_DEPTH - 1 go out (their slot held stage sidx - 1, which this warp
            // read before its last barrier); all but the newest WS_DIGIT_DEPTH - 1 groups have then landed
            fetch_digits(sidx + WS_DIGIT_DEPTH - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(WS_DIGIT_DEPTH - 1) : "memory");
            __syncwarp();
            // A: byte planes of this thread's eight coefficients
            if (!TILED && t < JOBS) {
                const int jj = t / (TC_ROWS * 8), rem = t % (TC_ROWS * 8), il = rem >> 3, blk = rem & 7;
                uint64_t c[8];
                if (PREMAT) {
#pragma unroll
                    for (int x = 0; x < 4; x++) {
                        c[2 * x] = creg[x].x;
                        c[2 * x + 1] = creg[x].y;
                    }
                } else {
                    prg_ring_block_pre(key, cols_pre, (uint32_t)(group * TC_ROWS + il), col_offset + js + jj, (uint32_t)blk, c);
                }
                const uint32_t kk = (uint32_t)(jj * D + 8 * blk);
                uint8_t* dst = A_sh + il * TC_SBO + (kk >> 4) * TC_CORE + (kk & 15);
                const int rot = (t >> 1) & 3;
#pragma unroll
                for (int b = 0; b < 8; b++) {
                    const int bp = (b & 4) | ((b + rot) & 3);
                    uint32_t w[8];
#pragma unroll
                    for (int x = 0; x < 8; x++) w[x] = b < 4 ? (uint32_t)c[x] : (uint32_t)(c[x] >> 32);
                    const uint32_t sel = (uint32_t)(bp & 3) | ((4u + (uint32_t)(bp & 3)) << 4);
                    const uint32_t lo = __byte_perm(__byte_perm(w[0], w[1], sel), __byte_perm(w[2], w[3], sel), 0x5410);
                    const uint32_t hi = __byte_perm(__byte_perm(w[4], w[5], sel), __byte_perm(w[6], w[7], sel), 0x5410);
                    *reinterpret_cast<uint2*>(dst + bp * 16) = make_uint2(lo, hi);
                }
            }
            // B: the 112 sliding rows of this warp's pairs, straight from the digits. The reversed, sign-wrapped
            // window of a pair has words W[i] = reverse(Z[15 - i]) for i < 16 and -reverse(Z[31 - i]) for i >= 16
            // (Z the 16 digit words); lane l < 28 reads W[l .. l + 4] and forms rows 4 l .. 4 l + 3 (byte offsets
            // 0 .. 3 into the same five words). The four stores of a lane go out rotated by l / 2, so that the
            // lanes of one store instruction cover eight different 16-byte slots of the banks.
#pragma unroll
            for (int q = 0; q < PAIRS_PER_WARP; q++) {
                const int cp = warp + WS_BUILD_WARPS * q;
                if (cp < PAIRS && lane < 28) {
                    const uint32_t* Z = reinterpret_cast<const uint32_t*>(DG_base + (sidx % WS_DIGIT_DEPTH) * (PAIRS * D) + cp * D);
                    uint32_t w[5];
#pragma unroll
                    for (int x = 0; x < 5; x++) {
                        const int i = lane + x;
                        const uint32_t z = Z[i < 16 ? 15 - i : 31 - i];
                        if (x == 0 && lane < 16 &&
                            (((z & 0xffu) == 0x80u) | ((z & 0xff00u) == 0x8000u) | ((z & 0xff0000u) == 0x800000u) | ((z >> 24) == 0x80u)))
                            bad_digit = 1;
                        const uint32_t rev = __byte_perm(z, 0, 0x0123);
                        w[x] = i < 16 ? rev : __vneg4(rev);
                    }
                    // row o of plane p goes to row group (o / 8) * np + p of the column's image: the planes are
                    // interleaved by core matrix, so that one descriptor walks all of them
                    const int jj = cp / np, p = cp - jj * np;
                    uint8_t* dst = B_sh + (size_t)jj * (np * TC_B_IMAGE) + p * TC_CORE + (lane >> 1) * (np * TC_CORE) + (lane & 1) * 64;
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int kk = (k + (lane >> 1)) & 3, sh = 8 * kk;
                        *reinterpret_cast<uint4*>(dst + 16 * kk) =
                            make_uint4(__funnelshift_r(w[0], w[1], sh), __funnelshift_r(w[1], w[2], sh), __funnelshift_r(w[2], w[3], sh),
                                       __funnelshift_r(w[3], w[4], sh));
                    }
                }
            }
            // next stage's global reads go out before this warp reports the stage
            if (sidx + 1 < n_stages) fetch(js + TC_STAGE_COLS);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_full[buf])) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this warp is still in flight when it leaves
    } else if (warp == WS_BUILD_WARPS + 1) {
        // ================= copies of the A images (tiled source) =================
        if (TILED && lane == 0) {
            for (int st = 0; st < n_stages; st++) {
                // the slot held stage st - A_SLOTS; its MMAs are done when the issuer's commit to the slot's barrier lands
                if (st >= A_SLOTS && !mbar_wait(smem_u32(&bar_afree[st % A_SLOTS]), (uint32_t)((st / A_SLOTS - 1) & 1))) { failed = true; break; }
                tma_issue(st);
                copies_issued = st + 1;
            }
        }
    } else if (lane == 0) {
        // ================= issuer =================
        const uint32_t idesc = umma_idesc_i8(64 * np);   // all planes in one MMA
        for (int sidx = 0; sidx < n_stages; sidx++) {
            const int buf = sidx % NB;
            if (!mbar_wait(smem_u32(&bar_full[buf]), (uint32_t)((sidx / NB) & 1))) { failed = true; break; }
            if (TILED && !mbar_wait(smem_u32(&bar_tma[sidx % A_SLOTS]), (uint32_t)((sidx / A_SLOTS) & 1))) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;");
            const uint32_t a_addr = smem_u32(A_base + (TILED ? (sidx % A_SLOTS) : buf) * A_SLOT);
            const uint32_t b_addr = smem_u32(B_base + buf * B_BYTES);
            // the descriptors advance by adding to their address field (bytes / 16, no carry out of its 14 bits)
            const uint64_t da0 = umma_desc(a_addr, TC_CORE, TC_SBO);
            // B: MMA column n = 8 g + i is row 8 g' + i of plane p with g = g' np + p; row groups 128 bytes apart,
            // K blocks 256 np bytes apart: core matrix (g, c) of the K step at 512 np s is group g' + 2 c + 4 s of plane p
            const uint64_t db0 = umma_desc(b_addr, 2 * TC_CORE * np, TC_CORE);
#pragma unroll
            for (int ks = 0; ks < TC_STAGE_K / 32; ks++) {
                const uint64_t da = da0 + (uint64_t)(ks * 2 * TC_CORE / 16);
                const int jj = ks >> 1, h = ks & 1;   // column of the stage, half of its 64 coefficients
                const uint64_t db = db0 + (uint64_t)((jj * np * TC_B_IMAGE + h * 4 * TC_CORE * np) / 16);
                const uint32_t acc = (sidx == 0 && ks == 0) ? 0u : 1u;
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                             ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar_empty[buf])) : "memory");
            if (TILED)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                             ::"r"(smem_u32(&bar_afree[sidx % A_SLOTS])) : "memory");
        }
        // the last commit covers every MMA issued before it
        if (!failed && n_stages > 0) {
            const int last = n_stages - 1;
            if (!mbar_wait(smem_u32(&bar_empty[last % NB]), (uint32_t)((last / NB) & 1))) failed = true;
        }
    }
    if (__syncthreads_or(failed)) failed = true;
    if (TILED && failed && warp == WS_BUILD_WARPS + 1 && lane == 0) {
        // a wait gave up somewhere: no copy of this CTA may still be in flight when it leaves (bounded waits again;
        // a landed copy's phase is complete whether or not the issuer consumed it)
        for (int st = copies_issued > A_SLOTS ? copies_issued - A_SLOTS : 0; st < copies_issued; st++)
            mbar_wait(smem_u32(&bar_tma[st % A_SLOTS]), (uint32_t)((st / A_SLOTS) & 1));
    }
    asm volatile("tcgen05.fence::after_thread_sync;");

    if (!failed && n_stages > 0 && warp < 16) {
        // Accumulator row m = 8 il + b holds byte plane b of matrix row il; a warp reads 32 rows (four values of
        // il) and a sixteenth of the columns at a time. c = sum_b 2^(8 b) D[(il, b)] exceeds 64 bits, so planes
        // 0..3 are summed into L and planes 4..7 into H as plain 64-bit integers (|.| < 2^57) and c = L + 2^32 H
        // is reduced once. The eight lanes of an il share the work: each shuffle round halves the columns a lane
        // keeps (a lane sends the half its partner keeps), so after three rounds every lane owns one of the
        // eight columns, summed over the planes.
        const int q = warp & 3, part = warp >> 2;   // four warps per quarter of the columns
        const int m = 32 * q + lane, b = m & 7, il = m >> 3;
        const bool b0 = b & 1, b1 = b & 2, b2 = b & 4;
        const int sh = 8 * (b & 3), e_own = 4 * (b & 1) + (b & 2) + (b >> 2);
        const int c_lo = part * (n_cols / 4), c_hi = c_lo + n_cols / 4;
        for (int c0 = c_lo; c0 < c_hi; c0 += 8) {
            uint32_t v[8];
            const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)c0;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                         : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            long long u[4], w2[2];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const long long lo = (long long)(int32_t)v[i] << sh, hi = (long long)(int32_t)v[i + 4] << sh;
                u[i] = (b0 ? hi : lo) + __shfl_xor_sync(0xffffffffu, b0 ? lo : hi, 1);       // column 4 b0 + i
            }
#pragma unroll
            for (int i = 0; i < 2; i++)
                w2[i] = (b1 ? u[i + 2] : u[i]) + __shfl_xor_sync(0xffffffffu, b1 ? u[i] : u[i + 2], 2);   // column 4 b0 + 2 b1 + i
            const long long mine = b2 ? w2[1] : w2[0];
            const long long other = __shfl_xor_sync(0xffffffffu, b2 ? w2[0] : w2[1], 4);
            const long long L = b2 ? other : mine, H = b2 ? mine : other;
            const uint64_t fl = L >= 0 ? (uint64_t)L : agl::P - (uint64_t)(-L);
            const uint64_t fh = H >= 0 ? (uint64_t)H : agl::P - (uint64_t)(-H);
            const uint64_t f = agl::add(fl, agl::reduce128(fh << 32, fh >> 32));
            if (il < TC_ROWS) {
                // column c0 + e: row group g = c0 / 8 = g' np + p, row 8 g' + e of plane p; the rows of B run in reverse
                const int g = c0 >> 3, gp = g / np, p = g - gp * np, r = 63 - (8 * gp + e_own);
                partial[(((size_t)blockIdx.x * 3 + group) * np + p) * (TC_ROWS * D) + il * D + r] = agl::canon(f);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols));
    if (failed && lane == 0) atomicMax(d_error, (int)TC_ERR_TIMEOUT);
    if (bad_digit) atomicMax(d_error, (int)TC_ERR_DIGIT_RANGE);
}

inline size_t tc_ws_smem_bytes(int src, int np) {
    const size_t pairs = (size_t)TC_STAGE_COLS * np;
    const size_t a = src == TC_SRC_TILED ? (size_t)ws_a_slots(np) * TCP_A_IMAGE : (size_t)WS_NB * TC_A_BYTES;
    const size_t nb = (size_t)ws_nb(src);
    // the tiled ring's last slot is read 4 KB past its image (rows 112..127 of the operand): B follows it
    return a + nb * pairs * TC_B_IMAGE + (size_t)WS_DIGIT_DEPTH * pairs * D + 4096;
}

// ---- sustained int8 rate of the tensor pipe, measured with this file's own issue loop -------------------
// One CTA per SM; the operands (A: 128 rows, B: 256 columns, K = 256 bytes, pseudo-random bytes, ordinary
// non-overlapping core-matrix layout) stay in shared memory; one thread issues `groups` times eight K = 32 MMAs
// of M = 128, N = n_cols into the same accumulators, committing every group to one of a ring of mbarriers and
// waiting (bounded) for the group `depth` groups back, so that the pipe always has work queued. A commit's
// arrival is seen well over a thousand cycles after its MMAs were issued: with depth 1 narrow MMAs measure that
// round trip, not the pipe (16 MMAs in flight: about 89 cycles per MMA whatever the width); depth 6 keeps 56 in
// flight. No operand is built and nothing is read back: this is the ceiling the commit kernel is compared with.
constexpr int PEAK_RING = 8;
static __global__ void __launch_bounds__(128, 1)
int8_peak_kernel(int groups, int n_cols, int depth, int* __restrict__ d_error) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t mbar[PEAK_RING];
    __shared__ uint32_t tmem_base_sh;
    const int t = threadIdx.x, warp = t >> 5;
    const uint32_t b_bytes = 32 * TC_SBO;   // 256 columns
    for (uint32_t x = t; x < (TC_A_BYTES + b_bytes) / 4; x += blockDim.x) {
        uint32_t h = x * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        reinterpret_cast<uint32_t*>(smem)[x] = h;
    }
    if (t == 0) {
        for (int q = 0; q < PEAK_RING; q++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[q])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t tmem_cols = 256u;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;");
    const uint32_t tmem = tmem_base_sh;
    bool failed = false;
    if (t == 0) {
        if (depth < 1) depth = 1;
        if (depth > PEAK_RING - 1) depth = PEAK_RING - 1;
        const uint32_t idesc = umma_idesc_i8(n_cols);
        const uint64_t da0 = umma_desc(smem_u32(smem), TC_CORE, TC_SBO), db0 = umma_desc(smem_u32(smem + TC_A_BYTES), TC_CORE, TC_SBO);
        for (int gidx = 0; gidx < groups && !failed; gidx++) {
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                const uint64_t da = da0 + (uint64_t)(ks * 2 * TC_CORE / 16), db = db0 + (uint64_t)(ks * 2 * TC_CORE / 16);
                const uint32_t acc = (gidx == 0 && ks == 0) ? 0u : 1u;
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                             ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         ::"r"(smem_u32(&mbar[gidx % PEAK_RING])) : "memory");
            if (gidx >= depth) {
                const int prev = gidx - depth;
                if (!mbar_wait(smem_u32(&mbar[prev % PEAK_RING]), (uint32_t)((prev / PEAK_RING) & 1))) failed = true;
            }
        }
        // the commits complete in order: the last one covers every group
        if (!failed && groups > 0) {
            const int last = groups - 1;
            if (!mbar_wait(smem_u32(&mbar[last % PEAK_RING]), (uint32_t)((last / PEAK_RING) & 1))) failed = true;
        }
        if (failed) atomicMax(d_error, (int)TC_ERR_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols));
}

inline size_t tc_pipe_smem_bytes(int np) {
    return 2 * (TC_A_BYTES + (size_t)TC_STAGE_COLS * np * TC_B_IMAGE) + TC_STAGE_COLS * TC_MAX_PLANES * TC_V_STRIDE;
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


}  // namespace aj
}  // namespace mb
