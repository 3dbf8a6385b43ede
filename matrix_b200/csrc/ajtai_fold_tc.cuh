// Witness multifold on the 5th-generation tensor cores (tcgen05.mma kind::i8):
//   out[j][k] = sum_i (r_i * z_i[j])_k = sum_{(i, l)} Z[j][(i, l)] T[(i, l)][k]
// is a GEMM with exact small-integer arithmetic: Z[j][(i, l)] in {-1, 0, 1} is bit l of instance i of ring
// element j (pos - neg for ternary instances), T[(i, l)][k] = r_i[k - l] for l <= k and -r_i[k - l + 64]
// otherwise (the negacyclic Toeplitz matrix of challenge i). M = 128 ring elements per CTA, N = 64 output
// coefficients, K = 64 per instance. The reference does this with WMMA after materialising Z as bytes in
// global memory (almost-goldilocks-cuda-rs/cuda/wrapper.cu:1566-1617, cuda_almost_goldilocks/ajtai_tc.cuh:44-411);
// here the bit masks are expanded to bytes straight into shared memory, so HBM traffic stays at the packed
// masks in and 16-bit coefficients out.
//
// Per stage of eight instances (K = 512): every thread expands the masks of its ring element into the
// no-swizzle K-major core-matrix layout (8 rows x 16 bytes, cores contiguous along K), the stage's slice of
// T (prepared once per call in that layout) is copied in, one thread issues sixteen K = 32 MMAs into 64
// columns of tensor memory and commits them to an mbarrier that gates the reuse of the buffers. Every
// wait is bounded and reports through an error word.
#pragma once
#include "ajtai_tc.cuh"
#include "ajtai_fold.cuh"

namespace mb {
namespace aj {

constexpr int MF_INST = 8;                       // instances per stage
constexpr int MF_KC = MF_INST * 64;              // 512 bytes of K per stage
constexpr uint32_t MF_SBO = (MF_KC / 16) * TC_CORE;   // 4096: next 8-row group
constexpr uint32_t MF_A_BYTES = 16 * MF_SBO;     // 128 rows
constexpr uint32_t MF_B_BYTES = 8 * MF_SBO;      // 64 rows
constexpr int MF_THREADS = 128;

// kind::i8 instruction descriptor: D = s32, A = s8, B = s8, both K-major, M = 128, N = 64.
__host__ __device__ constexpr uint32_t mf_idesc() {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// T in the stage layout: Bg[stage][(k_out / 8) * MF_SBO + (kk / 16) * 128 + (k_out % 8) * 16 + kk % 16],
// kk = 64 * (i % 8) + l; zero rows for instances beyond the last.
static __global__ void multifold_prepare_b_kernel(const int8_t* __restrict__ r_all, int total, int stages, int8_t* __restrict__ Bg) {
    const size_t n = (size_t)stages * MF_B_BYTES, step = (size_t)gridDim.x * blockDim.x;
    for (size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x; x < n; x += step) {
        const int stage = (int)(x / MF_B_BYTES), off = (int)(x % MF_B_BYTES);
        const int grp = off / (int)MF_SBO, rem = off % (int)MF_SBO, kc = rem / 128, row = (rem % 128) / 16, byte = rem % 16;
        const int k_out = grp * 8 + row, kk = kc * 16 + byte, i = stage * MF_INST + kk / 64, l = kk % 64;
        Bg[x] = i < total ? (int8_t)r_at(r_all + (size_t)i * 64, k_out, l) : (int8_t)0;
    }
}

// Eight bits to eight bytes of 0 / 1.
__device__ __forceinline__ uint64_t spread8(uint32_t b) {
    const uint64_t x = ((uint64_t)b * 0x0101010101010101ULL) & 0x8040201008040201ULL;
    return ((x + 0x7F7F7F7F7F7F7F7FULL) >> 7) & 0x0101010101010101ULL;
}

// grid = tiles of 128 ring elements (grid-stride); block = 128 threads; dynamic shared memory MF_A_BYTES + MF_B_BYTES.
static __global__ void __launch_bounds__(MF_THREADS)
multifold_tc_kernel(const uint64_t* __restrict__ zbin, const uint64_t* __restrict__ pos, const uint64_t* __restrict__ neg,
                    const int8_t* __restrict__ Bg, int16_t* __restrict__ out, int num_binary, int num_ternary, uint64_t N,
                    int* __restrict__ d_error) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* A_sh = smem;
    uint8_t* B_sh = smem + MF_A_BYTES;
    __shared__ __align__(8) uint64_t mbar;
    __shared__ uint32_t tmem_base_sh;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int total = num_binary + num_ternary, stages = (total + MF_INST - 1) / MF_INST;
    if (t == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar)));
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(64u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;");
    const uint32_t tmem = tmem_base_sh, bar = smem_u32(&mbar), idesc = mf_idesc();
    uint32_t phase = 0;
    bool failed = false, pending = false;
    const uint64_t tiles = (N + 127) / 128;
    // The masks of a stage (eight instances of this thread's ring element) are loaded one stage ahead, while the
    // MMAs of the stage before run: consumed at once, their latency was what the kernel waited for.
    uint64_t pm[MF_INST], mm[MF_INST];
    auto load_masks = [&](uint64_t tile_idx, int s) {
        const uint64_t j = tile_idx * 128 + t;
#pragma unroll
        for (int ii = 0; ii < MF_INST; ii++) {
            const int i = s * MF_INST + ii;
            pm[ii] = 0;
            mm[ii] = 0;
            if (tile_idx < tiles && j < N && i < total) {
                if (i < num_binary) pm[ii] = __ldcs(zbin + (uint64_t)i * N + j);
                else {
                    pm[ii] = __ldcs(pos + (uint64_t)(i - num_binary) * N + j);
                    mm[ii] = __ldcs(neg + (uint64_t)(i - num_binary) * N + j);
                }
            }
        }
    };
    if (blockIdx.x < tiles && stages > 0) load_masks(blockIdx.x, 0);
    for (uint64_t tile = blockIdx.x; tile < tiles && !failed; tile += gridDim.x) {
        for (int s = 0; s < stages && !failed; s++) {
            // the previous stage's MMAs must have read A and B before they are overwritten
            if (pending) {
                if (!mbar_wait(bar, phase)) failed = true;
                phase ^= 1;
                pending = false;
                if (__syncthreads_or(failed)) { failed = true; break; }
            }
            // ---- A: this thread's ring element, eight instances, 64 bytes each ----
#pragma unroll
            for (int ii = 0; ii < MF_INST; ii++) {
                const uint64_t p = pm[ii], m = mm[ii];
                uint8_t* dst = A_sh + (t >> 3) * MF_SBO + (ii * 4) * TC_CORE + (t & 7) * 16;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t pb = (uint32_t)(p >> (16 * q)) & 0xFFFFu, mb = (uint32_t)(m >> (16 * q)) & 0xFFFFu;
                    uint64_t lo = spread8(pb & 0xFF), hi = spread8(pb >> 8);
                    if (mb) {  // -1 bytes where the negative mask is set (the masks are disjoint)
                        lo |= spread8(mb & 0xFF) * 0xFFULL;
                        hi |= spread8(mb >> 8) * 0xFFULL;
                    }
                    *reinterpret_cast<uint4*>(dst + q * TC_CORE) =
                        make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
                }
            }
            // the next stage's masks (of this tile, or the first of this CTA's next tile) go out now
            if (s + 1 < stages) load_masks(tile, s + 1);
            else load_masks(tile + gridDim.x, 0);
            // ---- B: the stage's slice of T, already in layout ----
            {
                const uint4* src = reinterpret_cast<const uint4*>(Bg + (size_t)s * MF_B_BYTES);
                uint4* dstb = reinterpret_cast<uint4*>(B_sh);
                for (int x = t; x < (int)(MF_B_BYTES / 16); x += MF_THREADS) dstb[x] = src[x];
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if (t == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;");
                const uint32_t a_addr = smem_u32(A_sh), b_addr = smem_u32(B_sh);
#pragma unroll 1
                for (int ks = 0; ks < MF_KC / 32; ks++) {
                    const uint64_t da = umma_desc(a_addr + ks * 2 * TC_CORE, TC_CORE, MF_SBO);
                    const uint64_t db = umma_desc(b_addr + ks * 2 * TC_CORE, TC_CORE, MF_SBO);
                    const uint32_t acc = (s == 0 && ks == 0) ? 0u : 1u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
            }
            pending = true;
        }
        // ---- all MMAs of the tile done: drain 64 columns, 16-bit results, one 128-byte row per lane ----
        if (pending && !failed) {
            if (!mbar_wait(bar, phase)) failed = true;
            phase ^= 1;
            pending = false;
        }
        if (__syncthreads_or(failed)) { failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;");
        {
            const uint64_t row = tile * 128 + 32 * warp + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 8) {
                uint32_t v[8];
                const uint32_t taddr = tmem + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < N) {
                    uint4 w;
                    w.x = (v[0] & 0xFFFFu) | (v[1] << 16);
                    w.y = (v[2] & 0xFFFFu) | (v[3] << 16);
                    w.z = (v[4] & 0xFFFFu) | (v[5] << 16);
                    w.w = (v[6] & 0xFFFFu) | (v[7] << 16);
                    *reinterpret_cast<uint4*>(out + row * 64 + c0) = w;
                }
            }
        }
        // the next tile's first MMA overwrites the accumulators: every warp must have read them
        asm volatile("tcgen05.fence::before_thread_sync;");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64u));
    if (failed && t == 0) atomicMax(d_error, (int)TC_ERR_TIMEOUT);
}

}  // namespace aj
}  // namespace mb
