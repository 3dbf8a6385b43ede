// Basefold kernels over Goldilocks: bit reversal, hypercube interpolation and
// the foldable-code encoder as shared-memory multi-layer passes, codeword folds,
// and the opening's inner sumcheck (eq x bh) in coefficient form.
//
// What each computes is fixed by the reference (cuda/basefold.cuh:57-205 layer
// definitions, :287-761 opening kernels; host drivers
// goldilocks-cuda-rs/cuda/wrapper.cu:1242-1500). How it is computed differs:
//  * interpolation and encoding are per-bit 2x2 maps that commute across bits,
//    so up to 12 layers run per pass over a 32 KB shared-memory tile instead of
//    one global-memory pass per layer;
//  * the encoder's repetition step copies each coefficient 2^log_rate times and
//    the butterflies never touch the copy bits, so after the bit reversal the
//    codeword is 2^log_rate equal blocks: the butterflies run once on 2^nv
//    elements and the reversal writes every block;
//  * reductions use warp shuffles and finish on the device.
// All outputs are canonical.
#pragma once
#include "sumcheck_kernels.cuh"

namespace mb {
namespace bf {

using sc::GlAdd;
using sc::GlCanon;
using sc::block_sum_store;

constexpr int BLOCK = 256;
constexpr int TILE_LOG = 12;  // 4096 u64 = 32 KB of shared memory per tile

__device__ __forceinline__ size_t bit_reverse(size_t x, int bits) {
    return bits == 0 ? 0 : (size_t)(__brevll((unsigned long long)x) >> (64 - bits));
}

// ---- bit reversal ------------------------------------------------------------
// In place, W words per element (1 = base field, 2 = extension): the reference's
// swap formulation (cuda/basefold.cuh:57-90).
template <int W>
__global__ void bit_reverse_inplace_kernel(uint64_t* __restrict__ data, int log_n) {
    const size_t n = (size_t)1 << log_n;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        size_t r = bit_reverse(i, log_n);
        if (i < r) {
#pragma unroll
            for (int w = 0; w < W; w++) {
                uint64_t a = data[i * W + w], b = data[r * W + w];
                data[i * W + w] = b;
                data[r * W + w] = a;
            }
        }
    }
}

// Out of place through a 64 x 64 shared-memory tile so that both the reads and
// the writes are 512-byte runs: out[c * n + rev(i)] = canon(in[i]) for every
// copy c < copies. Needs log_n >= 12.
static __global__ void __launch_bounds__(256)
bit_reverse_tiled_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, int log_n, int copies) {
    constexpr int T = 6;
    __shared__ uint64_t tile[64][65];
    const int mid_bits = log_n - 2 * T;
    const size_t n = (size_t)1 << log_n;
    const size_t num_tiles = (size_t)1 << mid_bits;
    for (size_t m = blockIdx.x; m < num_tiles; m += gridDim.x) {
        const size_t rm = bit_reverse(m, mid_bits);
        // element (h, l): index = h << (log_n - T) | m << T | l
        for (int e = threadIdx.x; e < 4096; e += blockDim.x) {
            int h = e >> T, l = e & 63;
            tile[h][l] = gl::canon(in[((size_t)h << (log_n - T)) | (m << T) | (size_t)l]);
        }
        __syncthreads();
        // rev(index) = rev(l) << (log_n - T) | rev(m) << T | rev(h); write runs over rev(h)
        for (int e = threadIdx.x; e < 4096; e += blockDim.x) {
            int rl = e >> T, rh = e & 63;
            int l = (int)(__brev((unsigned)rl) >> (32 - T)), h = (int)(__brev((unsigned)rh) >> (32 - T));
            uint64_t v = tile[h][l];
            size_t o = ((size_t)rl << (log_n - T)) | (rm << T) | (size_t)rh;
            for (int c = 0; c < copies; c++) out[(size_t)c * n + o] = v;
        }
        __syncthreads();
    }
}

// Small sizes: direct gather.
static __global__ void bit_reverse_copy_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, int log_n,
                                        int copies) {
    const size_t n = (size_t)1 << log_n;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        uint64_t v = gl::canon(in[bit_reverse(i, log_n)]);
        for (int c = 0; c < copies; c++) out[(size_t)c * n + i] = v;
    }
}

// ---- multi-layer per-bit transforms --------------------------------------------
// Interp: (a, b) -> (a, b - a)       (cuda/basefold.cuh:103-147)
// Code:   (a, b) -> (a + b, a - b)   (cuda/basefold.cuh:181-205)
struct InterpOp {
    static __device__ __forceinline__ void apply(uint64_t& a, uint64_t& b) { b = gl::sub(b, a); }
};
struct CodeOp {
    static __device__ __forceinline__ void apply(uint64_t& a, uint64_t& b) {
        uint64_t s = gl::add(a, b), d = gl::sub(a, b);
        a = s;
        b = d;
    }
};

// One pass applies Op on index bits [bit_lo, bit_lo + nbits). A tile holds
// 2^nbits rows (stride 2^bit_lo) of 2^cbits consecutive elements, nbits + cbits
// <= TILE_LOG and cbits <= bit_lo (cbits = 0 when bit_lo = 0). `in` may equal `out`.
template <class Op>
__global__ void __launch_bounds__(BLOCK)
bit_layers_kernel(const uint64_t* in, uint64_t* out, int log_n, int bit_lo, int nbits, int cbits) {
    extern __shared__ uint64_t tile[];
    const int tile_log = nbits + cbits;
    const int tile_elems = 1 << tile_log;
    const int mid_bits = bit_lo - cbits;
    const size_t num_tiles = (size_t)1 << (log_n - tile_log);
    const size_t cmask = ((size_t)1 << cbits) - 1;
    for (size_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        size_t mid = t & (((size_t)1 << mid_bits) - 1), high = t >> mid_bits;
        size_t base = (high << (bit_lo + nbits)) | (mid << cbits);
        for (int e = threadIdx.x; e < tile_elems; e += blockDim.x)
            tile[e] = in[base | ((size_t)(e >> cbits) << bit_lo) | ((size_t)e & cmask)];
        __syncthreads();
        for (int b = 0; b < nbits; b++) {
            const int sh = cbits + b;
            for (int p = threadIdx.x; p < tile_elems / 2; p += blockDim.x) {
                int low = p & ((1 << sh) - 1), hi = p >> sh;
                int i0 = (hi << (sh + 1)) | low, i1 = i0 | (1 << sh);
                uint64_t a = tile[i0], c = tile[i1];
                Op::apply(a, c);
                tile[i0] = a;
                tile[i1] = c;
            }
            __syncthreads();
        }
        for (int e = threadIdx.x; e < tile_elems; e += blockDim.x)
            out[base | ((size_t)(e >> cbits) << bit_lo) | ((size_t)e & cmask)] = gl::canon(tile[e]);
        __syncthreads();
    }
}

// ---- codeword folds: v0 + (r - x0) (v1 - v0) w ----------------------------------
// table = (point, weight) pairs. cuda/basefold.cuh:397-419 (base), :522-550
// (base codeword, extension challenge), :739-761 (extension).
static __global__ void fold_gl_kernel(const uint64_t* __restrict__ cw, const uint64_t* __restrict__ table, uint64_t r,
                               uint64_t* __restrict__ out, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        ulonglong2 v = *reinterpret_cast<const ulonglong2*>(cw + 2 * i);
        ulonglong2 e = *reinterpret_cast<const ulonglong2*>(table + 2 * i);
        uint64_t dw = gl::mul(gl::sub(v.y, v.x), e.y);
        out[i] = gl::canon(gl::add(v.x, gl::mul(gl::sub(r, e.x), dw)));
    }
}

static __global__ void fold_mixed_kernel(const uint64_t* __restrict__ cw, const uint64_t* __restrict__ table, gl::E2 r,
                                  uint64_t* __restrict__ out, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        ulonglong2 v = *reinterpret_cast<const ulonglong2*>(cw + 2 * i);
        ulonglong2 e = *reinterpret_cast<const ulonglong2*>(table + 2 * i);
        uint64_t dw = gl::mul(gl::sub(v.y, v.x), e.y);
        gl::E2 cx{gl::sub(r.c0, e.x), r.c1};
        gl::E2 res{gl::add(v.x, gl::mul(cx.c0, dw)), gl::mul(cx.c1, dw)};
        gl::e2_store(out + 2 * i, gl::e2_canon(res));
    }
}

static __global__ void fold_ext2_kernel(const uint64_t* __restrict__ cw, const uint64_t* __restrict__ table, gl::E2 r,
                                 uint64_t* __restrict__ out, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        gl::E2 v0 = gl::e2_load(cw + 4 * i), v1 = gl::e2_load(cw + 4 * i + 2);
        ulonglong2 e = *reinterpret_cast<const ulonglong2*>(table + 2 * i);
        gl::E2 dw = gl::e2_mul_base(gl::e2_sub(v1, v0), e.y);
        gl::E2 cx{gl::sub(r.c0, e.x), r.c1};
        gl::e2_store(out + 2 * i, gl::e2_canon(gl::e2_add(v0, gl::e2_mul(cx, dw))));
    }
}

// ---- inner sumcheck of the opening, coefficient form ------------------------------
// interp: (a, b) -> (a, b - a) in place (cuda/basefold.cuh:287-300, ext2 :552-565)
template <int W>
__global__ void sc_interp_kernel(uint64_t* __restrict__ data, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
#pragma unroll
        for (int w = 0; w < W; w++) {
            uint64_t a = data[2 * W * i + w], b = data[2 * W * i + W + w];
            data[2 * W * i + w] = gl::canon(a);
            data[2 * W * i + W + w] = gl::canon(gl::sub(b, a));
        }
    }
}

// eval: out[i] = c + r d for pairs (c, d) (cuda/basefold.cuh:307-321, :502-520, :567-582)
static __global__ void sc_eval_gl_kernel(const uint64_t* __restrict__ data, uint64_t r, uint64_t* __restrict__ out, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        ulonglong2 v = *reinterpret_cast<const ulonglong2*>(data + 2 * i);
        out[i] = gl::canon(gl::add(v.x, gl::mul(r, v.y)));
    }
}
static __global__ void sc_eval_mixed_kernel(const uint64_t* __restrict__ data, gl::E2 r, uint64_t* __restrict__ out, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        ulonglong2 v = *reinterpret_cast<const ulonglong2*>(data + 2 * i);
        gl::E2 res{gl::add(v.x, gl::mul(r.c0, v.y)), gl::mul(r.c1, v.y)};
        gl::e2_store(out + 2 * i, gl::e2_canon(res));
    }
}
static __global__ void sc_eval_ext2_kernel(const uint64_t* __restrict__ data, gl::E2 r, uint64_t* __restrict__ out, size_t pairs) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        gl::E2 c = gl::e2_load(data + 4 * i), d = gl::e2_load(data + 4 * i + 2);
        gl::e2_store(out + 2 * i, gl::e2_canon(gl::e2_add(c, gl::e2_mul(r, d))));
    }
}

// Block partials land in three separate arrays indexed by block, as the
// reference's callers expect (goldilocks-cuda-rs/src/basefold.rs:616-622).
template <int W>
__device__ __forceinline__ void store_c012(uint64_t (&v)[3 * W], uint64_t* p0, uint64_t* p1, uint64_t* p2) {
    __shared__ uint64_t res[3 * W];
    block_sum_store<3 * W>(v, res, GlAdd(), GlCanon());
    __syncthreads();
    if (threadIdx.x < W) {
        p0[(size_t)blockIdx.x * W + threadIdx.x] = res[threadIdx.x];
        p1[(size_t)blockIdx.x * W + threadIdx.x] = res[W + threadIdx.x];
        p2[(size_t)blockIdx.x * W + threadIdx.x] = res[2 * W + threadIdx.x];
    }
}

// product over data already in (even, odd = difference) form:
// c0 = sum e_e b_e, c1 = sum (e_e b_o + e_o b_e), c2 = sum e_o b_o
static __global__ void __launch_bounds__(BLOCK)
sc_product_gl_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ bh, uint64_t* p0, uint64_t* p1,
                     uint64_t* p2, size_t pairs) {
    uint64_t v[3] = {0, 0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        ulonglong2 e = *reinterpret_cast<const ulonglong2*>(eq + 2 * i);
        ulonglong2 b = *reinterpret_cast<const ulonglong2*>(bh + 2 * i);
        v[0] = gl::add(v[0], gl::mul(e.x, b.x));
        v[1] = gl::add(v[1], gl::add(gl::mul(e.x, b.y), gl::mul(e.y, b.x)));
        v[2] = gl::add(v[2], gl::mul(e.y, b.y));
    }
    store_c012<1>(v, p0, p1, p2);
}

static __global__ void __launch_bounds__(BLOCK)
sc_product_mixed_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ bh, uint64_t* p0, uint64_t* p1,
                        uint64_t* p2, size_t pairs) {
    gl::E2 a0{0, 0}, a1{0, 0}, a2{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        gl::E2 ee = gl::e2_load(eq + 4 * i), eo = gl::e2_load(eq + 4 * i + 2);
        ulonglong2 b = *reinterpret_cast<const ulonglong2*>(bh + 2 * i);
        a0 = gl::e2_add(a0, gl::e2_mul_base(ee, b.x));
        a1 = gl::e2_add(a1, gl::e2_add(gl::e2_mul_base(ee, b.y), gl::e2_mul_base(eo, b.x)));
        a2 = gl::e2_add(a2, gl::e2_mul_base(eo, b.y));
    }
    uint64_t v[6] = {a0.c0, a0.c1, a1.c0, a1.c1, a2.c0, a2.c1};
    store_c012<2>(v, p0, p1, p2);
}

static __global__ void __launch_bounds__(BLOCK)
sc_product_ext2_kernel(const uint64_t* __restrict__ eq, const uint64_t* __restrict__ bh, uint64_t* p0, uint64_t* p1,
                       uint64_t* p2, size_t pairs) {
    gl::E2 a0{0, 0}, a1{0, 0}, a2{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        gl::E2 ee = gl::e2_load(eq + 4 * i), eo = gl::e2_load(eq + 4 * i + 2);
        gl::E2 be = gl::e2_load(bh + 4 * i), bo = gl::e2_load(bh + 4 * i + 2);
        a0 = gl::e2_add(a0, gl::e2_mul(ee, be));
        a1 = gl::e2_add(a1, gl::e2_add(gl::e2_mul(ee, bo), gl::e2_mul(eo, be)));
        a2 = gl::e2_add(a2, gl::e2_mul(eo, bo));
    }
    uint64_t v[6] = {a0.c0, a0.c1, a1.c0, a1.c1, a2.c0, a2.c1};
    store_c012<2>(v, p0, p1, p2);
}

// Fused round (cuda/basefold.cuh:654-735): inputs in (value, difference) form,
// 4 per output pair; evaluates both tables at r, rewrites them in (value,
// difference) form and accumulates the next (c0, c1, c2).
static __global__ void __launch_bounds__(BLOCK)
sc_fused_round_ext2_kernel(const uint64_t* __restrict__ eq_in, const uint64_t* __restrict__ bh_in, gl::E2 r,
                           uint64_t* __restrict__ eq_out, uint64_t* __restrict__ bh_out, uint64_t* p0, uint64_t* p1,
                           uint64_t* p2, size_t pairs) {
    gl::E2 a0{0, 0}, a1{0, 0}, a2{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
        const uint64_t* pe = eq_in + 8 * i;
        const uint64_t* pb = bh_in + 8 * i;
        gl::E2 ea = gl::e2_add(gl::e2_load(pe), gl::e2_mul(r, gl::e2_load(pe + 2)));
        gl::E2 eb = gl::e2_add(gl::e2_load(pe + 4), gl::e2_mul(r, gl::e2_load(pe + 6)));
        gl::E2 ba = gl::e2_add(gl::e2_load(pb), gl::e2_mul(r, gl::e2_load(pb + 2)));
        gl::E2 bb = gl::e2_add(gl::e2_load(pb + 4), gl::e2_mul(r, gl::e2_load(pb + 6)));
        gl::E2 eo = gl::e2_sub(eb, ea), bo = gl::e2_sub(bb, ba);
        a0 = gl::e2_add(a0, gl::e2_mul(ea, ba));
        a1 = gl::e2_add(a1, gl::e2_add(gl::e2_mul(ea, bo), gl::e2_mul(eo, ba)));
        a2 = gl::e2_add(a2, gl::e2_mul(eo, bo));
        gl::e2_store(eq_out + 4 * i, gl::e2_canon(ea));
        gl::e2_store(eq_out + 4 * i + 2, gl::e2_canon(eo));
        gl::e2_store(bh_out + 4 * i, gl::e2_canon(ba));
        gl::e2_store(bh_out + 4 * i + 2, gl::e2_canon(bo));
    }
    uint64_t v[6] = {a0.c0, a0.c1, a1.c0, a1.c1, a2.c0, a2.c1};
    store_c012<2>(v, p0, p1, p2);
}

// Dot products: per-block partial sums (goldilocks-cuda-rs/cuda/wrapper.cu:1533-1590).
static __global__ void __launch_bounds__(BLOCK)
dot_gl_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b, uint64_t* partial, size_t n) {
    uint64_t v[1] = {0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        v[0] = gl::add(v[0], gl::mul(a[i], b[i]));
    block_sum_store<1>(v, partial + blockIdx.x, GlAdd(), GlCanon());
}
static __global__ void __launch_bounds__(BLOCK)
dot_mixed_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b, uint64_t* partial, size_t n) {
    gl::E2 acc{0, 0};
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        acc = gl::e2_add(acc, gl::e2_mul_base(gl::e2_load(b + 2 * i), a[i]));
    uint64_t v[2] = {acc.c0, acc.c1};
    block_sum_store<2>(v, partial + 2 * (size_t)blockIdx.x, GlAdd(), GlCanon());
}

}  // namespace bf
}  // namespace mb
