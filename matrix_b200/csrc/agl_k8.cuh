// K = F_q[Theta]/(Theta^8 - 3) over almost-Goldilocks, the scalar field of the
// Morpheus PIOP (zk-torch-4/src/morpheus/field8.rs:1-120; device twin
// cuda_almost_goldilocks/morpheus_auth.cuh k8_mul), and the product sumcheck
// over tables of K elements (cuda_almost_goldilocks/morpheus_piop.cuh:186-282,
// CPU zk-torch-4/src/morpheus/piop/mod.rs:785-840).
//
// An element is eight canonical words (64 bytes). Eight consecutive lanes of a
// warp work on one element, lane c holding coefficient c: loads and stores are
// one coalesced 64-byte access per element, a register holds one word instead
// of eight (six tables and seven evaluation points fit without spilling), and
// a product costs each lane eight multiply-accumulates into one exact sum:
//   (a b)_c = sum_{i <= c} a_i b_{c-i} + 3 sum_{i > c} a_i b_{c-i+8}.
// The factor 3 is applied by the sending lane (it knows i + j >= 8), so one
// shuffle per operand and step suffices. All 32 lanes of a warp take part.
#pragma once
#include "common.cuh"
#include "agl_field.cuh"

namespace mb {
namespace k8 {

constexpr int MAXTAB = 6;  // morpheus_piop.cuh:18

// Coefficient c of a * b; a, b, c as held by this lane. Loose result.
__device__ __forceinline__ uint64_t mul_lane(uint64_t a, uint64_t b, int c) {
    const uint64_t b3 = agl::mul_small(b, 3);
    gl::Acc s = gl::acc_zero();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint64_t send = (i + c >= 8) ? b3 : b;  // this lane is source j = c of step i
        const uint64_t ai = __shfl_sync(0xffffffffu, a, i, 8);
        const uint64_t bj = __shfl_sync(0xffffffffu, send, (c - i) & 7, 8);
        gl::acc_mul(s, ai, bj);
    }
    return agl::acc_reduce(s);
}

// A factor every lane holds whole (a challenge), with its triple.
struct Uniform {
    uint64_t r[8], r3[8];
};
__device__ __forceinline__ Uniform make_uniform(const uint64_t* r) {
    Uniform u;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        u.r[i] = agl::canon(r[i]);
        u.r3[i] = agl::mul_small(u.r[i], 3);
    }
    return u;
}
// Coefficient c of u * d, plus `addend` (this lane's coefficient of it).
__device__ __forceinline__ uint64_t fma_uniform_lane(const Uniform& u, uint64_t d, uint64_t addend, int c) {
    gl::Acc s = gl::acc_from(addend);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint64_t dj = __shfl_sync(0xffffffffu, d, (c - i) & 7, 8);
        gl::acc_mul(s, i > c ? u.r3[i] : u.r[i], dj);
    }
    return agl::acc_reduce(s);
}

struct Tabs {
    const uint64_t* t[MAXTAB];
    int ntab;
};
struct OutTabs {
    uint64_t* t[MAXTAB];
};
struct Elem {
    uint64_t c[8];
};

// s[t] += prod_j (vals[j] + t diffs[j]) for t = 0..d (this lane's coefficient); consumes vals.
__device__ __forceinline__ void accumulate(uint64_t (&vals)[MAXTAB], const uint64_t (&diffs)[MAXTAB], int ntab, int d,
                                           uint64_t (&s)[MAXTAB + 1], int c) {
#pragma unroll
    for (int t = 0; t <= MAXTAB; t++) {
        if (t > d) break;
        if (t > 0) {
#pragma unroll
            for (int j = 0; j < MAXTAB; j++)
                if (j < ntab) vals[j] = agl::add(vals[j], diffs[j]);
        }
        uint64_t p = vals[0];
#pragma unroll
        for (int j = 1; j < MAXTAB; j++)
            if (j < ntab) p = mul_lane(p, vals[j], c);
        s[t] = agl::add(s[t], p);
    }
}

// Sum over the element groups of the block, then the last block sums the block
// rows: out[(d + 1) * 8] canonical words. partial: [gridDim.x][MAXTAB + 1][8].
__device__ __forceinline__ void finish_sums(uint64_t (&s)[MAXTAB + 1], int d, int c, uint64_t* partial, unsigned int* counter,
                                            uint64_t* out) {
    __shared__ uint64_t red[8][MAXTAB + 1][8];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int t = 0; t <= MAXTAB; t++) {
        s[t] = agl::add(s[t], __shfl_xor_sync(0xffffffffu, s[t], 8));
        s[t] = agl::add(s[t], __shfl_xor_sync(0xffffffffu, s[t], 16));
        if (lane < 8) red[warp][t][lane] = s[t];
    }
    __syncthreads();
    const int nv = (MAXTAB + 1) * 8;
    if ((int)threadIdx.x < nv) {
        const int t = threadIdx.x >> 3, cc = threadIdx.x & 7;
        uint64_t v = 0;
        for (int w = 0; w < nwarp; w++) v = agl::add(v, red[w][t][cc]);
        partial[(size_t)blockIdx.x * nv + threadIdx.x] = agl::canon(v);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if ((int)threadIdx.x < (d + 1) * 8) {
        uint64_t v = 0;
        for (unsigned int b = 0; b < gridDim.x; b++) v = agl::add(v, __ldcg(partial + (size_t)b * nv + threadIdx.x));
        out[threadIdx.x] = agl::canon(v);
    }
    if (threadIdx.x == 0) *counter = 0;
    (void)c;
}

// Round sums s[t] = sum_k prod_j (T_j[2k] + t (T_j[2k+1] - T_j[2k])), t = 0..d.
static __global__ void __launch_bounds__(256)
sc_round_kernel(Tabs T, uint64_t npairs, int d, uint64_t* partial, unsigned int* counter, uint64_t* out) {
    const int c = threadIdx.x & 7;
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (npairs + groups - 1) / groups;
    uint64_t k = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    uint64_t s[MAXTAB + 1];
#pragma unroll
    for (int t = 0; t <= MAXTAB; t++) s[t] = 0;
    for (uint64_t it = 0; it < rounds; it++, k += groups) {
        const bool live = k < npairs;
        uint64_t vals[MAXTAB], diffs[MAXTAB];
#pragma unroll
        for (int j = 0; j < MAXTAB; j++) {
            vals[j] = diffs[j] = 0;
            if (j < T.ntab && live) {
                const uint64_t lo = T.t[j][16 * k + c], hi = T.t[j][16 * k + 8 + c];
                vals[j] = agl::canon(lo);
                diffs[j] = agl::sub(hi, lo);
            }
        }
        accumulate(vals, diffs, T.ntab, d, s, c);
    }
    finish_sums(s, d, c, partial, counter, out);
}

// out[k] = in[2k] + r (in[2k+1] - in[2k]).
static __global__ void __launch_bounds__(256)
sc_fold_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, uint64_t nout, Elem r) {
    const int c = threadIdx.x & 7;
    const Uniform u = make_uniform(r.c);
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (nout + groups - 1) / groups;
    uint64_t k = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    for (uint64_t it = 0; it < rounds; it++, k += groups) {
        const bool live = k < nout;
        const uint64_t lo = live ? in[16 * k + c] : 0, hi = live ? in[16 * k + 8 + c] : 0;
        const uint64_t f = fma_uniform_lane(u, agl::sub(hi, lo), lo, c);
        if (live) out[8 * k + c] = agl::canon(f);
    }
}

// Fold every table on r into O and return the sums of the next round (over the folded tables).
static __global__ void __launch_bounds__(256)
sc_fold_round_kernel(Tabs T, OutTabs O, uint64_t nquads, Elem r, int d, uint64_t* partial, unsigned int* counter,
                     uint64_t* out) {
    const int c = threadIdx.x & 7;
    const Uniform u = make_uniform(r.c);
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (nquads + groups - 1) / groups;
    uint64_t k = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    uint64_t s[MAXTAB + 1];
#pragma unroll
    for (int t = 0; t <= MAXTAB; t++) s[t] = 0;
    for (uint64_t it = 0; it < rounds; it++, k += groups) {
        const bool live = k < nquads;
        uint64_t vals[MAXTAB], diffs[MAXTAB];
#pragma unroll
        for (int j = 0; j < MAXTAB; j++) {
            vals[j] = diffs[j] = 0;
            if (j < T.ntab) {
                uint64_t x0 = 0, x1 = 0, x2 = 0, x3 = 0;
                if (live) {
                    const uint64_t* p = T.t[j] + 32 * k + c;
                    x0 = p[0]; x1 = p[8]; x2 = p[16]; x3 = p[24];
                }
                const uint64_t f0 = agl::canon(fma_uniform_lane(u, agl::sub(x1, x0), x0, c));
                const uint64_t f1 = agl::canon(fma_uniform_lane(u, agl::sub(x3, x2), x2, c));
                if (live) {
                    O.t[j][16 * k + c] = f0;
                    O.t[j][16 * k + 8 + c] = f1;
                }
                vals[j] = f0;
                diffs[j] = agl::sub(f1, f0);
            }
        }
        accumulate(vals, diffs, T.ntab, d, s, c);
    }
    finish_sums(s, d, c, partial, counter, out);
}

// out[2i] = in[i] (1 - r), out[2i + 1] = in[i] r  (one eq doubling step; morpheus_piop.cuh:144-151)
static __global__ void __launch_bounds__(256)
eq_double_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, uint64_t half, Elem r) {
    const int c = threadIdx.x & 7;
    const Uniform u = make_uniform(r.c);
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (half + groups - 1) / groups;
    uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    for (uint64_t it = 0; it < rounds; it++, i += groups) {
        const bool live = i < half;
        const uint64_t v = live ? in[8 * i + c] : 0;
        const uint64_t vr = agl::canon(fma_uniform_lane(u, v, 0, c));
        if (live) {
            out[16 * i + c] = agl::canon(agl::sub(v, vr));
            out[16 * i + 8 + c] = vr;
        }
    }
}

// out[x] = lo[x mod 2^nlo] * hi[x >> nlo]  (morpheus_piop.cuh:153-158)
static __global__ void __launch_bounds__(256)
eq_outer_kernel(const uint64_t* __restrict__ lo, int nlo, const uint64_t* __restrict__ hi, uint64_t n, uint64_t* __restrict__ out) {
    const int c = threadIdx.x & 7;
    const uint64_t m = ((uint64_t)1 << nlo) - 1;
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (n + groups - 1) / groups;
    uint64_t x = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    for (uint64_t it = 0; it < rounds; it++, x += groups) {
        const bool live = x < n;
        const uint64_t a = live ? lo[8 * (x & m) + c] : 0, b = live ? hi[8 * (x >> nlo) + c] : 0;
        const uint64_t p = mul_lane(a, b, c);
        if (live) out[8 * x + c] = agl::canon(p);
    }
}

// out[x] += coeff * in[x]  (morpheus_piop.cuh:174-178)
static __global__ void __launch_bounds__(256)
axpy_kernel(uint64_t* out, const uint64_t* __restrict__ in, uint64_t n, Elem coeff) {
    const int c = threadIdx.x & 7;
    const Uniform u = make_uniform(coeff.c);
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (n + groups - 1) / groups;
    uint64_t x = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    for (uint64_t it = 0; it < rounds; it++, x += groups) {
        const bool live = x < n;
        const uint64_t v = live ? in[8 * x + c] : 0, o = live ? out[8 * x + c] : 0;
        const uint64_t f = fma_uniform_lane(u, v, agl::canon(o), c);
        if (live) out[8 * x + c] = agl::canon(f);
    }
}

// Base-field words to K (zero high coefficients; morpheus_piop.cuh:180-184).
static __global__ void lift_kernel(const uint64_t* __restrict__ in, uint64_t n, uint64_t* __restrict__ out) {
    const uint64_t total = n * 8, step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step)
        out[t] = (t & 7) == 0 ? agl::canon(in[t >> 3]) : 0;
}

// ---- helpers over base-field tables (morpheus_piop.cuh:20-140,160-172) ---------------------------
constexpr int MAXV = 32;
struct VarMap {
    int n;
    int pos[MAXV];
};
// bit j of x goes to bit pos[j]
__device__ __forceinline__ uint64_t deposit(uint64_t x, const VarMap& m) {
    uint64_t r = 0;
    for (int j = 0; j < m.n; j++) r |= ((x >> j) & 1ULL) << m.pos[j];
    return r;
}

// Partial evaluation of a base-field table against a K table e over the `fix` variables:
//   out[r] = sum_f vals[deposit(r, rest) | deposit(f, fix)] e[f].
// A block handles output r = blockIdx.x (grid-stride) and the slice blockIdx.y of f: 32 sub-lanes times the
// eight coefficient lanes; partial[(r * gridDim.y + blockIdx.y) * 8 + c], summed by sum_rows_kernel.
static __global__ void __launch_bounds__(256)
pe_kernel(const uint64_t* __restrict__ vals, VarMap rest, VarMap fix, const uint64_t* __restrict__ e, uint64_t nrest,
          uint64_t nfix, uint64_t* __restrict__ partial) {
    __shared__ uint64_t red[32][8];
    const int c = threadIdx.x & 7, sub = threadIdx.x >> 3;
    const uint64_t per = (nfix + gridDim.y - 1) / gridDim.y;
    const uint64_t f0 = (uint64_t)blockIdx.y * per, f1 = f0 + per < nfix ? f0 + per : nfix;
    for (uint64_t r = blockIdx.x; r < nrest; r += gridDim.x) {
        const uint64_t ro = deposit(r, rest);
        gl::Acc acc = gl::acc_zero();
        for (uint64_t f = f0 + sub; f < f1; f += 32) {
            const uint64_t v = vals[ro | deposit(f, fix)];
            if (v) gl::acc_mul(acc, agl::canon(v), e[8 * f + c]);
        }
        red[sub][c] = agl::acc_reduce_wide(acc);
        __syncthreads();
        if (sub == 0) {
            uint64_t s = 0;
            for (int k = 0; k < 32; k++) s = agl::add(s, red[k][c]);
            partial[(r * gridDim.y + blockIdx.y) * 8 + c] = agl::canon(s);
        }
        __syncthreads();
    }
}
// out[r * 8 + c] = sum over `rows` partial rows
static __global__ void sum_rows_kernel(const uint64_t* __restrict__ partial, uint64_t nout, int rows, uint64_t* __restrict__ out) {
    const uint64_t total = nout * 8, step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
        const uint64_t r = t >> 3;
        const int c = (int)(t & 7);
        uint64_t s = 0;
        for (int k = 0; k < rows; k++) s = agl::add(s, partial[(r * rows + k) * 8 + c]);
        out[t] = agl::canon(s);
    }
}

// sum_x a[x] b[x] over K: partial[blockIdx.x * 8 + c] (block sums; eight lanes per element).
static __global__ void __launch_bounds__(256)
dot_kernel(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b, uint64_t n, uint64_t* __restrict__ partial) {
    __shared__ uint64_t red[8][8];
    const int c = threadIdx.x & 7, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) >> 3;
    const uint64_t rounds = (n + groups - 1) / groups;
    uint64_t x = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3, s = 0;
    for (uint64_t it = 0; it < rounds; it++, x += groups) {
        const bool live = x < n;
        const uint64_t av = live ? a[8 * x + c] : 0, bv = live ? b[8 * x + c] : 0;
        s = agl::add(s, mul_lane(av, bv, c));
    }
    s = agl::add(s, __shfl_xor_sync(0xffffffffu, s, 8));
    s = agl::add(s, __shfl_xor_sync(0xffffffffu, s, 16));
    if (lane < 8) red[warp][lane] = s;
    __syncthreads();
    if (threadIdx.x < 8) {
        uint64_t v = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) v = agl::add(v, red[w][threadIdx.x]);
        partial[(uint64_t)blockIdx.x * 8 + threadIdx.x] = agl::canon(v);
    }
}

// out[x] = in[sum_j ((x >> pos[j]) & 1) << j]  (morpheus_piop.cuh:166-172)
static __global__ void gather_kernel(const uint64_t* __restrict__ in, VarMap m, uint64_t n, uint64_t* __restrict__ out) {
    const uint64_t total = n * 8, step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
        const uint64_t x = t >> 3;
        uint64_t idx = 0;
        for (int j = 0; j < m.n; j++) idx |= ((x >> m.pos[j]) & 1ULL) << j;
        out[t] = in[8 * idx + (t & 7)];
    }
}
// out[i] = table[(sel[i] >> shift) & mask]  (morpheus_piop.cuh:160-164)
static __global__ void sel_lookup_kernel(const uint64_t* __restrict__ sel, uint64_t n, int shift, uint64_t mask,
                                         const uint64_t* __restrict__ table, uint64_t* __restrict__ out) {
    const uint64_t total = n * 8, step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step)
        out[t] = table[8 * ((sel[t >> 3] >> shift) & mask) + (t & 7)];
}

}  // namespace k8
}  // namespace mb
