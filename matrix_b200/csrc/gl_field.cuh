// Goldilocks field p = 2^64 - 2^32 + 1 and its quadratic extension
// F_p[X]/(X^2 - 7) for sm_100a device code.
//
// Same field as the reference's cuda/goldilocks.cuh:27 and cuda/extension.cuh:23;
// the arithmetic here is written for this library: values travel between
// operations as "loose" residues anywhere in [0, 2^64) and are brought to the
// canonical range [0, p) only where they leave a kernel or enter a hash
// comparison. Sums of canonical residues are order independent, so any
// reduction tree gives bit-identical results to the reference's CPU prover.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

// Every function is also callable from host code so that the exact device
// arithmetic can be unit-tested on a machine without a GPU.
#define GLF __host__ __device__ __forceinline__

namespace gl {

GLF uint64_t umulhi(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    return __umul64hi(a, b);
#else
    return (uint64_t)(((unsigned __int128)a * b) >> 64);
#endif
}

constexpr uint64_t P = 0xFFFFFFFF00000001ULL;
constexpr uint64_t EPS = 0xFFFFFFFFULL;  // 2^64 mod p

// The integer datapath of an SM issues about one 32-bit operation per lane every
// two cycles whatever the operation, so the cost of field arithmetic is its
// instruction count (measured: 0.57 warp instructions per cycle and scheduler for
// any mix of additions, logic and multiply-adds). The device forms below use the
// carry flag and one multiply-add for the +-EPS repair: canon 4 instructions,
// add_c 4, add 8, sub_c 5, sub 9, where the comparison forms compile to 9 - 19.
#ifdef __CUDA_ARCH__
// carry of a + b and the wrapped sum
__device__ __forceinline__ uint64_t add_cc(uint64_t a, uint64_t b, uint32_t& carry) {
    uint64_t r;
    asm("add.cc.u64 %0, %2, %3;\n\taddc.u32 %1, 0, 0;" : "=l"(r), "=r"(carry) : "l"(a), "l"(b));
    return r;
}
// x + k * EPS mod 2^64 (one multiply-add)
__device__ __forceinline__ uint64_t plus_eps(uint64_t x, uint32_t k) {
    uint64_t r;
    asm("mad.wide.u32 %0, %1, 0xFFFFFFFF, %2;" : "=l"(r) : "r"(k), "l"(x));
    return r;
}
#endif

// x >= p exactly when x + EPS wraps; then x - p = x + EPS - 2^64.
GLF uint64_t canon(uint64_t x) {
#ifdef __CUDA_ARCH__
    uint32_t c;
    (void)add_cc(x, EPS, c);
    return plus_eps(x, c);
#else
    return x >= P ? x - P : x;
#endif
}

// a + b where b < p: one wrap at most, and the repaired sum stays below 2^64.
GLF uint64_t add_c(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint32_t c;
    uint64_t s = add_cc(a, b, c);
    return plus_eps(s, c);
#else
    uint64_t s = a + b;
    return s < a ? s + EPS : s;
#endif
}

// a + b for loose a, b. The wrapped sum is made canonical first, so the repair
// of the wrap (+ EPS) cannot wrap again.
GLF uint64_t add(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint32_t c;
    uint64_t s = add_cc(a, b, c);
    return plus_eps(canon(s), c);
#else
    uint64_t s = a + b;
    if (s < a) {
        s += EPS;
        if (s < EPS) s += EPS;
    }
    return s;
#endif
}

// a - b where b < p: a borrow is repaired by - EPS, which cannot underflow
// because the wrapped difference exceeds 2^64 - p = EPS.
GLF uint64_t sub_c(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint64_t r;
    uint32_t m;
    asm("sub.cc.u64 %0, %2, %3;\n\tsubc.u32 %1, 0, 0;" : "=l"(r), "=r"(m) : "l"(a), "l"(b));
    return r - (uint64_t)m;
#else
    uint64_t d = a - b;
    return a < b ? d - EPS : d;
#endif
}

GLF uint64_t sub(uint64_t a, uint64_t b) { return sub_c(a, canon(b)); }

GLF uint64_t neg(uint64_t a) { return sub(0, a); }

// ---- 32-bit limb helpers ------------------------------------------------------
// The integer datapath of an SM issues one 32-bit operation per lane every two
// cycles whatever the operation, so the cost of field arithmetic is its
// instruction count. mad.wide.u32 (32 x 32 + 64 -> 64) folds an addition into
// every multiplication; the reductions below are built from it and need one
// borrow (or carry) fix-up each, with bounds that rule out a second one.
GLF uint32_t lo32(uint64_t x) { return (uint32_t)x; }
GLF uint32_t hi32(uint64_t x) { return (uint32_t)(x >> 32); }
GLF uint64_t pack64(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }

// a * b + c, exact in 64 bits (callers keep the sum below 2^64).
GLF uint64_t madwide(uint32_t a, uint32_t b, uint64_t c) {
#ifdef __CUDA_ARCH__
    uint64_t r;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"(a), "r"(b), "l"(c));
    return r;
#else
    return (uint64_t)a * b + c;
#endif
}

// a - b and the borrow as a mask (0 or 0xFFFFFFFF = EPS).
GLF uint64_t sub_borrow(uint64_t a, uint64_t b, uint32_t& mask) {
#ifdef __CUDA_ARCH__
    uint64_t r;
    asm("sub.cc.u64 %0, %2, %3;\n\tsubc.u32 %1, 0, 0;" : "=l"(r), "=r"(mask) : "l"(a), "l"(b));
    return r;
#else
    mask = a < b ? 0xFFFFFFFFu : 0u;
    return a - b;
#endif
}

// a + b and the carry (0 or 1).
GLF uint64_t add_carry(uint64_t a, uint64_t b, uint32_t& carry) {
#ifdef __CUDA_ARCH__
    uint64_t r;
    asm("add.cc.u64 %0, %2, %3;\n\taddc.u32 %1, 0, 0;" : "=l"(r), "=r"(carry) : "l"(a), "l"(b));
    return r;
#else
    uint64_t r = a + b;
    carry = r < a ? 1u : 0u;
    return r;
#endif
}

// z = z0 + z1 2^32 + z2 2^64 + z3 2^96 mod p, loose result.
// With 2^64 = 2^32 - 1 and 2^96 = -1 (mod p): z = z0 + 2^32 (z1 + z2) - (z2 + z3).
// A = z1 + z2 has 33 bits; its top bit is worth 2^64 = EPS and is added to
// W = (A_lo : z0) without overflow (A_c = 1 forces A_lo <= 2^32 - 2). Then one
// subtraction of B = z2 + z3 < 2^33; a borrow is repaired by - EPS, which
// cannot underflow because the wrapped value exceeds 2^64 - 2^33.
GLF uint64_t reduce_limbs(uint32_t z0, uint32_t z1, uint32_t z2, uint32_t z3) {
    uint64_t A = madwide(z2, 1u, (uint64_t)z1);
    uint64_t B = madwide(z3, 1u, (uint64_t)z2);
    uint64_t W = madwide(hi32(A), 0xFFFFFFFFu, pack64(z0, lo32(A)));
    uint32_t m;
    uint64_t R = sub_borrow(W, B, m);
    return R - (uint64_t)m;
}

// (hi:lo) mod p, loose result.
GLF uint64_t reduce128(uint64_t lo, uint64_t hi) { return reduce_limbs(lo32(lo), hi32(lo), lo32(hi), hi32(hi)); }

// L + H 2^32 mod p for limb sums L, H < 2^40 (sums of up to 256 low / high
// halves), loose result. W = (A_lo : L_lo) with A = L_hi + H_lo; the remaining
// weight k = A_c + H_hi < 2^9 is worth k EPS; one carry fix-up, and the wrapped
// value is below k EPS so it cannot carry again.
GLF uint64_t reduce_limb_sums(uint64_t L, uint64_t H) {
    uint64_t A = madwide(hi32(L), 1u, (uint64_t)lo32(H));
    uint32_t k = hi32(A) + hi32(H);
    uint64_t W = pack64(lo32(L), lo32(A));
    uint64_t kE = madwide(k, 0xFFFFFFFFu, 0);
    uint32_t c;
    uint64_t s = add_carry(W, kE, c);
    return madwide(c, 0xFFFFFFFFu, s);
}

GLF uint64_t mul(uint64_t a, uint64_t b) {
    return reduce128(a * b, umulhi(a, b));
}

// a * b + c mod p for loose a, b, c: the 128-bit sum cannot overflow
// ((2^64 - 1)^2 + 2^64 - 1 < 2^128), so the addition costs two instructions
// instead of a modular add after the reduction.
GLF uint64_t mul_add(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t lo = a * b, hi = umulhi(a, b);
    uint32_t carry;
    uint64_t l2 = add_carry(lo, c, carry);
    return reduce128(l2, hi + carry);
}

GLF uint64_t sqr(uint64_t a) { return mul(a, a); }

// a * k for a small constant k < 2^32: the high word has hh = 0.
GLF uint64_t mul_small(uint64_t a, uint32_t k) {
    uint64_t lo = a * (uint64_t)k, hi = umulhi(a, (uint64_t)k);  // hi < 2^32
    uint64_t t1 = (hi << 32) - hi;
    uint64_t r = lo + t1;
    if (r < t1) r += EPS;
    return r;
}

GLF uint64_t pw(uint64_t a, uint64_t e) {
    uint64_t r = 1;
    while (e) {
        if (e & 1) r = mul(r, a);
        a = sqr(a);
        e >>= 1;
    }
    return r;
}

// Fermat inverse; inv(0) = 0.
GLF uint64_t inv(uint64_t a) { return pw(a, P - 2); }

// ---- lazily reduced sums of products ------------------------------------------
// A sum of a few 128-bit products (and 64-bit addends) is kept exact in 160 bits
// and reduced once: per product that is five multiply-adds for the product and
// five additions with carry, against a full reduction and a modular addition
// when every product is reduced on its own.

// x * y as (hi : lo), from four 32 x 32 products. No step overflows:
// (2^32 - 1)^2 + 2 (2^32 - 1) = 2^64 - 1.
GLF void mul128(uint64_t x, uint64_t y, uint64_t& lo, uint64_t& hi) {
#ifdef __CUDA_ARCH__
    const uint32_t x0 = lo32(x), x1 = hi32(x), y0 = lo32(y), y1 = hi32(y);
    uint64_t p00 = madwide(x0, y0, 0);
    uint64_t p01 = madwide(x0, y1, (uint64_t)hi32(p00));
    uint64_t p10 = madwide(x1, y0, (uint64_t)lo32(p01));
    uint64_t p11 = madwide(x1, y1, (uint64_t)hi32(p01));
    lo = pack64(lo32(p00), lo32(p10));
    hi = madwide(hi32(p10), 1u, p11);
#else
    unsigned __int128 f = (unsigned __int128)x * y;
    lo = (uint64_t)f;
    hi = (uint64_t)(f >> 64);
#endif
}

// Five 32-bit limbs, a4 the top (room for 2^32 products).
struct Acc {
    uint32_t a0, a1, a2, a3, a4;
};
GLF Acc acc_zero() { return Acc{0, 0, 0, 0, 0}; }
GLF Acc acc_from(uint64_t v) { return Acc{lo32(v), hi32(v), 0, 0, 0}; }
GLF void acc_add128(Acc& s, uint64_t lo, uint64_t hi) {
#ifdef __CUDA_ARCH__
    asm("add.cc.u32 %0, %0, %5;\n\taddc.cc.u32 %1, %1, %6;\n\taddc.cc.u32 %2, %2, %7;\n\taddc.cc.u32 %3, %3, %8;\n\t"
        "addc.u32 %4, %4, 0;"
        : "+r"(s.a0), "+r"(s.a1), "+r"(s.a2), "+r"(s.a3), "+r"(s.a4)
        : "r"(lo32(lo)), "r"(hi32(lo)), "r"(lo32(hi)), "r"(hi32(hi)));
#else
    unsigned __int128 cur = ((unsigned __int128)pack64(s.a2, s.a3) << 64) | pack64(s.a0, s.a1);
    unsigned __int128 add = ((unsigned __int128)hi << 64) | lo;
    unsigned __int128 r = cur + add;
    if (r < cur) s.a4++;
    s.a0 = (uint32_t)r; s.a1 = (uint32_t)(r >> 32); s.a2 = (uint32_t)(r >> 64); s.a3 = (uint32_t)(r >> 96);
#endif
}
GLF void acc_add(Acc& s, uint64_t v) { acc_add128(s, v, 0); }
// s += x * y: the even columns x0 y0, x1 y1 in one carry chain, then the two
// cross products (13 multiply-adds and carry additions in all).
GLF void acc_mul(Acc& s, uint64_t x, uint64_t y) {
#ifdef __CUDA_ARCH__
    asm("mad.lo.cc.u32 %0, %5, %7, %0;\n\t"
        "madc.hi.cc.u32 %1, %5, %7, %1;\n\t"
        "madc.lo.cc.u32 %2, %6, %8, %2;\n\t"
        "madc.hi.cc.u32 %3, %6, %8, %3;\n\t"
        "addc.u32 %4, %4, 0;\n\t"
        "mad.lo.cc.u32 %1, %5, %8, %1;\n\t"
        "madc.hi.cc.u32 %2, %5, %8, %2;\n\t"
        "addc.cc.u32 %3, %3, 0;\n\t"
        "addc.u32 %4, %4, 0;\n\t"
        "mad.lo.cc.u32 %1, %6, %7, %1;\n\t"
        "madc.hi.cc.u32 %2, %6, %7, %2;\n\t"
        "addc.cc.u32 %3, %3, 0;\n\t"
        "addc.u32 %4, %4, 0;"
        : "+r"(s.a0), "+r"(s.a1), "+r"(s.a2), "+r"(s.a3), "+r"(s.a4)
        : "r"(lo32(x)), "r"(hi32(x)), "r"(lo32(y)), "r"(hi32(y)));
#else
    uint64_t lo, hi;
    mul128(x, y, lo, hi);
    acc_add128(s, lo, hi);
#endif
}
// s mod p for a top limb below 2^8, loose result. 2^128 = -2^32 (mod p), so the top
// limb joins the subtrahend of reduce_limbs: B = z2 + z3 + 2^32 top < 2^41, and the
// repair of a borrow still cannot underflow (the wrapped value exceeds 2^64 - 2^41).
GLF uint64_t acc_reduce(const Acc& s) {
    uint64_t A = madwide(s.a2, 1u, (uint64_t)s.a1);
    uint64_t B0 = madwide(s.a3, 1u, (uint64_t)s.a2);
    uint64_t B = pack64(lo32(B0), hi32(B0) + s.a4);
    uint64_t W = madwide(hi32(A), 0xFFFFFFFFu, pack64(s.a0, lo32(A)));
    uint32_t m;
    uint64_t R = sub_borrow(W, B, m);
    return R - (uint64_t)m;
}
// s mod p for any top limb (long-running accumulators): top 2^128 = -top 2^32.
GLF uint64_t acc_reduce_wide(const Acc& s) {
    return sub(reduce_limbs(s.a0, s.a1, s.a2, s.a3), (uint64_t)s.a4 << 32);
}

// a - b for canonical a, b; canonical result (one borrow repair: + p = - EPS mod 2^64).
GLF uint64_t sub_canon(uint64_t a, uint64_t b) { return sub_c(a, b); }

// ---------------------------------------------------------------------------
// Quadratic extension, X^2 = 7. Stored as (c0, c1), two consecutive u64.
// ---------------------------------------------------------------------------
struct E2 {
    uint64_t c0, c1;
};

GLF E2 e2(uint64_t c0, uint64_t c1) { return E2{c0, c1}; }
GLF E2 e2_add(E2 a, E2 b) { return E2{add(a.c0, b.c0), add(a.c1, b.c1)}; }
GLF E2 e2_sub(E2 a, E2 b) { return E2{sub(a.c0, b.c0), sub(a.c1, b.c1)}; }
GLF E2 e2_canon(E2 a) { return E2{canon(a.c0), canon(a.c1)}; }

GLF E2 e2_mul(E2 a, E2 b) {
    uint64_t m0 = mul(a.c0, b.c0), m1 = mul(a.c1, b.c1);
    uint64_t x = mul(add(a.c0, a.c1), add(b.c0, b.c1));
    return E2{add(m0, mul_small(m1, 7)), sub(sub(x, m0), m1)};
}

GLF E2 e2_mul_base(E2 a, uint64_t b) { return E2{mul(a.c0, b), mul(a.c1, b)}; }

// A loop-invariant extension factor with 7 c1 precomputed: r * d needs four
// products and two reductions, no modular additions.
struct E2Pre {
    uint64_t c0, c1, c1w;
};
GLF E2Pre e2_pre(E2 r) { return E2Pre{canon(r.c0), canon(r.c1), canon(mul_small(canon(r.c1), 7))}; }
// a + r * d
GLF E2 e2_fma_pre(E2Pre r, E2 d, E2 a) {
    Acc s0 = acc_from(a.c0), s1 = acc_from(a.c1);
    acc_mul(s0, r.c0, d.c0);
    acc_mul(s0, r.c1w, d.c1);
    acc_mul(s1, r.c0, d.c1);
    acc_mul(s1, r.c1, d.c0);
    return E2{acc_reduce(s0), acc_reduce(s1)};
}
GLF E2 e2_mul_pre(E2Pre r, E2 d) { return e2_fma_pre(r, d, E2{0, 0}); }
// a + r * d for a base-field d
GLF E2 e2_fma_pre_base(E2Pre r, uint64_t d, uint64_t a) {
    Acc s0 = acc_from(a), s1 = acc_zero();
    acc_mul(s0, r.c0, d);
    acc_mul(s1, r.c1, d);
    return E2{acc_reduce(s0), acc_reduce(s1)};
}

// Lazy accumulator of extension products: sum a_k b_k as three exact sums.
struct E2Acc {
    Acc s00, s11, s01;
};
GLF E2Acc e2acc_zero() { return E2Acc{acc_zero(), acc_zero(), acc_zero()}; }
GLF void e2acc_mul(E2Acc& q, E2 a, E2 b) {
    acc_mul(q.s00, a.c0, b.c0);
    acc_mul(q.s11, a.c1, b.c1);
    acc_mul(q.s01, a.c0, b.c1);
    acc_mul(q.s01, a.c1, b.c0);
}
// one product through the lazy sums: four multiplications, three reductions
GLF E2 e2_mul_lazy(E2 a, E2 b);
// at most 64 products accumulated (top limbs below 2^8)
GLF E2 e2acc_reduce(const E2Acc& q) {
    return E2{add(acc_reduce(q.s00), mul_small(acc_reduce(q.s11), 7)), acc_reduce(q.s01)};
}
GLF E2 e2_mul_lazy(E2 a, E2 b) {
    E2Acc q = e2acc_zero();
    e2acc_mul(q, a, b);
    return e2acc_reduce(q);
}

GLF E2 e2_inv(E2 a) {
    uint64_t n = sub(sqr(a.c0), mul_small(sqr(a.c1), 7));
    uint64_t ni = inv(n);
    return E2{mul(a.c0, ni), mul(neg(a.c1), ni)};
}

// 16-byte vector access to an extension element.
GLF E2 e2_load(const uint64_t* p) {
    ulonglong2 v = *reinterpret_cast<const ulonglong2*>(p);
    return E2{v.x, v.y};
}
GLF void e2_store(uint64_t* p, E2 v) {
    *reinterpret_cast<ulonglong2*>(p) = make_ulonglong2(v.c0, v.c1);
}

}  // namespace gl
