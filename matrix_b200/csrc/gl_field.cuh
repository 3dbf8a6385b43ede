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

GLF uint64_t canon(uint64_t x) { return x >= P ? x - P : x; }

// a + b for loose a, b. Each wrap past 2^64 is worth +EPS; a second wrap is only
// possible when both operands are at or above p.
GLF uint64_t add(uint64_t a, uint64_t b) {
    uint64_t s = a + b;
    if (s < a) {
        s += EPS;
        if (s < EPS) s += EPS;
    }
    return s;
}

// a + b where b < p: one correction suffices.
GLF uint64_t add_c(uint64_t a, uint64_t b) {
    uint64_t s = a + b;
    return s < a ? s + EPS : s;
}

GLF uint64_t sub(uint64_t a, uint64_t b) {
    uint64_t d = a - b;
    if (a < b) {
        uint64_t e = d - EPS;
        d = (d < EPS) ? e - EPS : e;
    }
    return d;
}

// a - b where b < p.
GLF uint64_t sub_c(uint64_t a, uint64_t b) {
    uint64_t d = a - b;
    return a < b ? d - EPS : d;
}

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
