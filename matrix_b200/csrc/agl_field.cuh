// Almost-Goldilocks field q = 2^64 - 2^32 - 31 and its quadratic extension
// F_q[X]/(X^2 - 3) for sm_100a device code (same field as the reference's
// cuda_almost_goldilocks/almost_goldilocks.cuh:32 and almost_extension.cuh:32).
//
// 2^64 = c = 2^32 + 31 (mod q). Values travel as loose residues in [0, 2^64)
// and are made canonical where they are written out. The reduction works on
// 32-bit limbs: with 2^96 = 2^37 + 31 (mod q),
//   z0 + z1 2^32 + z2 2^64 + z3 2^96 = (z0 + 31 z2 + 31 z3) + 2^32 (z1 + z2 + 32 z3),
// two limb sums below 2^39 that are folded once (the reference's
// agl_reduce128, almost_goldilocks.cuh:176-193, runs three multiply passes).
#pragma once
#include "gl_field.cuh"

namespace agl {

using gl::add_carry;
using gl::hi32;
using gl::lo32;
using gl::madwide;
using gl::pack64;
using gl::umulhi;

constexpr uint64_t P = 0xFFFFFFFEFFFFFFE1ULL;  // q
constexpr uint64_t C = 0x000000010000001FULL;  // 2^64 mod q = 2^32 + 31

// Device forms use the carry flag and one multiply-add for the +-c repair, like the Goldilocks
// primitives (the cost of this arithmetic is its instruction count).
#ifdef __CUDA_ARCH__
// x + k c mod 2^64 for k in {0, 1}: c = 2^32 + 31
__device__ __forceinline__ uint64_t plus_c(uint64_t x, uint32_t k) {
    return madwide(k, 31u, x) + ((uint64_t)k << 32);
}
#endif

// x >= q exactly when x + c wraps; then x - q = x + c - 2^64.
GLF uint64_t canon(uint64_t x) {
#ifdef __CUDA_ARCH__
    uint32_t carry;
    (void)gl::add_cc(x, C, carry);
    return plus_c(x, carry);
#else
    return x >= P ? x - P : x;
#endif
}

// a + b where b < q: one wrap at most, and the repaired sum stays below 2^64.
GLF uint64_t add_c(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint32_t carry;
    uint64_t s = gl::add_cc(a, b, carry);
    return plus_c(s, carry);
#else
    uint64_t s = a + b;
    return s < a ? s + C : s;
#endif
}

// a + b for loose a, b: the wrapped sum is made canonical first, so the repair cannot wrap again.
GLF uint64_t add(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint32_t carry;
    uint64_t s = gl::add_cc(a, b, carry);
    return plus_c(canon(s), carry);
#else
    uint64_t s = a + b;
    if (s < a) {
        s += C;
        if (s < C) s += C;
    }
    return s;
#endif
}

// a - b where b < q: a borrow is repaired by - c, which cannot underflow (the wrapped difference exceeds c).
GLF uint64_t sub_c(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint64_t r;
    uint32_t m;
    asm("sub.cc.u64 %0, %2, %3;\n\tsubc.u32 %1, 0, 0;" : "=l"(r), "=r"(m) : "l"(a), "l"(b));
    return r - ((uint64_t)(m & 1u) << 32) - (uint64_t)(m & 31u);
#else
    uint64_t d = a - b;
    return a < b ? d - C : d;
#endif
}
GLF uint64_t sub(uint64_t a, uint64_t b) { return sub_c(a, canon(b)); }
GLF uint64_t neg(uint64_t a) { return sub(0, a); }

// L + H 2^32 mod q for L, H < 2^40, loose result. W = (A_lo : L_lo) with
// A = L_hi + H_lo; the weight k = A_c + H_hi < 2^9 of 2^64 is worth k c < 2^42;
// one carry fix-up, and the wrapped value is below k c so it cannot carry again.
GLF uint64_t reduce_limb_sums(uint64_t L, uint64_t H) {
    uint64_t A = madwide(hi32(L), 1u, (uint64_t)lo32(H));
    uint32_t k = hi32(A) + hi32(H);
    uint64_t W = pack64(lo32(L), lo32(A));
    uint64_t kc = madwide(k, 31u, (uint64_t)k << 32);
    uint32_t carry;
    uint64_t s = add_carry(W, kc, carry);
    return madwide(carry, 31u, s) + ((uint64_t)carry << 32);
}

GLF uint64_t reduce_limbs(uint32_t z0, uint32_t z1, uint32_t z2, uint32_t z3) {
    uint64_t L = madwide(z3, 31u, madwide(z2, 31u, (uint64_t)z0));
    uint64_t H = madwide(z3, 32u, madwide(z2, 1u, (uint64_t)z1));
    return reduce_limb_sums(L, H);
}
GLF uint64_t reduce128(uint64_t lo, uint64_t hi) { return reduce_limbs(lo32(lo), hi32(lo), lo32(hi), hi32(hi)); }

// An exact 160-bit sum of products (gl::Acc: the accumulation is integer
// arithmetic, the same for both fields) mod q, top limb below 2^8, loose result:
// 2^128 = c^2 = 63 2^32 + 992 (mod q) joins the two limb sums of reduce_limbs.
GLF uint64_t acc_reduce(const gl::Acc& s) {
    uint64_t L = madwide(s.a4, 992u, madwide(s.a3, 31u, madwide(s.a2, 31u, (uint64_t)s.a0)));
    uint64_t H = madwide(s.a4, 63u, madwide(s.a3, 32u, madwide(s.a2, 1u, (uint64_t)s.a1)));
    return reduce_limb_sums(L, H);
}

// The same for any top limb (long-running accumulators): top 2^128 = top (63 2^32 + 992) mod q.
GLF uint64_t mul(uint64_t a, uint64_t b);
GLF uint64_t acc_reduce_wide(const gl::Acc& s) {
    const uint64_t low = reduce_limbs(s.a0, s.a1, s.a2, s.a3);
    return add(low, mul((uint64_t)s.a4, 63ULL * (1ULL << 32) + 992ULL));
}

GLF uint64_t mul(uint64_t a, uint64_t b) { return reduce128(a * b, umulhi(a, b)); }
GLF uint64_t sqr(uint64_t a) { return mul(a, a); }
GLF uint64_t mul_small(uint64_t a, uint32_t k) {
    uint64_t lo = a * (uint64_t)k, hi = umulhi(a, (uint64_t)k);
    return reduce128(lo, hi);
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
GLF uint64_t inv(uint64_t a) { return pw(a, P - 2); }

// Quadratic extension, X^2 = 3.
struct E2 {
    uint64_t c0, c1;
};
GLF E2 e2_add(E2 a, E2 b) { return E2{add(a.c0, b.c0), add(a.c1, b.c1)}; }
GLF E2 e2_sub(E2 a, E2 b) { return E2{sub(a.c0, b.c0), sub(a.c1, b.c1)}; }
GLF E2 e2_canon(E2 a) { return E2{canon(a.c0), canon(a.c1)}; }
GLF E2 e2_mul(E2 a, E2 b) {
    uint64_t m0 = mul(a.c0, b.c0), m1 = mul(a.c1, b.c1);
    uint64_t x = mul(add(a.c0, a.c1), add(b.c0, b.c1));
    return E2{add(m0, mul_small(m1, 3)), sub(sub(x, m0), m1)};
}
GLF E2 e2_mul_base(E2 a, uint64_t b) { return E2{mul(a.c0, b), mul(a.c1, b)}; }

// Products through exact 160-bit sums reduced once (gl::Acc), as for Goldilocks.
// One product: four multiplications, three reductions, no modular additions inside.
GLF E2 e2_mul_lazy(E2 a, E2 b) {
    gl::Acc s00 = gl::acc_zero(), s11 = gl::acc_zero(), s01 = gl::acc_zero();
    gl::acc_mul(s00, a.c0, b.c0);
    gl::acc_mul(s11, a.c1, b.c1);
    gl::acc_mul(s01, a.c0, b.c1);
    gl::acc_mul(s01, a.c1, b.c0);
    return E2{add(agl::acc_reduce(s00), mul_small(agl::acc_reduce(s11), 3)), agl::acc_reduce(s01)};
}
// A loop-invariant factor with 3 c1 precomputed: a + r d needs four products and two reductions.
struct E2Pre {
    uint64_t c0, c1, c1w;
};
GLF E2Pre e2_pre(E2 r) { return E2Pre{canon(r.c0), canon(r.c1), canon(mul_small(canon(r.c1), 3))}; }
GLF E2 e2_fma_pre(E2Pre r, E2 d, E2 a) {
    gl::Acc s0 = gl::acc_from(a.c0), s1 = gl::acc_from(a.c1);
    gl::acc_mul(s0, r.c0, d.c0);
    gl::acc_mul(s0, r.c1w, d.c1);
    gl::acc_mul(s1, r.c0, d.c1);
    gl::acc_mul(s1, r.c1, d.c0);
    return E2{agl::acc_reduce(s0), agl::acc_reduce(s1)};
}
GLF E2 e2_fma_pre_base(E2Pre r, uint64_t d, uint64_t a) {
    gl::Acc s0 = gl::acc_from(a), s1 = gl::acc_zero();
    gl::acc_mul(s0, r.c0, d);
    gl::acc_mul(s1, r.c1, d);
    return E2{agl::acc_reduce(s0), agl::acc_reduce(s1)};
}
GLF E2 e2_inv(E2 a) {
    uint64_t n = sub(sqr(a.c0), mul_small(sqr(a.c1), 3));
    uint64_t ni = inv(n);
    return E2{mul(a.c0, ni), mul(neg(a.c1), ni)};
}
GLF E2 e2_load(const uint64_t* p) {
    ulonglong2 v = *reinterpret_cast<const ulonglong2*>(p);
    return E2{v.x, v.y};
}
GLF void e2_store(uint64_t* p, E2 v) { *reinterpret_cast<ulonglong2*>(p) = make_ulonglong2(v.c0, v.c1); }

}  // namespace agl
