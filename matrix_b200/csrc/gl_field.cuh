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

// (hi:lo) mod p, loose result. 2^64 = EPS and 2^96 = -1 (mod p).
GLF uint64_t reduce128(uint64_t lo, uint64_t hi) {
    uint64_t hh = hi >> 32, hl = hi & EPS;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= EPS;
    uint64_t t1 = (hl << 32) - hl;  // hl * EPS
    uint64_t r = t0 + t1;
    if (r < t1) r += EPS;
    return r;
}

GLF uint64_t mul(uint64_t a, uint64_t b) {
    return reduce128(a * b, umulhi(a, b));
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
