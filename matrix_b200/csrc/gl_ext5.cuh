// Degree-5 extension of Goldilocks, F_p[X]/(X^5 - 3): five consecutive u64 per
// element, coefficient of X^i at word i (reference: cuda/extension.cuh:27-28,
// 299-700; element layout goldilocks-cuda-rs/cuda/wrapper.cu:567-587).
//
// Products go through five exact 160-bit sums (one per output coefficient) with
// the wrapped terms' factor 3 folded into the second operand once, so a product
// costs 25 multiply-accumulate chains and five reductions instead of the 29
// reduced multiplications and 20 modular additions of the term-by-term form.
// The inverse uses the Frobenius map twice on partial products
// (a^(p + p^2) = (a a^p)^p, a^(p^3 + p^4) = (a^(p + p^2))^(p^2)): two full
// products, one coefficient of a third, one base-field inversion.
#pragma once
#include "gl_field.cuh"

namespace gl {

struct E5 {
    uint64_t c[5];
};

constexpr uint32_t E5_W = 3;
// DTH^k for DTH = 3^((p - 1) / 5) = 1041288259238279555 (cuda/extension.cuh:28);
// X^p = DTH X, and DTH^5 = 1.
#define MB_E5_DTH(k)                                                                      \
    ((k) == 0 ? 1ull : (k) == 1 ? 0x0e736627a0aeb983ull : (k) == 2 ? 0xdb8edc802dc0b266ull \
     : (k) == 3 ? 0x02efb5c2a6f35241ull : 0x130e07948a9d41d6ull)

GLF E5 e5_zero() { return E5{{0, 0, 0, 0, 0}}; }
GLF E5 e5_one() { return E5{{1, 0, 0, 0, 0}}; }
GLF E5 e5_canon(E5 a) {
    E5 r;
#pragma unroll
    for (int i = 0; i < 5; i++) r.c[i] = canon(a.c[i]);
    return r;
}
GLF E5 e5_load(const uint64_t* p) {
    E5 r;
#pragma unroll
    for (int i = 0; i < 5; i++) r.c[i] = p[i];
    return r;
}
GLF void e5_store(uint64_t* p, E5 v) {
#pragma unroll
    for (int i = 0; i < 5; i++) p[i] = canon(v.c[i]);
}

// a * b; any representatives in, loose residues out.
GLF E5 e5_mul(E5 a, E5 b) {
    uint64_t bw[5];
#pragma unroll
    for (int j = 1; j < 5; j++) bw[j] = mul_small(b.c[j], E5_W);
    bw[0] = 0;
    E5 r;
#pragma unroll
    for (int k = 0; k < 5; k++) {
        Acc s = acc_zero();
#pragma unroll
        for (int i = 0; i < 5; i++) {
            const int j = k - i;  // i + j = k, or i + j = k + 5 with the factor 3
            if (j >= 0) acc_mul(s, a.c[i], b.c[j]);
            else acc_mul(s, a.c[i], bw[j + 5]);
        }
        r.c[k] = acc_reduce(s);
    }
    return r;
}

// coefficient 0 of a * b
GLF uint64_t e5_mul_c0(E5 a, E5 b) {
    Acc s = acc_zero();
    acc_mul(s, a.c[0], b.c[0]);
#pragma unroll
    for (int i = 1; i < 5; i++) acc_mul(s, a.c[i], mul_small(b.c[5 - i], E5_W));
    return acc_reduce(s);
}

GLF E5 e5_mul_base(E5 a, uint64_t s) {
    E5 r;
#pragma unroll
    for (int i = 0; i < 5; i++) r.c[i] = mul(a.c[i], s);
    return r;
}

// a^(p^k): coefficient i times DTH^(i k mod 5)
template <int K>
GLF E5 e5_frobenius(E5 a) {
    E5 r;
    r.c[0] = a.c[0];
#pragma unroll
    for (int i = 1; i < 5; i++) r.c[i] = mul(a.c[i], MB_E5_DTH((i * K) % 5));
    return r;
}

// 1 / a (0 for a = 0, like the reference's exponentiation-based base inverse)
GLF E5 e5_inv(E5 a) {
    E5 u = e5_frobenius<1>(e5_mul(a, e5_frobenius<1>(a)));  // a^(p + p^2)
    E5 conj = e5_mul(u, e5_frobenius<2>(u));                // a^(p + p^2 + p^3 + p^4)
    uint64_t norm = e5_mul_c0(a, conj);                     // a^(1 + p + ... + p^4), in F_p
    return e5_mul_base(conj, inv(norm));
}

// a^e, square and multiply from the low bit
GLF E5 e5_pow(E5 a, uint64_t e) {
    E5 r = e5_one(), b = a;
    while (e) {
        if (e & 1) r = e5_mul(r, b);
        e >>= 1;
        if (e) b = e5_mul(b, b);
    }
    return r;
}

}  // namespace gl
