// Field traits of almost-Goldilocks for the generic sumcheck / eq / partial
// evaluation kernels (the Goldilocks traits live in sumcheck_kernels.cuh).
#pragma once
#include "agl_field.cuh"
#include "sumcheck_kernels.cuh"

namespace mb {
namespace sc {

struct AglAdd {
    __device__ __forceinline__ uint64_t operator()(uint64_t a, uint64_t b) const { return agl::add(a, b); }
};
struct AglCanon {
    __host__ __device__ __forceinline__ uint64_t operator()(uint64_t a) const { return agl::canon(a); }
};

struct AglBase {
    using T = uint64_t;
    using WordAdd = AglAdd;
    using WordCanon = AglCanon;
    static constexpr int NW = 1;
    static __device__ __forceinline__ T load(const uint64_t* p, size_t i) { return p[i]; }
    static __device__ __forceinline__ void load2(const uint64_t* p, size_t i, T& a, T& b) {
        ulonglong2 v = *reinterpret_cast<const ulonglong2*>(p + i);
        a = v.x; b = v.y;
    }
    static __device__ __forceinline__ void store(uint64_t* p, size_t i, T v) { p[i] = agl::canon(v); }
    static __device__ __forceinline__ void store2(uint64_t* p, size_t i, T a, T b) {
        *reinterpret_cast<ulonglong2*>(p + i) = make_ulonglong2(agl::canon(a), agl::canon(b));
    }
    static __device__ __forceinline__ T add(T a, T b) { return agl::add(a, b); }
    static __device__ __forceinline__ T sub(T a, T b) { return agl::sub(a, b); }
    static __device__ __forceinline__ T mul(T a, T b) { return agl::mul(a, b); }
    static __device__ __forceinline__ T zero() { return 0; }
    static __device__ __forceinline__ void to_words(T v, uint64_t* w) { w[0] = v; }
    static __device__ __forceinline__ T from_words(const uint64_t* w) { return w[0]; }
    // a factor used many times (nothing to prepare in the base field)
    using Pre = uint64_t;
    static __device__ __forceinline__ Pre pre(T x) { return x; }
    static __device__ __forceinline__ T mul_pre(Pre p, T x) { return agl::mul(p, x); }
};

struct AglExt2 {
    using T = agl::E2;
    using WordAdd = AglAdd;
    using WordCanon = AglCanon;
    static constexpr int NW = 2;
    static __device__ __forceinline__ T load(const uint64_t* p, size_t i) { return agl::e2_load(p + 2 * i); }
    static __device__ __forceinline__ void load2(const uint64_t* p, size_t i, T& a, T& b) {
        a = agl::e2_load(p + 2 * i);
        b = agl::e2_load(p + 2 * i + 2);
    }
    static __device__ __forceinline__ void store(uint64_t* p, size_t i, T v) { agl::e2_store(p + 2 * i, agl::e2_canon(v)); }
    static __device__ __forceinline__ void store2(uint64_t* p, size_t i, T a, T b) {
        store(p, i, a);
        store(p, i + 1, b);
    }
    static __device__ __forceinline__ T add(T a, T b) { return agl::e2_add(a, b); }
    static __device__ __forceinline__ T sub(T a, T b) { return agl::e2_sub(a, b); }
    static __device__ __forceinline__ T mul(T a, T b) { return agl::e2_mul_lazy(a, b); }
    static __device__ __forceinline__ T zero() { return agl::E2{0, 0}; }
    static __device__ __forceinline__ void to_words(T v, uint64_t* w) { w[0] = v.c0; w[1] = v.c1; }
    static __device__ __forceinline__ T from_words(const uint64_t* w) { return T{w[0], w[1]}; }
    // a factor used many times, with its c1 times the non-residue prepared: four products, two reductions
    using Pre = agl::E2Pre;
    static __device__ __forceinline__ Pre pre(T x) { return agl::e2_pre(x); }
    static __device__ __forceinline__ T mul_pre(Pre p, T x) { return agl::e2_fma_pre(p, x, agl::E2{0, 0}); }
    // an exact sum of at most 64 products of 64-bit words, reduced to a loose residue
    static __device__ __forceinline__ uint64_t reduce_acc(const gl::Acc& s) { return agl::acc_reduce(s); }
};

template <>
struct Lazy<AglBase> {
    using A = gl::Acc;
    static __device__ __forceinline__ A zero() { return gl::acc_zero(); }
    static __device__ __forceinline__ void mul(A& s, uint64_t x, uint64_t y) { gl::acc_mul(s, x, y); }
    static __device__ __forceinline__ uint64_t reduce(const A& s) { return agl::acc_reduce(s); }
};
// sum x_k y_k over the extension X^2 = 3 as three exact sums (c0 c0, c1 c1, cross terms)
struct AglE2Acc {
    gl::Acc s00, s11, s01;
};
template <>
struct Lazy<AglExt2> {
    using A = AglE2Acc;
    static __device__ __forceinline__ A zero() { return A{gl::acc_zero(), gl::acc_zero(), gl::acc_zero()}; }
    static __device__ __forceinline__ void mul(A& q, agl::E2 x, agl::E2 y) {
        gl::acc_mul(q.s00, x.c0, y.c0);
        gl::acc_mul(q.s11, x.c1, y.c1);
        gl::acc_mul(q.s01, x.c0, y.c1);
        gl::acc_mul(q.s01, x.c1, y.c0);
    }
    static __device__ __forceinline__ agl::E2 reduce(const A& q) {
        return agl::E2{agl::add(agl::acc_reduce(q.s00), agl::mul_small(agl::acc_reduce(q.s11), 3)), agl::acc_reduce(q.s01)};
    }
};

template <>
struct FoldOp<AglBase, AglExt2> {
    static __device__ __forceinline__ agl::E2 apply(uint64_t a, uint64_t b, agl::E2 r) {
        return agl::e2_fma_pre_base(agl::e2_pre(r), agl::sub(b, a), a);
    }
};
template <>
struct FoldOp<AglExt2, AglExt2> {
    static __device__ __forceinline__ agl::E2 apply(agl::E2 a, agl::E2 b, agl::E2 r) {
        return agl::e2_fma_pre(agl::e2_pre(r), agl::e2_sub(b, a), a);
    }
};

}  // namespace sc
}  // namespace mb
