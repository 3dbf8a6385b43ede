// Microbenchmark of the Goldilocks arithmetic primitives: one kernel per variant, every thread runs the
// primitive 1024 times on changing operands. Run plain for times, under ncu
// (smsp__inst_executed.sum, sm__inst_executed_pipe_alu.sum, sm__inst_executed_pipe_fmaheavy.sum) for the
// instruction count per call; variant 8 is the loop and operand update alone.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I.. -o gl_arith_microbench gl_arith_microbench.cu
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "gl_field.cuh"
using namespace gl;

struct A5 { uint32_t a0, a1, a2, a3, a4; };
struct AccOld { uint64_t lo, hi; uint32_t top; };
__device__ __forceinline__ void old_add128(AccOld& s, uint64_t lo, uint64_t hi) { asm("add.cc.u64 %0, %0, %3;\n\taddc.cc.u64 %1, %1, %4;\n\taddc.u32 %2, %2, 0;" : "+l"(s.lo), "+l"(s.hi), "+r"(s.top) : "l"(lo), "l"(hi)); }

__device__ __forceinline__ void v3_acc(A5& s, uint64_t x, uint64_t y) {
    uint32_t x0 = lo32(x), x1 = hi32(x), y0 = lo32(y), y1 = hi32(y);
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
        : "r"(x0), "r"(x1), "r"(y0), "r"(y1));
}
__device__ __forceinline__ void v2_acc(AccOld& s, uint64_t x, uint64_t y) {
    asm("mad.lo.cc.u64 %0, %3, %4, %0;\n\tmadc.hi.cc.u64 %1, %3, %4, %1;\n\taddc.u32 %2, %2, 0;"
        : "+l"(s.lo), "+l"(s.hi), "+r"(s.top) : "l"(x), "l"(y));
}
__device__ __forceinline__ void v1_acc(AccOld& s, uint64_t x, uint64_t y) {
    old_add128(s, x * y, __umul64hi(x, y));
}
// even/odd: wide products, 32-bit add chains
__device__ __forceinline__ void v4_acc(A5& s, uint64_t x, uint64_t y) {
    uint32_t x0 = lo32(x), x1 = hi32(x), y0 = lo32(y), y1 = hi32(y);
    uint64_t p00, p11, p01, p10;
    asm("mul.wide.u32 %0, %4, %6;\n\tmul.wide.u32 %1, %5, %7;\n\tmul.wide.u32 %2, %4, %7;\n\tmul.wide.u32 %3, %5, %6;"
        : "=l"(p00), "=l"(p11), "=l"(p01), "=l"(p10) : "r"(x0), "r"(x1), "r"(y0), "r"(y1));
    uint32_t e0 = lo32(p00), e1 = hi32(p00), e2 = lo32(p11), e3 = hi32(p11);
    uint32_t o1 = lo32(p01), o2 = hi32(p01), q1 = lo32(p10), q2 = hi32(p10);
    asm("add.cc.u32 %0, %0, %5;\n\taddc.cc.u32 %1, %1, %6;\n\taddc.cc.u32 %2, %2, %7;\n\taddc.cc.u32 %3, %3, %8;\n\taddc.u32 %4, %4, 0;\n\t"
        "add.cc.u32 %1, %1, %9;\n\taddc.cc.u32 %2, %2, %10;\n\taddc.cc.u32 %3, %3, 0;\n\taddc.u32 %4, %4, 0;\n\t"
        "add.cc.u32 %1, %1, %11;\n\taddc.cc.u32 %2, %2, %12;\n\taddc.cc.u32 %3, %3, 0;\n\taddc.u32 %4, %4, 0;"
        : "+r"(s.a0), "+r"(s.a1), "+r"(s.a2), "+r"(s.a3), "+r"(s.a4)
        : "r"(e0), "r"(e1), "r"(e2), "r"(e3), "r"(o1), "r"(o2), "r"(q1), "r"(q2));
}

template <int V>
__global__ void kern(const uint64_t* in, uint64_t* out, int iters) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t x = in[2 * t], y = in[2 * t + 1];
    Acc sn = acc_zero();
    AccOld s = {0, 0, 0};
    A5 s5 = {0, 0, 0, 0, 0};
    uint64_t r = 0;
#pragma unroll 4
    for (int i = 0; i < iters; i++) {
        if (V == 0) acc_mul(sn, x, y);
        else if (V == 1) v1_acc(s, x, y);
        else if (V == 2) v2_acc(s, x, y);
        else if (V == 3) v3_acc(s5, x, y);
        else if (V == 4) v4_acc(s5, x, y);
        else if (V == 5) r = add(r, mul(x, y));                       // reduce every product
        else if (V == 6) { uint64_t lo, hi; mul128(x, y, lo, hi); r = add(r, reduce128(lo, hi)); }
        else if (V == 7) r = mul_add(x, y, r);
        else if (V == 8) r += x;                                       // baseline: the perturbation alone
        else if (V == 9) r = add(r, x);                                // modular add
        else if (V == 10) r = sub(r, x);
        else if (V == 11) r = canon(r + x);
        else if (V == 12) r = sub_canon(canon(r), canon(x));
        else if (V == 13) r = add_c(r, x);
        else if (V == 14) { uint64_t lo, hi; mul128(x, y, lo, hi); r ^= lo ^ hi; }
        else if (V == 15) { r ^= (x * y) ^ __umul64hi(x, y); }
        else if (V == 16) { r ^= reduce128(x, y); }
        else if (V == 17) { r ^= acc_reduce(Acc{lo32(x), hi32(x), lo32(y), hi32(y), (uint32_t)i & 7}); }
        else if (V == 18) { E2 q = e2_mul(E2{x, y}, E2{y, r}); r ^= q.c0 ^ q.c1; }
        else if (V == 19) { E2 q = e2_mul_lazy(E2{x, y}, E2{y, r}); r ^= q.c0 ^ q.c1; }
        else if (V == 20) { r ^= sqr(x); }
        x += 0x9E3779B97F4A7C15ULL;                                    // perturbation (2 instr)
        y ^= x;
    }
    out[t] = r ^ s.lo ^ s.hi ^ s.top ^ sn.a0 ^ sn.a1 ^ sn.a2 ^ sn.a3 ^ sn.a4 ^ s5.a0 ^ s5.a1 ^ s5.a2 ^ s5.a3 ^ s5.a4 ^ x ^ y;
}

int main() {
    const int threads = 148 * 256 * 8, iters = 1024;
    uint64_t *in, *out;
    cudaMalloc(&in, 16 * (size_t)threads);
    cudaMalloc(&out, 8 * (size_t)threads);
    cudaMemset(in, 0x5a, 16 * (size_t)threads);
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
#define RUN(V) { kern<V><<<threads / 256, 256>>>(in, out, iters); cudaEventRecord(a); kern<V><<<threads / 256, 256>>>(in, out, iters); cudaEventRecord(b); cudaEventSynchronize(b); float ms; cudaEventElapsedTime(&ms, a, b); printf("V%d %.3f ms  %.2f cycles/iter/warp-slot\n", V, ms, ms * 1e-3 * 1.965e9 * 148 * 4 / ((double)threads / 32 * iters)); }
    RUN(0) RUN(1) RUN(2) RUN(3) RUN(4) RUN(5) RUN(6) RUN(7) RUN(8) RUN(9) RUN(10) RUN(11) RUN(12) RUN(13) RUN(14) RUN(15) RUN(16) RUN(17) RUN(18) RUN(19) RUN(20)
    printf("%s\n", cudaGetErrorString(cudaDeviceSynchronize()));
    return 0;
}
