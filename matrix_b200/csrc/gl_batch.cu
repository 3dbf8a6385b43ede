// C-ABI: element-wise batch operations over Goldilocks and its quadratic
// extension (reference: goldilocks-cuda-rs/src/ffi.rs:31-58,165-285,629-655;
// definitions goldilocks-cuda-rs/cuda/wrapper.cu:100-575,1807-1860,2446-2460).
#include "batch_ops.cuh"
#include "gl_ext5.cuh"
#include "gl_field.cuh"

using namespace mb;
using namespace mb::bo;
MB_FIELD_ADAPTER(GlF, gl);

// Degree-5 extension, five words per element (goldilocks-cuda-rs/src/ffi.rs:229-281;
// definitions goldilocks-cuda-rs/cuda/wrapper.cu:567-860). Addition, subtraction,
// negation and the scalar product act on coefficients, so they run the base-field
// kernels over 5 n words; the Frobenius map scales word i by DTH^(i mod 5).
namespace {

enum E5Op { E5_MUL, E5_SQUARE, E5_INV, E5_EXP };

template <int OP>
__global__ void __launch_bounds__(256)
e5_kernel(const uint64_t* a, const uint64_t* b, uint64_t* r, size_t n, uint64_t e) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        gl::E5 x = gl::e5_load(a + 5 * i), y;
        if (OP == E5_MUL) y = gl::e5_mul(x, gl::e5_load(b + 5 * i));
        else if (OP == E5_SQUARE) y = gl::e5_mul(x, x);
        else if (OP == E5_INV) y = gl::e5_inv(x);
        else y = gl::e5_pow(x, e);
        gl::e5_store(r + 5 * i, y);
    }
}

__global__ void __launch_bounds__(256)
e5_frobenius_kernel(const uint64_t* __restrict__ a, uint64_t* __restrict__ r, size_t words) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += step) {
        const int k = (int)(i % 5);
        r[i] = gl::canon(k ? gl::mul(a[i], MB_E5_DTH(k)) : a[i]);
    }
}

__global__ void __launch_bounds__(256)
e5_lift_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t words) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += step)
        out[i] = (i % 5) ? 0 : gl::canon(in[i / 5]);
}

__global__ void __launch_bounds__(256)
e5_project_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) out[i] = gl::canon(in[5 * i]);
}

template <int OP>
int run_e5(const uint64_t* a, const uint64_t* b, uint64_t* r, int n, uint64_t e = 0) {
    if (n < 0 || !a || !r || (OP == E5_MUL && !b)) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("ext5_batch");
    e5_kernel<OP><<<grid_for((size_t)n, 256, 4), 256, 0, MB_STREAM>>>(a, b, r, (size_t)n, e);
    return finish_async();
}

// coefficient-wise operations: the base-field kernels over 5 n words
template <int OP>
int run_e5_words(const uint64_t* a, const uint64_t* b, uint64_t* r, int n, uint64_t s = 0) {
    constexpr bool binary = OP == ADD || OP == SUB;
    if (n < 0 || !a || !r || (binary && !b)) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    const size_t words = 5 * (size_t)n;
    MB_KERNEL("ext5_batch");
    base_kernel<GlF, OP><<<grid_for(words, 256, 8), 256, 0, MB_STREAM>>>(a, b, r, words, s);
    return finish_async();
}

}  // namespace

extern "C" {

int gl_batch_add(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_base<GlF, ADD>("gl_batch", a, b, r, n); }
int gl_batch_sub(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_base<GlF, SUB>("gl_batch", a, b, r, n); }
int gl_batch_mul(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_base<GlF, MUL>("gl_batch", a, b, r, n); }
int gl_batch_div(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_base<GlF, DIV>("gl_batch", a, b, r, n); }
int gl_batch_inverse(const uint64_t* a, uint64_t* r, int n) { return run_base<GlF, INV>("gl_batch", a, nullptr, r, n); }
int gl_batch_neg(const uint64_t* a, uint64_t* r, int n) { return run_base<GlF, NEG>("gl_batch", a, nullptr, r, n); }
int gl_batch_square(const uint64_t* a, uint64_t* r, int n) { return run_base<GlF, SQUARE>("gl_batch", a, nullptr, r, n); }
int gl_batch_double(const uint64_t* a, uint64_t* r, int n) { return run_base<GlF, DOUBLE>("gl_batch", a, nullptr, r, n); }
int gl_batch_mul_scalar(uint64_t scalar, const uint64_t* a, uint64_t* r, int n) {
    return run_base<GlF, MUL_SCALAR>("gl_batch", a, nullptr, r, n, scalar);
}
int gl_batch_exp(const uint64_t* a, uint64_t exp, uint64_t* r, int n) { return run_base<GlF, EXP>("gl_batch", a, nullptr, r, n, exp); }

int ext2_batch_add_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_ext<GlF, ADD>("ext2_batch", a, b, r, n); }
int ext2_batch_sub_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_ext<GlF, SUB>("ext2_batch", a, b, r, n); }
int ext2_batch_mul_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_ext<GlF, MUL>("ext2_batch", a, b, r, n); }
int ext2_batch_inverse_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<GlF, INV>("ext2_batch", a, nullptr, r, n); }
int ext2_batch_neg_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<GlF, NEG>("ext2_batch", a, nullptr, r, n); }
int ext2_batch_square_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<GlF, SQUARE>("ext2_batch", a, nullptr, r, n); }
int ext2_batch_frobenius_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<GlF, CONJ>("ext2_batch", a, nullptr, r, n); }
int ext2_batch_conjugate_ffi(const uint64_t* a, uint64_t* r, int n) { return run_ext<GlF, CONJ>("ext2_batch", a, nullptr, r, n); }
int ext2_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* a, uint64_t* r, int n) {
    return run_ext<GlF, MUL_SCALAR>("ext2_batch", a, nullptr, r, n, scalar);
}
int ext2_batch_exp_ffi(const uint64_t* a, uint64_t exp, uint64_t* r, int n) { return run_ext<GlF, EXP>("ext2_batch", a, nullptr, r, n, exp); }
// acc[i] += scalar * src[i]
int ext2_scale_accumulate_ffi(uint64_t scalar_c0, uint64_t scalar_c1, const uint64_t* d_src, uint64_t* d_acc, int n) {
    return run_ext<GlF, SCALE_ACC>("ext2_batch", d_src, nullptr, d_acc, n, scalar_c0, scalar_c1);
}

int gl_to_ext2_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n) { return run_lift<GlF>(d_input, d_output, n); }
int ext2_to_gl_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n) { return run_project<GlF>(d_input, d_output, n); }
int ext5_batch_add_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_e5_words<ADD>(a, b, r, n); }
int ext5_batch_sub_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_e5_words<SUB>(a, b, r, n); }
int ext5_batch_neg_ffi(const uint64_t* a, uint64_t* r, int n) { return run_e5_words<NEG>(a, nullptr, r, n); }
int ext5_batch_mul_scalar_ffi(uint64_t scalar, const uint64_t* a, uint64_t* r, int n) {
    return run_e5_words<MUL_SCALAR>(a, nullptr, r, n, scalar);
}
int ext5_batch_mul_ffi(const uint64_t* a, const uint64_t* b, uint64_t* r, int n) { return run_e5<E5_MUL>(a, b, r, n); }
int ext5_batch_square_ffi(const uint64_t* a, uint64_t* r, int n) { return run_e5<E5_SQUARE>(a, nullptr, r, n); }
int ext5_batch_inverse_ffi(const uint64_t* a, uint64_t* r, int n) { return run_e5<E5_INV>(a, nullptr, r, n); }
int ext5_batch_exp_ffi(const uint64_t* a, uint64_t exp, uint64_t* r, int n) { return run_e5<E5_EXP>(a, nullptr, r, n, exp); }
int ext5_batch_frobenius_ffi(const uint64_t* a, uint64_t* r, int n) {
    if (n < 0 || !a || !r) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("ext5_batch");
    e5_frobenius_kernel<<<grid_for(5 * (size_t)n, 256, 8), 256, 0, MB_STREAM>>>(a, r, 5 * (size_t)n);
    return finish_async();
}
int gl_to_ext5_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n) {
    if (n < 0 || !d_input || !d_output) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("lift_to_ext5");
    e5_lift_kernel<<<grid_for(5 * (size_t)n, 256, 8), 256, 0, MB_STREAM>>>(d_input, d_output, 5 * (size_t)n);
    return finish_async();
}
int ext5_to_gl_batch_ffi(const uint64_t* d_input, uint64_t* d_output, int n) {
    if (n < 0 || !d_input || !d_output) return MB_ERR_ARG;
    if (n == 0) return MB_OK;
    MB_KERNEL("ext5_to_base");
    e5_project_kernel<<<grid_for((size_t)n, 256, 8), 256, 0, MB_STREAM>>>(d_input, d_output, (size_t)n);
    return finish_async();
}
int gl_zero_buffer(uint64_t* d_buf, int n) { return n < 0 ? MB_ERR_ARG : run_zero(d_buf, (size_t)n); }
int bit_permute_gl_ffi(const uint64_t* d_input, uint64_t* d_output, const int* d_perm_map, int n_bits, int total) {
    return run_bit_permute(d_input, d_output, d_perm_map, n_bits, total);
}

}  // extern "C"
