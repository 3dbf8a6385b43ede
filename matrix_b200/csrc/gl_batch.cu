// C-ABI: element-wise batch operations over Goldilocks and its quadratic
// extension (reference: goldilocks-cuda-rs/src/ffi.rs:31-58,165-285,629-655;
// definitions goldilocks-cuda-rs/cuda/wrapper.cu:100-575,1807-1860,2446-2460).
#include "batch_ops.cuh"
#include "gl_field.cuh"

using namespace mb;
using namespace mb::bo;
MB_FIELD_ADAPTER(GlF, gl);

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
int gl_zero_buffer(uint64_t* d_buf, int n) { return n < 0 ? MB_ERR_ARG : run_zero(d_buf, (size_t)n); }
int bit_permute_gl_ffi(const uint64_t* d_input, uint64_t* d_output, const int* d_perm_map, int n_bits, int total) {
    return run_bit_permute(d_input, d_output, d_perm_map, n_bits, total);
}

}  // extern "C"
