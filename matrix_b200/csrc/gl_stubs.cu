// Entry points of the reference's FFI that lie outside the prover's field-arithmetic path (model operators: einsum, convolution, scaling and bit-decomposition helpers):
// exported so that the Rust crates link against this library unchanged. Each returns -3 (unsupported)
// whatever it is given and touches nothing; the profiler range markers are no-ops.
#include "common.cuh"

extern "C" {

int gl_einsum2(...) { return MB_ERR_UNSUPPORTED; }
int gl_einsum1(...) { return MB_ERR_UNSUPPORTED; }
int gl_scale_down(...) { return MB_ERR_UNSUPPORTED; }
int gl_scale_up(...) { return MB_ERR_UNSUPPORTED; }
int gl_decompose_bits32(...) { return MB_ERR_UNSUPPORTED; }
int gl_conv2d(...) { return MB_ERR_UNSUPPORTED; }
int gl_flatten_kernel2d(...) { return MB_ERR_UNSUPPORTED; }
int gl_relu_helper(...) { return MB_ERR_UNSUPPORTED; }
int gl_conv3d(...) { return MB_ERR_UNSUPPORTED; }
int gl_flatten_kernel3d(...) { return MB_ERR_UNSUPPORTED; }
int gl_depthwise_conv2d(...) { return MB_ERR_UNSUPPORTED; }

}  // extern "C"
