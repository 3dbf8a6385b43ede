// C-ABI entry points of the Goldilocks sumcheck path.
//
// Drop-in for the reference's sumcheck exports (declarations
// goldilocks-cuda-rs/src/ffi.rs:588-627, definitions
// goldilocks-cuda-rs/cuda/wrapper.cu:1716-1785), plus the fused fold+message
// entry points this library adds. Declarations: include/goldilocks_cuda_wrapper.h.
#include "sumcheck_kernels.cuh"
#include "gl_sumcheck_launch.cuh"

using namespace mb;
using namespace mb::sc;

extern "C" {

int sumcheck_round_message_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                               size_t half, int num_blocks) {
    int rc = launch_round_message<GlBase>(d_polys, d_partial, d, original_size, half, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

int sumcheck_fold_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge, int d,
                      size_t original_size, size_t half) {
    int rc = launch_fold<GlBase>(d_input, d_output, gl::canon(challenge), d, original_size, half, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

int sumcheck_round_message_ext2_ffi(const uint64_t* d_polys, uint64_t* d_partial, int d, size_t original_size,
                                    size_t half, int num_blocks) {
    int rc = launch_round_message<GlExt2>(d_polys, d_partial, d, original_size, half, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

int sumcheck_fold_ext2_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                           uint64_t challenge_c1, int d, size_t original_size, size_t half) {
    gl::E2 r{gl::canon(challenge_c0), gl::canon(challenge_c1)};
    int rc = launch_fold<GlExt2>(d_input, d_output, r, d, original_size, half, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// ---- additions: fold on the challenge fused with the next round's message ----

// Extension tables in, extension tables out. `quarter` = (live length)/4 is the
// number of pairs of the folded table; partials land as
// d_partial[(block*(d+1) + c)*2 + {0,1}] for block < num_blocks.
int sumcheck_fold_round_ext2_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                                 uint64_t challenge_c1, int d, size_t original_size, size_t quarter,
                                 uint64_t* d_partial, int num_blocks) {
    gl::E2 r{gl::canon(challenge_c0), gl::canon(challenge_c1)};
    int rc = launch_fold_message<GlExt2, GlExt2>(d_input, d_output, r, nullptr, d, original_size, original_size,
                                                 quarter, d_partial, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// Base-field tables in (stride original_size u64), extension tables out
// (stride original_size extension elements).
int sumcheck_fold_round_mixed_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                                  uint64_t challenge_c1, int d, size_t original_size, size_t quarter,
                                  uint64_t* d_partial, int num_blocks) {
    gl::E2 r{gl::canon(challenge_c0), gl::canon(challenge_c1)};
    int rc = launch_fold_message<GlBase, GlExt2>(d_input, d_output, r, nullptr, d, original_size, original_size,
                                                 quarter, d_partial, num_blocks, MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

// Base-field tables in, extension tables out, no message (used when only two
// live elements per table remain).
int sumcheck_fold_mixed_ffi(const uint64_t* d_input, uint64_t* d_output, uint64_t challenge_c0,
                            uint64_t challenge_c1, int d, size_t original_size, size_t half) {
    gl::E2 r{gl::canon(challenge_c0), gl::canon(challenge_c1)};
    int rc = launch_fold_lift<GlBase, GlExt2>(d_input, d_output, r, nullptr, d, original_size, original_size, half,
                                              MB_STREAM);
    return rc != MB_OK ? rc : finish_sync();
}

}  // extern "C"
