// Entry points of the reference's FFI that lie outside the prover's field-arithmetic path (Morpheus protocol layers, model operators, a tensor-core probe, profiler range markers):
// exported so that the Rust crates link against this library unchanged. Each returns -3 (unsupported)
// whatever it is given and touches nothing; the profiler range markers are no-ops.
#include "common.cuh"

extern "C" {

int agl_morpheus_gauss_words(...) { return MB_ERR_UNSUPPORTED; }
int agl_morpheus_gauss_dev(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_wtable(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_ev(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_decode(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_combine_multi(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_combine(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_norm(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_pack37(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_unpack37(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink_phase1(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink_fold(...) { return MB_ERR_UNSUPPORTED; }
int agl_morpheus_coins(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_consts(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_round(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_range_bin1(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_coarse_init(...) { return MB_ERR_UNSUPPORTED; }
int agl_i64_to_i32(...) { return MB_ERR_UNSUPPORTED; }
int agl_add_i32_i64(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_coarse_init2(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_b_build(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_b_halve(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_dense_expand(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_coarse_round(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_coarse_fold(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_onehot3(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_onehot_pre(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_onehot_bin(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_rep_reduce(...) { return MB_ERR_UNSUPPORTED; }
int agl_morpheus_permute(...) { return MB_ERR_UNSUPPORTED; }
int agl_morpheus_unpack2(...) { return MB_ERR_UNSUPPORTED; }
int agl_morpheus_permute2(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_ev_packed_batch(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_combine_tc(...) { return MB_ERR_UNSUPPORTED; }
int agl_mauth_combine_packed(...) { return MB_ERR_UNSUPPORTED; }
int agl_gauss_low_priority(...) { return MB_ERR_UNSUPPORTED; }
int agl_mlink2_index(...) { return MB_ERR_UNSUPPORTED; }
int agl_morpheus_gauss_scatter(...) { return MB_ERR_UNSUPPORTED; }
void agl_nvtx_push(...) {}
void agl_nvtx_pop(...) {}
int ajtai_tc_commit_probe_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_einsum2_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_einsum1_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_relu_helper_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_conv2d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_flatten_kernel2d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_conv3d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_flatten_kernel3d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_depthwise_conv2d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_conv_transpose2d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_conv_transpose3d_ffi(...) { return MB_ERR_UNSUPPORTED; }
int agl_conv_full_ffi(...) { return MB_ERR_UNSUPPORTED; }

}  // extern "C"
