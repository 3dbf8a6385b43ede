// C-ABI: folding of Ajtai witnesses and commitments (reference declarations
// almost-goldilocks-cuda-rs/src/ffi.rs:435-492,635-647; definitions
// almost-goldilocks-cuda-rs/cuda/wrapper.cu:1468-1629,1717-1739).
#include "ajtai_fold_tc.cuh"
#include "ajtai_kernels.cuh"

using namespace mb;
using namespace mb::aj;

namespace {

bool valid_chunk(int chunk) { return chunk == 64 || chunk == 128 || chunk == 256 || chunk == 1024 || chunk == 4096; }

// 64 host coefficients to a device scratch (freed by the caller with pool_free).
int upload_challenge(const int8_t* h_r, int8_t** d_r) {
    if (pool_alloc((void**)d_r, 64) != cudaSuccess) return MB_ERR_CUDA;
    if (cudaMemcpyAsync(*d_r, h_r, 64, cudaMemcpyHostToDevice, MB_STREAM) != cudaSuccess) return MB_ERR_CUDA;
    return cudaStreamSynchronize(MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;  // h_r is the caller's
}

int multifold_scalar(const uint64_t* zbin, const uint64_t* pos, const uint64_t* neg, const int8_t* d_r, int16_t* d_out, int nb, int nt,
                     uint64_t N) {
    MB_KERNEL("ajtai_multifold_scalar");
    const int grid = (int)(N < (uint64_t)sm_count() * 16 ? N : (uint64_t)sm_count() * 16);
    multifold_witness_scalar_kernel<true><<<grid, 64, (size_t)(nb + nt) * 64, MB_STREAM>>>(nullptr, zbin, pos, neg, d_r, d_out, nb, nt, N);
    return finish_async();
}

// The tensor-core path; any number of instances (stages of eight), any N.
int multifold_tc(const uint64_t* zbin, const uint64_t* pos, const uint64_t* neg, const int8_t* d_r, int16_t* d_out, int nb, int nt,
                 uint64_t N) {
    const int total = nb + nt, stages = (total + MF_INST - 1) / MF_INST;
    int8_t* Bg = nullptr;
    int* d_err = nullptr;
    MB_CUDA(pool_alloc((void**)&Bg, (size_t)stages * MF_B_BYTES));
    if (pool_alloc((void**)&d_err, sizeof(int)) != cudaSuccess) { pool_free(Bg); return MB_ERR_CUDA; }
    int rc = cudaMemsetAsync(d_err, 0, sizeof(int), MB_STREAM) == cudaSuccess ? MB_OK : MB_ERR_CUDA;
    const size_t smem = MF_A_BYTES + MF_B_BYTES;
    if (rc == MB_OK && cudaFuncSetAttribute(multifold_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        rc = MB_ERR_CUDA;
    if (rc == MB_OK) {
        {
            MB_KERNEL("ajtai_multifold_prepare");
            multifold_prepare_b_kernel<<<grid_for((size_t)stages * MF_B_BYTES, 256, 4), 256, 0, MB_STREAM>>>(d_r, total, stages, Bg);
        }
        {
            MB_KERNEL("ajtai_multifold_tc");
            const uint64_t tiles = (N + 127) / 128;
            const int grid = (int)(tiles < (uint64_t)sm_count() * 2 ? tiles : (uint64_t)sm_count() * 2);
            multifold_tc_kernel<<<grid, MF_THREADS, smem, MB_STREAM>>>(zbin, pos, neg, Bg, d_out, nb, nt, N, d_err);
        }
        rc = finish_async();
    }
    int h_err = 0;
    if (rc == MB_OK && cudaMemcpyAsync(&h_err, d_err, sizeof(int), cudaMemcpyDeviceToHost, MB_STREAM) != cudaSuccess) rc = MB_ERR_CUDA;
    if (rc == MB_OK) rc = finish_sync();
    pool_free(Bg);
    pool_free(d_err);
    if (rc == MB_OK && h_err != 0) rc = MB_ERR_CUDA;  // a bounded wait gave up
    return rc;
}

int multifold(const uint64_t* zbin, const uint64_t* pos, const uint64_t* neg, const int8_t* d_r, int16_t* d_out, int nb, int nt,
              uint64_t N, bool scalar) {
    if (nb < 0 || nt < 0 || nb + nt < 1 || nb + nt > 512 || !d_r || !d_out || (nb && !zbin) || (nt && (!pos || !neg))) return MB_ERR_ARG;
    if (N == 0) return MB_OK;
    return scalar ? multifold_scalar(zbin, pos, neg, d_r, d_out, nb, nt, N) : multifold_tc(zbin, pos, neg, d_r, d_out, nb, nt, N);
}

}  // namespace

extern "C" {

// d_out[N_ring][64] = z1 + r * z2 as canonical field elements; z1, z2 binary masks; r_coeffs: 64 host coefficients.
int ajtai_fold_witness_ffi(const uint64_t* d_z1, const uint64_t* d_z2, const int8_t* r_coeffs, uint64_t N_ring, int chunk,
                           uint64_t* d_out) {
    if (!valid_chunk(chunk)) return MB_ERR_UNSUPPORTED;
    if (!d_z1 || !d_z2 || !r_coeffs || !d_out) return MB_ERR_ARG;
    if (N_ring == 0) return MB_OK;
    int8_t* d_r = nullptr;
    int rc = upload_challenge(r_coeffs, &d_r);
    if (rc == MB_OK) {
        MB_KERNEL("ajtai_fold_witness");
        const int grid = (int)(N_ring < (uint64_t)sm_count() * 16 ? N_ring : (uint64_t)sm_count() * 16);
        multifold_witness_scalar_kernel<false><<<grid, 64, 64, MB_STREAM>>>(d_z1, d_z2, nullptr, nullptr, d_r, d_out, 1, 0, N_ring);
        rc = finish_async();
    }
    pool_free(d_r);
    return rc;
}

// d_out[42][64] = c1 + r * c2
int ajtai_fold_commitment_ffi(const uint64_t* d_c1, const uint64_t* d_c2, const int8_t* r_coeffs, uint64_t* d_out) {
    if (!d_c1 || !d_c2 || !r_coeffs || !d_out) return MB_ERR_ARG;
    int8_t* d_r = nullptr;
    int rc = upload_challenge(r_coeffs, &d_r);
    if (rc == MB_OK) {
        MB_KERNEL("ajtai_fold_commitment");
        multifold_commitment_kernel<<<KAPPA, 64, 64, MB_STREAM>>>(d_c1, d_c2, d_r, 1, d_out);
        rc = finish_async();
    }
    pool_free(d_r);
    return rc;
}

// d_out[42][64] = sum_m r_m * c_m; d_c_packed[m][42][64], d_r_all[m][64] on the device.
int ajtai_multifold_commitment_ffi(const uint64_t* d_c_packed, const int8_t* d_r_all, int num_instances, uint64_t* d_out) {
    if (!d_c_packed || !d_r_all || !d_out || num_instances < 1 || num_instances > 512) return MB_ERR_ARG;
    MB_KERNEL("ajtai_multifold_commitment");
    multifold_commitment_kernel<<<KAPPA, 64, (size_t)num_instances * 64, MB_STREAM>>>(nullptr, d_c_packed, d_r_all, num_instances, d_out);
    return finish_async();
}

// d_out[N_ring][64] (16-bit) = sum_i r_i * z_i; z_i binary masks d_z_packed[i * N_ring + j]. chunk_size is the
// reference's tuning knob and is ignored.
int ajtai_multifold_witness_ffi(const uint64_t* d_z_packed, const int8_t* d_r_all, int16_t* d_out, int num_instances, uint64_t N_ring,
                                uint64_t chunk_size) {
    (void)chunk_size;
    return multifold(d_z_packed, nullptr, nullptr, d_r_all, d_out, num_instances, 0, N_ring, false);
}
// num_binary masks, then num_ternary (pos, neg) pairs; challenges in that order.
int ajtai_multifold_mixed_witness_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed, const uint64_t* d_neg_packed,
                                      const int8_t* d_r_all, int16_t* d_out, int num_binary, int num_ternary, uint64_t N_ring,
                                      uint64_t chunk_size) {
    (void)chunk_size;
    return multifold(d_z_bin_packed, d_pos_packed, d_neg_packed, d_r_all, d_out, num_binary, num_ternary, N_ring, false);
}
// The reference's tensor-core variants: the same computation (one path here).
int ajtai_multifold_mixed_witness_tc_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed, const uint64_t* d_neg_packed,
                                         const int8_t* d_r_all, int16_t* d_out, int num_binary, int num_ternary, uint64_t N_ring) {
    return multifold(d_z_bin_packed, d_pos_packed, d_neg_packed, d_r_all, d_out, num_binary, num_ternary, N_ring, false);
}
int ajtai_multifold_mixed_witness_tc_fused_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed,
                                               const uint64_t* d_neg_packed, const int8_t* d_r_all, int16_t* d_out, int num_binary,
                                               int num_ternary, uint64_t N_ring) {
    return multifold(d_z_bin_packed, d_pos_packed, d_neg_packed, d_r_all, d_out, num_binary, num_ternary, N_ring, false);
}
// Addition: the scalar form of the same fold (one thread per coefficient), kept as an independent check.
int ajtai_multifold_mixed_witness_scalar_ffi(const uint64_t* d_z_bin_packed, const uint64_t* d_pos_packed,
                                             const uint64_t* d_neg_packed, const int8_t* d_r_all, int16_t* d_out, int num_binary,
                                             int num_ternary, uint64_t N_ring) {
    return multifold(d_z_bin_packed, d_pos_packed, d_neg_packed, d_r_all, d_out, num_binary, num_ternary, N_ring, true);
}

// 16-bit coefficients to 13 ternary planes (bits of |v| above the 13th are dropped, as in the reference).
int ajtai_split_witness_ffi(const int16_t* d_z_wide, uint64_t* d_pos_chunks, uint64_t* d_neg_chunks, uint64_t N_ring) {
    if (!d_z_wide || !d_pos_chunks || !d_neg_chunks) return MB_ERR_ARG;
    if (N_ring == 0) return MB_OK;
    int* d_err = nullptr;
    MB_CUDA(pool_alloc((void**)&d_err, sizeof(int)));
    {
        MB_KERNEL("ajtai_split_witness");
        wide_to_ternary_kernel<<<grid_for(N_ring, 128, 8), 128, 0, MB_STREAM>>>(d_z_wide, d_pos_chunks, d_neg_chunks, d_err, N_ring, 13);
    }
    int rc = finish_async();
    pool_free(d_err);
    return rc;
}

}  // extern "C"
