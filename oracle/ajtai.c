/*
 * CPU oracle (test infrastructure, not the product): Ajtai ring commitment over
 * almost-Goldilocks, R = F_q[X]/(X^64 + 1), KAPPA = 42 ring rows.
 *
 * Restates cuda_almost_goldilocks/ajtai_chacha8.cuh:60-178 (ChaCha8 block and
 * the rejection-sampled ring block), ajtai_cpu_reference.cuh:65-186 (negacyclic
 * products and the commit loop) and the device layout of
 * cuda_almost_goldilocks/ajtai.cuh:94-161 (dense planes z[b*N + j], output
 * [b][i][r], col_offset shifting j in the PRG only). Pinned against the
 * reference's own CPU code compiled into oracle/_ref/libajtai_ref.so.
 */
#include "agl.h"
#include <stdlib.h>
#include <string.h>

#define AJ_D 64
#define AJ_KAPPA 42

#define ROTL32(x, n) (((x) << (n)) | ((x) >> (32 - (n))))
#define QR(a, b, c, d) do { a += b; d ^= a; d = ROTL32(d, 16); c += d; b ^= c; b = ROTL32(b, 12); \
                            a += b; d ^= a; d = ROTL32(d, 8);  c += d; b ^= c; b = ROTL32(b, 7); } while (0)

void oracle_chacha8_block(const uint32_t key[8], uint32_t counter, const uint32_t nonce[3], uint32_t out[16]) {
    uint32_t s[16] = { 0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, key[0], key[1], key[2], key[3],
                       key[4], key[5], key[6], key[7], counter, nonce[0], nonce[1], nonce[2] };
    uint32_t x[16];
    memcpy(x, s, sizeof(x));
    for (int dr = 0; dr < 4; dr++) {
        QR(x[0], x[4], x[8], x[12]); QR(x[1], x[5], x[9], x[13]); QR(x[2], x[6], x[10], x[14]); QR(x[3], x[7], x[11], x[15]);
        QR(x[0], x[5], x[10], x[15]); QR(x[1], x[6], x[11], x[12]); QR(x[2], x[7], x[8], x[13]); QR(x[3], x[4], x[9], x[14]);
    }
    for (int i = 0; i < 16; i++) out[i] = x[i] + s[i];
}

/* 8 coefficients: words of blocks counter = block_idx, block_idx + 8, ... below q, first 8 kept (<= 16 blocks). */
static void prg_ring_block(const uint32_t key[8], uint32_t row, uint64_t j, uint32_t block_idx, uint64_t out[8]) {
    uint32_t nonce[3] = { row, (uint32_t)j, (uint32_t)(j >> 32) };
    int written = 0;
    memset(out, 0, 64);
    for (uint32_t retry = 0; retry < 16 && written < 8; retry++) {
        uint32_t buf[16];
        oracle_chacha8_block(key, block_idx + 8u * retry, nonce, buf);
        for (int k = 0; k < 8 && written < 8; k++) {
            uint64_t v = ((uint64_t)buf[2 * k + 1] << 32) | buf[2 * k];
            if (v < AGL_Q) out[written++] = v;
        }
    }
}

void oracle_ajtai_ring_elem(const uint32_t key[8], uint32_t row, uint64_t j, uint64_t out[AJ_D]) {
    for (uint32_t b = 0; b < AJ_D / 8; b++) prg_ring_block(key, row, j, b, out + 8 * b);
}

/* acc += m * z in R for field-valued z (negacyclic schoolbook, ajtai_cpu_reference.cuh:85-101) */
static void ring_mul_acc(uint64_t acc[AJ_D], const uint64_t m[AJ_D], const uint64_t z[AJ_D]) {
    for (int l = 0; l < AJ_D; l++) {
        if (z[l] == 0) continue;
        for (int k = 0; k < AJ_D; k++) {
            uint64_t v = agl_mul(m[k], z[l]);
            int r = k + l;
            if (r < AJ_D) acc[r] = agl_add(acc[r], v);
            else acc[r - AJ_D] = agl_sub(acc[r - AJ_D], v);
        }
    }
}

/*
 * General commit: planes of witnesses, out[p][i][r] = sum_j M[i][col_offset + j] * z_p[j].
 * kind 0: z = u64 bit masks, z[p*N + j], bit l = coefficient l (dense binary planes)
 * kind 1: z = int8 digits, z[(p*N + j)*64 + l] (signed small coefficients)
 * kind 2: z = u64 field coefficients, z[(p*N + j)*64 + l] (wide)
 */
void oracle_ajtai_commit(const uint32_t key[8], const void *z, int kind, uint64_t N, int planes, uint64_t col_offset,
                         uint64_t *out) {
    memset(out, 0, sizeof(uint64_t) * (size_t)planes * AJ_KAPPA * AJ_D);
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < AJ_KAPPA; i++) {
        uint64_t m[AJ_D], zc[AJ_D];
        for (uint64_t j = 0; j < N; j++) {
            oracle_ajtai_ring_elem(key, (uint32_t)i, col_offset + j, m);
            for (int p = 0; p < planes; p++) {
                if (kind == 0) {
                    uint64_t bits = ((const uint64_t *)z)[(size_t)p * N + j];
                    if (!bits) continue;
                    for (int l = 0; l < AJ_D; l++) zc[l] = (bits >> l) & 1;
                } else if (kind == 1) {
                    const int8_t *d = (const int8_t *)z + ((size_t)p * N + j) * AJ_D;
                    for (int l = 0; l < AJ_D; l++) zc[l] = d[l] >= 0 ? (uint64_t)d[l] : AGL_Q - (uint64_t)(-(int)d[l]);
                } else {
                    const uint64_t *w = (const uint64_t *)z + ((size_t)p * N + j) * AJ_D;
                    for (int l = 0; l < AJ_D; l++) zc[l] = agl_canon(w[l]);
                }
                ring_mul_acc(out + ((size_t)p * AJ_KAPPA + i) * AJ_D, m, zc);
            }
        }
    }
}

/* Sparse commit (ajtai_cpu_reference.cuh:192-219): position p = 64 j + l contributes X^l M[i][j]. */
void oracle_ajtai_commit_sparse(const uint32_t key[8], const uint64_t *positions, uint64_t K, uint64_t *out) {
    memset(out, 0, sizeof(uint64_t) * AJ_KAPPA * AJ_D);
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < AJ_KAPPA; i++) {
        uint64_t m[AJ_D];
        uint64_t have = ~0ULL;
        for (uint64_t k = 0; k < K; k++) {
            uint64_t j = positions[k] >> 6;
            int l = (int)(positions[k] & 63);
            if (j != have) { oracle_ajtai_ring_elem(key, (uint32_t)i, j, m); have = j; }
            uint64_t *c = out + (size_t)i * AJ_D;
            for (int r = 0; r < AJ_D; r++) {
                uint64_t v = m[(r - l) & 63];
                c[r] = r >= l ? agl_add(c[r], v) : agl_sub(c[r], v);
            }
        }
    }
}

