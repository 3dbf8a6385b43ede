/* CPU ORACLE (test infrastructure, never shipped or timed as the product):
 * the module commitment over R = F_q[Y]/(Y^4096 + 1), q = 2^64 - 2^32 - 31.
 *
 *   key element (kind, row, col): 512 blocks of 8 coefficients, block b = the first 64
 *     bytes of SHAKE256("MORPHEUS/KEY/SHAKE256/v2\0" || seed || counter || nonce) read as
 *     eight little-endian u64, values >= q rejected, up to 16 blocks with counters
 *     b + 512 retry, zero fill          zk-torch-4/src/morpheus/keys.rs:48-93
 *   commitment  C[row] = sum_c key[row][col_c] * x_c + err[row]  with the key centred
 *     and the products taken as integer negacyclic convolutions, reduced mod q at the
 *     end                                zk-torch-4/src/morpheus/commit.rs:48-83
 *     (the reference's own test pins this against schoolbook products, commit.rs:92-131;
 *      its transform/CRT route, ring.rs, is one way to obtain the same integers)
 *
 * Pins: the SHAKE block is checked against the reference's known answer
 * (keys.rs:133-135) and against Python's hashlib in tests/test_mcommit.py.
 * SHAKE256 is FIPS 202 (sha3 0.10.9 in the reference's lock file), restated here.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MC_N 4096
static const uint64_t MC_Q = 0xFFFFFFFEFFFFFFE1ULL;

static uint64_t rol(uint64_t x, int s) { return s ? (x << s) | (x >> (64 - s)) : x; }

static void keccak_f(uint64_t A[25]) {
    static const uint64_t RC[24] = {
        0x0000000000000001ULL, 0x0000000000008082ULL, 0x800000000000808aULL, 0x8000000080008000ULL, 0x000000000000808bULL,
        0x0000000080000001ULL, 0x8000000080008081ULL, 0x8000000000008009ULL, 0x000000000000008aULL, 0x0000000000000088ULL,
        0x0000000080008009ULL, 0x000000008000000aULL, 0x000000008000808bULL, 0x800000000000008bULL, 0x8000000000008089ULL,
        0x8000000000008003ULL, 0x8000000000008002ULL, 0x8000000000000080ULL, 0x000000000000800aULL, 0x800000008000000aULL,
        0x8000000080008081ULL, 0x8000000000008080ULL, 0x0000000080000001ULL, 0x8000000080008008ULL};
    for (int round = 0; round < 24; round++) {
        uint64_t C[5], B[25];
        for (int x = 0; x < 5; x++) C[x] = A[x] ^ A[x + 5] ^ A[x + 10] ^ A[x + 15] ^ A[x + 20];
        for (int x = 0; x < 5; x++) {
            uint64_t D = C[(x + 4) % 5] ^ rol(C[(x + 1) % 5], 1);
            for (int y = 0; y < 5; y++) A[x + 5 * y] ^= D;
        }
        /* rho offsets by walking (x, y) -> (y, 2x + 3y) from (1, 0): offset (t+1)(t+2)/2 */
        B[0] = A[0];
        int x = 1, y = 0;
        for (int t = 0; t < 24; t++) {
            int nx = y, ny = (2 * x + 3 * y) % 5;
            B[nx + 5 * ny] = rol(A[x + 5 * y], ((t + 1) * (t + 2) / 2) % 64);
            x = nx;
            y = ny;
        }
        for (int yy = 0; yy < 5; yy++)
            for (int xx = 0; xx < 5; xx++) A[xx + 5 * yy] = B[xx + 5 * yy] ^ (~B[(xx + 1) % 5 + 5 * yy] & B[(xx + 2) % 5 + 5 * yy]);
        A[0] ^= RC[round];
    }
}

/* SHAKE256 of a message shorter than one 136-byte block, first `outlen` <= 136 bytes. */
static void shake256_short(const uint8_t* msg, size_t len, uint8_t* out, size_t outlen) {
    uint8_t block[200];
    memset(block, 0, sizeof block);
    memcpy(block, msg, len);
    block[len] ^= 0x1f;
    block[135] ^= 0x80;
    uint64_t A[25];
    for (int i = 0; i < 25; i++) {
        A[i] = 0;
        for (int b = 0; b < 8; b++) A[i] |= (uint64_t)block[8 * i + b] << (8 * b);
    }
    keccak_f(A);
    for (size_t i = 0; i < outlen; i++) out[i] = (uint8_t)(A[i / 8] >> (8 * (i % 8)));
}

void oracle_shake256_short(const uint8_t* msg, size_t len, uint8_t* out, size_t outlen) { shake256_short(msg, len, out, outlen); }

/* keys.rs:48-59 */
void oracle_mcommit_shake_block(const uint32_t seed[8], uint32_t counter, const uint32_t nonce[3], uint32_t out[16]) {
    static const char tag[] = "MORPHEUS/KEY/SHAKE256/v2"; /* sizeof counts the terminator */
    uint8_t msg[sizeof tag + 48];
    size_t n = 0;
    memcpy(msg, tag, sizeof tag);
    n = sizeof tag;
    for (int i = 0; i < 12; i++) {
        uint32_t w = i < 8 ? seed[i] : (i == 8 ? counter : nonce[i - 9]);
        for (int b = 0; b < 4; b++) msg[n++] = (uint8_t)(w >> (8 * b));
    }
    uint8_t o[64];
    shake256_short(msg, n, o, 64);
    for (int i = 0; i < 16; i++)
        out[i] = (uint32_t)o[4 * i] | ((uint32_t)o[4 * i + 1] << 8) | ((uint32_t)o[4 * i + 2] << 16) | ((uint32_t)o[4 * i + 3] << 24);
}

/* keys.rs:62-93: canonical coefficients of A_kind[row][col]. */
void oracle_mcommit_key_element(const uint32_t seed[8], uint32_t kind, uint32_t row, uint64_t col, uint64_t* out) {
    uint32_t nonce[3] = {(kind << 16) | row, (uint32_t)col, (uint32_t)(col >> 32)};
    for (uint32_t b = 0; b < MC_N / 8; b++) {
        uint64_t* v = out + 8 * b;
        int written = 0;
        for (int i = 0; i < 8; i++) v[i] = 0;
        for (uint32_t retry = 0; retry < 16 && written < 8; retry++) {
            uint32_t w[16];
            oracle_mcommit_shake_block(seed, b + 512u * retry, nonce, w);
            for (int t = 0; t < 8 && written < 8; t++) {
                uint64_t x = (uint64_t)w[2 * t] | ((uint64_t)w[2 * t + 1] << 32);
                if (x < MC_Q) v[written++] = x;
            }
        }
    }
}

static uint64_t mod_q_i128(__int128 v) {
    __int128 r = v % (__int128)MC_Q;
    if (r < 0) r += MC_Q;
    return (uint64_t)r;
}

/* out[row][4096] = sum_c centre(key[row][cols[c]]) * x[c] (negacyclic, over the integers) + err[row], mod q.
 * x: ncols columns of 4096 signed coefficients; err may be null. The exact sums must fit 127 bits:
 * |key| < 2^63, so callers keep ncols * 4096 * max|x| below 2^64. */
void oracle_mcommit_commit(const uint32_t seed[8], uint32_t kind, int rows, const uint64_t* cols, int ncols, const int64_t* x,
                           const int64_t* err, uint64_t* out) {
#pragma omp parallel for schedule(dynamic)
    for (int row = 0; row < rows; row++) {
        uint64_t* key = (uint64_t*)malloc(MC_N * sizeof(uint64_t));
        int64_t* kc = (int64_t*)malloc(MC_N * sizeof(int64_t));
        __int128* acc = (__int128*)calloc(MC_N, sizeof(__int128));
        for (int c = 0; c < ncols; c++) {
            oracle_mcommit_key_element(seed, kind, (uint32_t)row, cols[c], key);
            for (int i = 0; i < MC_N; i++) kc[i] = key[i] > (MC_Q - 1) / 2 ? -(int64_t)(MC_Q - key[i]) : (int64_t)key[i];
            const int64_t* xc = x + (size_t)c * MC_N;
            for (int i = 0; i < MC_N; i++) {
                if (xc[i] == 0) continue;
                const __int128 xi = xc[i];
                for (int j = 0; j < MC_N - i; j++) acc[i + j] += xi * kc[j];
                for (int j = MC_N - i; j < MC_N; j++) acc[i + j - MC_N] -= xi * kc[j];
            }
        }
        for (int j = 0; j < MC_N; j++) {
            __int128 v = acc[j];
            if (err) v += err[(size_t)row * MC_N + j];
            out[(size_t)row * MC_N + j] = mod_q_i128(v);
        }
        free(key);
        free(kc);
        free(acc);
    }
}
