// The exchange a sharded prover needs, behind two calls.
//
// A proof that is partitioned over several GPUs (one host thread or process
// per GPU, "ranks") talks to the other ranks in two ways only:
//   all_gather_host    a few words per round (partial round polynomials,
//                      subtree roots) that the host transcript needs anyway;
//   all_to_all_device  bulk data resident on the GPUs, once per proof (the
//                      transposition between the evaluations' partition and
//                      the codeword's partition).
// The prover is written against this struct; who moves the bytes is the
// caller's choice: threads of one process (mb_exchange_local_create), a
// mailbox in POSIX shared memory for the host words with the device exchange
// delegated to the caller's collective library (mb_exchange_shm_create), or
// any other pair of functions.
//
// No kernel of this library waits for another rank: every wait is a host wait
// with a time limit, after which the call fails with MB_ERR_CUDA's sibling
// code MB_ERR_EXCHANGE.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define MB_ERR_EXCHANGE (-4)

extern "C" {

typedef struct mb_exchange {
    void* ctx;
    int rank;
    int world;
    // Every rank passes `words` words of host memory; `all` receives world * words words, rank-major.
    // Collective: every rank calls it with the same `words`. Returns 0 on success.
    int (*all_gather_host)(void* ctx, const uint64_t* mine, size_t words, uint64_t* all);
    // d_send and d_recv hold `world` pieces of `words_per_rank` words of device memory. Piece r of d_send goes to
    // rank r; piece g of d_recv comes from rank g. The caller's stream has been synchronised before the call;
    // on return d_recv is complete and d_send may be reused. Returns 0 on success.
    int (*all_to_all_device)(void* ctx, const uint64_t* d_send, uint64_t* d_recv, size_t words_per_rank);
} mb_exchange;

typedef int (*mb_all_to_all_fn)(void* ctx, const uint64_t* d_send, uint64_t* d_recv, size_t words_per_rank);

}  // extern "C"
