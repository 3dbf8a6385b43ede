// Two implementations of mb_exchange (exchange.hpp).
//
// local   ranks are host threads of one process, each with its own stream on
//         the same or on different GPUs of the process; host words go through
//         pointers published under a barrier, device pieces by device-to-device
//         copies. This is how one GPU stands in for several in the tests, and
//         how a single host process drives several GPUs.
// shm     ranks are processes on one machine; host words go through a mailbox
//         in POSIX shared memory (one slot per rank, a sequence number and two
//         payload buffers each); the device all-to-all is a function the
//         caller supplies (NCCL in the benchmark).
//
// Every wait is on the host and bounded (MB_EXCHANGE_TIMEOUT_S seconds, default
// 120); a rank that gives up returns MB_ERR_EXCHANGE and the proof call fails.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "../common.cuh"
#include "exchange.hpp"

namespace {

double timeout_seconds() {
    static double t = [] {
        const char* e = std::getenv("MB_EXCHANGE_TIMEOUT_S");
        double v = e ? std::atof(e) : 0.0;
        return v > 0.0 ? v : 120.0;
    }();
    return t;
}

struct ExchangeBase {
    mb_exchange ex{};
    virtual ~ExchangeBase() {}
};

// ---- ranks as threads of one process ------------------------------------------------------------
struct LocalShared {
    explicit LocalShared(int w) : world(w), host_ptr(w, nullptr), dev_ptr(w, nullptr) {}
    int world;
    std::mutex mu;
    std::condition_variable cv;
    int arrived = 0;
    uint64_t generation = 0;
    bool failed = false;
    std::vector<const uint64_t*> host_ptr;
    std::vector<const uint64_t*> dev_ptr;

    // All ranks arrive, or the wait runs out and every later call fails too.
    int barrier() {
        std::unique_lock<std::mutex> lk(mu);
        if (failed) return MB_ERR_EXCHANGE;
        const uint64_t gen = generation;
        if (++arrived == world) {
            arrived = 0;
            generation++;
            cv.notify_all();
            return MB_OK;
        }
        const auto limit = std::chrono::duration<double>(timeout_seconds());
        if (!cv.wait_for(lk, limit, [&] { return generation != gen || failed; }) || failed) {
            failed = true;
            cv.notify_all();
            return MB_ERR_EXCHANGE;
        }
        return MB_OK;
    }
};

struct LocalExchange : ExchangeBase {
    std::shared_ptr<LocalShared> sh;

    static int gather(void* ctx, const uint64_t* mine, size_t words, uint64_t* all) {
        auto* self = static_cast<LocalExchange*>(static_cast<ExchangeBase*>(ctx));
        LocalShared& s = *self->sh;
        s.host_ptr[self->ex.rank] = mine;
        int rc = s.barrier();
        if (rc != MB_OK) return rc;
        for (int g = 0; g < s.world; g++) std::memcpy(all + (size_t)g * words, s.host_ptr[g], words * sizeof(uint64_t));
        return s.barrier();   // nobody reuses `mine` before everyone has copied it
    }
    static int all_to_all(void* ctx, const uint64_t* d_send, uint64_t* d_recv, size_t w) {
        auto* self = static_cast<LocalExchange*>(static_cast<ExchangeBase*>(ctx));
        LocalShared& s = *self->sh;
        if (cudaStreamSynchronize(MB_STREAM) != cudaSuccess) return MB_ERR_CUDA;
        s.dev_ptr[self->ex.rank] = d_send;
        int rc = s.barrier();
        if (rc != MB_OK) return rc;
        for (int g = 0; g < s.world; g++) {
            if (cudaMemcpyAsync(d_recv + (size_t)g * w, s.dev_ptr[g] + (size_t)self->ex.rank * w, w * sizeof(uint64_t),
                                cudaMemcpyDefault, MB_STREAM) != cudaSuccess)
                return MB_ERR_CUDA;
        }
        if (cudaStreamSynchronize(MB_STREAM) != cudaSuccess) return MB_ERR_CUDA;
        return s.barrier();   // every rank has read every send buffer
    }
};

// ---- ranks as processes: mailbox in shared memory --------------------------------------------------
struct alignas(64) SlotHeader {
    std::atomic<uint64_t> seq;
    uint64_t pad[7];
};
static_assert(sizeof(SlotHeader) == 64, "slot header is one cache line");
static_assert(std::atomic<uint64_t>::is_always_lock_free, "sequence numbers must be address-free");

struct ShmExchange : ExchangeBase {
    std::string name;
    int fd = -1;
    uint8_t* base = nullptr;
    size_t bytes = 0, slot_words = 0;
    uint64_t gen = 0;
    mb_all_to_all_fn a2a = nullptr;
    void* a2a_ctx = nullptr;

    ~ShmExchange() override {
        if (base) munmap(base, bytes);
        if (fd >= 0) close(fd);
        if (ex.rank == 0 && !name.empty()) shm_unlink(name.c_str());
    }
    size_t slot_bytes() const { return sizeof(SlotHeader) + 2 * slot_words * sizeof(uint64_t); }
    SlotHeader* header(int r) const { return reinterpret_cast<SlotHeader*>(base + (size_t)r * slot_bytes()); }
    uint64_t* payload(int r, int parity) const {
        return reinterpret_cast<uint64_t*>(base + (size_t)r * slot_bytes() + sizeof(SlotHeader)) + (size_t)parity * slot_words;
    }

    // One message per rank and generation. A rank writes generation k + 2 into the buffer generation k used
    // only after it has seen every peer at k + 1, and a peer announces k + 1 only after it has read all of k.
    int gather_chunk(const uint64_t* mine, size_t words, uint64_t* all, size_t stride) {
        gen++;
        const int parity = (int)(gen & 1);
        std::memcpy(payload(ex.rank, parity), mine, words * sizeof(uint64_t));
        header(ex.rank)->seq.store(gen, std::memory_order_release);
        const auto t0 = std::chrono::steady_clock::now();
        for (int g = 0; g < ex.world; g++) {
            unsigned spins = 0;
            while (header(g)->seq.load(std::memory_order_acquire) < gen) {
                if ((++spins & 0x3ff) == 0) {
                    std::chrono::duration<double> dt = std::chrono::steady_clock::now() - t0;
                    if (dt.count() > timeout_seconds()) return MB_ERR_EXCHANGE;
                    if (spins > (1u << 20)) std::this_thread::yield();
                }
            }
            std::memcpy(all + (size_t)g * stride, payload(g, parity), words * sizeof(uint64_t));
        }
        return MB_OK;
    }
    static int gather(void* ctx, const uint64_t* mine, size_t words, uint64_t* all) {
        auto* self = static_cast<ShmExchange*>(static_cast<ExchangeBase*>(ctx));
        for (size_t done = 0; done < words; done += self->slot_words) {
            size_t chunk = words - done < self->slot_words ? words - done : self->slot_words;
            int rc = self->gather_chunk(mine + done, chunk, all + done, words);
            if (rc != MB_OK) return rc;
        }
        return MB_OK;
    }
    static int all_to_all(void* ctx, const uint64_t* d_send, uint64_t* d_recv, size_t w) {
        auto* self = static_cast<ShmExchange*>(static_cast<ExchangeBase*>(ctx));
        if (!self->a2a) return MB_ERR_EXCHANGE;
        return self->a2a(self->a2a_ctx, d_send, d_recv, w);
    }
};

}  // namespace

extern "C" {

// `world` exchange objects for `world` host threads of this process (rank r uses out[r]).
int mb_exchange_local_create(int world, mb_exchange** out) {
    if (world < 1 || world > 64 || !out) return MB_ERR_ARG;
    auto sh = std::make_shared<LocalShared>(world);
    for (int r = 0; r < world; r++) {
        auto* e = new (std::nothrow) LocalExchange;
        if (!e) return MB_ERR_CUDA;
        e->sh = sh;
        e->ex.ctx = static_cast<ExchangeBase*>(e);
        e->ex.rank = r;
        e->ex.world = world;
        e->ex.all_gather_host = &LocalExchange::gather;
        e->ex.all_to_all_device = &LocalExchange::all_to_all;
        out[r] = &e->ex;
    }
    return MB_OK;
}

// One rank of `world` processes on this machine. `name` (e.g. "/mb_x_<port>") must be the same on every rank and
// unused by any other run; slot_words is the largest message sent in one piece (longer ones are cut). The device
// all-to-all is `a2a` (with `a2a_ctx`), supplied by the caller.
int mb_exchange_shm_create(const char* name, int rank, int world, size_t slot_words, mb_all_to_all_fn a2a, void* a2a_ctx,
                           mb_exchange** out) {
    if (!name || name[0] != '/' || rank < 0 || rank >= world || world > 64 || slot_words < 16 || !out) return MB_ERR_ARG;
    auto* e = new (std::nothrow) ShmExchange;
    if (!e) return MB_ERR_CUDA;
    e->ex.rank = rank;
    e->ex.world = world;
    e->slot_words = slot_words;
    e->bytes = (size_t)world * e->slot_bytes();
    e->fd = shm_open(name, O_CREAT | O_RDWR, 0600);
    if (e->fd < 0 || ftruncate(e->fd, (off_t)e->bytes) != 0) { delete e; return MB_ERR_EXCHANGE; }
    void* p = mmap(nullptr, e->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, e->fd, 0);
    if (p == MAP_FAILED) { delete e; return MB_ERR_EXCHANGE; }
    e->base = static_cast<uint8_t*>(p);
    e->name = name;
    e->a2a = a2a;
    e->a2a_ctx = a2a_ctx;
    e->ex.ctx = static_cast<ExchangeBase*>(e);
    e->ex.all_gather_host = &ShmExchange::gather;
    e->ex.all_to_all_device = &ShmExchange::all_to_all;
    *out = &e->ex;
    return MB_OK;
}

int mb_exchange_destroy(mb_exchange* ex) {
    if (ex) delete static_cast<ExchangeBase*>(ex->ctx);
    return MB_OK;
}

// The two calls, exposed so that a host in another language (or a test) can drive an exchange object directly.
int mb_exchange_all_gather_host(mb_exchange* ex, const uint64_t* mine, size_t words, uint64_t* all) {
    if (!ex || !mine || !all) return MB_ERR_ARG;
    return ex->all_gather_host(ex->ctx, mine, words, all);
}
int mb_exchange_all_to_all_device(mb_exchange* ex, const uint64_t* d_send, uint64_t* d_recv, size_t words_per_rank) {
    if (!ex || !d_send || !d_recv) return MB_ERR_ARG;
    return ex->all_to_all_device(ex->ctx, d_send, d_recv, words_per_rank);
}

}  // extern "C"
