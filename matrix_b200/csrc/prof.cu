// Implementation of the launch counter and per-kernel stopwatch (see prof.cuh).
#include "prof.cuh"
#include "common.cuh"
#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace mb {
namespace prof {

static std::atomic<uint64_t> g_launches{0};
static std::atomic<int> g_enabled{0};
static std::mutex g_mu;

struct Pending {
    const char* name;
    cudaEvent_t a, b;
};
static std::vector<Pending> g_pending;
static std::vector<cudaEvent_t> g_free_events;
struct Stat {
    uint64_t launches = 0;
    double ms = 0.0;
};
static std::map<std::string, Stat> g_stats;
static thread_local Pending t_open{nullptr, nullptr, nullptr};

static cudaEvent_t get_event() {
    if (!g_free_events.empty()) {
        cudaEvent_t e = g_free_events.back();
        g_free_events.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

void scope_begin(const char* name, cudaStream_t st) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (!g_enabled.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lk(g_mu);
    t_open.name = name;
    t_open.a = get_event();
    t_open.b = get_event();
    cudaEventRecord(t_open.a, st);
}

void scope_end(cudaStream_t st) {
    if (!t_open.name) return;
    std::lock_guard<std::mutex> lk(g_mu);
    cudaEventRecord(t_open.b, st);
    g_pending.push_back(t_open);
    t_open.name = nullptr;
}

// Folds finished event pairs into the per-name statistics.
static void drain() {
    for (auto& p : g_pending) {
        cudaEventSynchronize(p.b);
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) {
            Stat& s = g_stats[p.name];
            s.launches++;
            s.ms += ms;
        }
        g_free_events.push_back(p.a);
        g_free_events.push_back(p.b);
    }
    g_pending.clear();
}

}  // namespace prof
}  // namespace mb

extern "C" {

// Kernels launched by this library in this process so far.
uint64_t mb_launch_count() { return mb::prof::g_launches.load(); }

int mb_prof_enable(int on) {
    mb::prof::g_enabled.store(on ? 1 : 0);
    return MB_OK;
}

int mb_prof_reset() {
    std::lock_guard<std::mutex> lk(mb::prof::g_mu);
    mb::prof::drain();
    mb::prof::g_stats.clear();
    return MB_OK;
}

// Writes "name launches total_ms\n" lines into buf (NUL terminated, truncated
// to cap). Returns the number of bytes the full report needs.
size_t mb_prof_report(char* buf, size_t cap) {
    std::lock_guard<std::mutex> lk(mb::prof::g_mu);
    mb::prof::drain();
    std::string out;
    char line[256];
    for (auto& kv : mb::prof::g_stats) {
        snprintf(line, sizeof(line), "%s %llu %.6f\n", kv.first.c_str(), (unsigned long long)kv.second.launches, kv.second.ms);
        out += line;
    }
    if (buf && cap) {
        size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
        memcpy(buf, out.data(), n);
        buf[n] = '\0';
    }
    return out.size() + 1;
}

}  // extern "C"
