// Launch accounting and an optional per-kernel stopwatch.
//
// Every kernel launch of the library sits inside an MB_KERNEL("name") scope.
// The scope always bumps a launch counter (what a benchmark reports as the
// number of this library's kernels it ran). When profiling is switched on
// (mb_prof_enable(1)), the scope also records a CUDA event on the launching
// stream before and after the launch, and mb_prof_report() returns, per name,
// the launch count and the summed device time between the two events.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {
namespace prof {

void scope_begin(const char* name, cudaStream_t st);
void scope_end(cudaStream_t st);

struct Scope {
    cudaStream_t st;
    Scope(const char* name, cudaStream_t s) : st(s) { scope_begin(name, s); }
    ~Scope() { scope_end(st); }
};

}  // namespace prof
}  // namespace mb

#define MB_CAT2(a, b) a##b
#define MB_CAT(a, b) MB_CAT2(a, b)
#define MB_KERNEL(name) mb::prof::Scope MB_CAT(mb_scope_, __LINE__)(name, MB_STREAM)
#define MB_KERNEL_ON(name, stream) mb::prof::Scope MB_CAT(mb_scope_, __LINE__)(name, stream)
