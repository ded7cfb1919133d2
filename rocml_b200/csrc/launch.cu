// Launch policy shared by all kernels.
#include "common.cuh"
#include <cstdlib>
#include <cstring>

namespace rb {
// Programmatic dependent launch is on unless the environment says RB_PDL=0 (for debugging).
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("RB_PDL");
        return !(v && std::strcmp(v, "0") == 0);
    }();
    return on;
}
}  // namespace rb

// Keeps the stream busy for about `microseconds` (one thread spinning on the global timer, which counts
// nanoseconds whatever the clocks do; at most a second).  The profiler holds the GPU back with it while the
// host enqueues a step, so that the step's kernels then run back to back.
__global__ void hold_kernel(unsigned long long ns) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
        __nanosleep(1000);
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < ns);
}

extern "C" int rb_hold(long long microseconds, void* stream) {
    if (microseconds <= 0) return RB_OK;
    if (microseconds > 1000000) microseconds = 1000000;
    hold_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((unsigned long long)microseconds * 1000ull);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
