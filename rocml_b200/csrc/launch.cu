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
