// Error reporting, version queries and launch policy shared by all kmll_b200 entry points.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace kmll {

char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return KMLL_OK;
}

// Programmatic dependent launch is on unless KMLL_PDL=0 is set in the environment.
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("KMLL_PDL");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

}  // namespace kmll

extern "C" {
const char* kmll_last_error(void) { return kmll::last_error_buffer(); }
int kmll_version(void) { return 100; }
int kmll_compiled_arch(void) { return 100; }
}
