// Error reporting, version queries and launch policy shared by all kmll_b200 entry points.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

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


unsigned long long& launch_counter() {
    static thread_local unsigned long long n = 0;
    return n;
}

namespace {
struct TraceLaunch { int kernel_id; int blocks; size_t offset_words; };
struct TraceState {
    std::mutex mu;
    unsigned long long* buf = nullptr;
    size_t capacity_words = 0, next_word = 0;
    std::vector<TraceLaunch> launches;
    unsigned long long generation = 0;
} g_trace;
}  // namespace

unsigned long long trace_generation() {
    std::lock_guard<std::mutex> lock(g_trace.mu);
    return g_trace.generation;
}

unsigned long long* trace_next_slot(int kernel_id, int blocks) {
    std::lock_guard<std::mutex> lock(g_trace.mu);
    if (g_trace.buf == nullptr) return nullptr;
    const size_t need = (size_t)blocks * kTraceStamps;
    if (g_trace.next_word + need > g_trace.capacity_words) return nullptr;  // buffer full: later launches are not traced
    unsigned long long* slot = g_trace.buf + g_trace.next_word;
    g_trace.launches.push_back({kernel_id, blocks, g_trace.next_word});
    g_trace.next_word += need;
    return slot;
}

}  // namespace kmll

extern "C" {
const char* kmll_last_error(void) { return kmll::last_error_buffer(); }
int kmll_version(void) { return 100; }
int kmll_compiled_arch(void) { return 100; }

int kmll_trace_attach(void* device_buffer, size_t bytes) {
    std::lock_guard<std::mutex> lock(kmll::g_trace.mu);
    kmll::g_trace.buf = static_cast<unsigned long long*>(device_buffer);
    kmll::g_trace.capacity_words = device_buffer ? bytes / sizeof(unsigned long long) : 0;
    kmll::g_trace.next_word = 0;
    kmll::g_trace.launches.clear();
    ++kmll::g_trace.generation;  // cached CUDA graphs hold slot pointers of the previous buffer: they are captured again
    return KMLL_OK;
}

int kmll_trace_launches(int* kernel_ids, int* blocks, size_t* offset_words, int max_launches, int* count_out) {
    std::lock_guard<std::mutex> lock(kmll::g_trace.mu);
    const int n = (int)kmll::g_trace.launches.size();
    if (count_out) *count_out = n;
    for (int i = 0; i < n && i < max_launches; ++i) {
        if (kernel_ids) kernel_ids[i] = kmll::g_trace.launches[i].kernel_id;
        if (blocks) blocks[i] = kmll::g_trace.launches[i].blocks;
        if (offset_words) offset_words[i] = kmll::g_trace.launches[i].offset_words;
    }
    return KMLL_OK;
}
}
