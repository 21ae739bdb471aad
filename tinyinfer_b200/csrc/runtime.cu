// Error text and launch counter shared by the launchers of one library.
#include "common.cuh"
#include <atomic>
#include <cstdarg>
#include <cstdlib>

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void ti_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
void ti_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool ti_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("TINYINFER_B200_PDL");
        on = (v && v[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

TI_API const char* ti_last_error() { return g_error; }
// Kernels launched through this library since it was loaded.
TI_API long long ti_launch_count() { return g_launches.load(std::memory_order_relaxed); }
