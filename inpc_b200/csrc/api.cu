// Error reporting and process-wide state shared by the entry points of the inpc_b200 library.
#include "common.cuh"
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

namespace inpc {

namespace {
thread_local char g_error[512] = "";
unsigned* g_status_host = nullptr;   // mapped pinned memory, STATUS_WORDS words
unsigned* g_status_dev = nullptr;
}  // namespace

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s failed: %s", what, cudaGetErrorString(e));
    return INPC_E_CUDA;
}

unsigned* device_status_ptr() {
    if (!g_status_dev) {
        void* h = nullptr;
        if (cudaHostAlloc(&h, sizeof(unsigned) * STATUS_WORDS, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            cuda_fail(cudaGetLastError(), "cudaHostAlloc(status)");
            return nullptr;
        }
        std::memset(h, 0, sizeof(unsigned) * STATUS_WORDS);
        void* d = nullptr;
        if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            cuda_fail(cudaGetLastError(), "cudaHostGetDevicePointer(status)");
            cudaFreeHost(h);
            return nullptr;
        }
        g_status_host = static_cast<unsigned*>(h);
        g_status_dev = static_cast<unsigned*>(d);
    }
    return g_status_dev;
}

unsigned read_and_clear_status(int word) {
    if (!g_status_host || word < 0 || word >= (int)STATUS_WORDS) return 0u;
    volatile unsigned* p = g_status_host + word;
    const unsigned v = *p;
    if (v) *p = 0u;
    return v;
}

// ---- launch counter and per-stage event timing --------------------------------------------------
namespace {
std::atomic<long long> g_launches{0};
std::atomic<bool> g_profile{false};
std::mutex g_profile_mutex;
struct Pending { int stage; cudaEvent_t start, stop; };
std::vector<Pending> g_pending;
std::vector<cudaEvent_t> g_free_events;
double g_stage_ms[STAGE_COUNT] = {0};
long long g_stage_count[STAGE_COUNT] = {0};
constexpr size_t kMaxPending = 1 << 16;

cudaEvent_t take_event() {
    if (!g_free_events.empty()) { cudaEvent_t e = g_free_events.back(); g_free_events.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
    return e;
}
}  // namespace

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

StageScope::StageScope(Stage stage, cudaStream_t s) : slot(-1), stream(s) {
    if (!g_profile.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    if (g_pending.size() >= kMaxPending) return;
    Pending p{(int)stage, take_event(), take_event()};
    if (!p.start || !p.stop) return;
    cudaEventRecord(p.start, stream);
    g_pending.push_back(p);
    slot = (int)g_pending.size() - 1;
}

StageScope::~StageScope() {
    if (slot < 0) return;
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    if (slot < (int)g_pending.size()) cudaEventRecord(g_pending[slot].stop, stream);
}

}  // namespace inpc

extern "C" long long inpc_launch_count(void) { return inpc::g_launches.load(); }

extern "C" int inpc_profile_enable(int on) {
    inpc::g_profile.store(on != 0);
    return INPC_OK;
}

extern "C" int inpc_profile_read(double* stage_ms, long long* stage_calls, int n, int reset) {
    using namespace inpc;
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    for (const Pending& p : g_pending) {
        float ms = 0.0f;
        if (cudaEventSynchronize(p.stop) == cudaSuccess && cudaEventElapsedTime(&ms, p.start, p.stop) == cudaSuccess) {
            g_stage_ms[p.stage] += ms;
            g_stage_count[p.stage] += 1;
        }
        g_free_events.push_back(p.start);
        g_free_events.push_back(p.stop);
    }
    g_pending.clear();
    (void)cudaGetLastError();
    for (int k = 0; k < n && k < (int)STAGE_COUNT; ++k) {
        if (stage_ms) stage_ms[k] = g_stage_ms[k];
        if (stage_calls) stage_calls[k] = g_stage_count[k];
    }
    if (reset)
        for (int k = 0; k < (int)STAGE_COUNT; ++k) { g_stage_ms[k] = 0.0; g_stage_count[k] = 0; }
    return INPC_OK;
}

extern "C" const char* inpc_last_error(void) { return inpc::g_error; }
extern "C" int inpc_version(void) { return 100; }
