// Error reporting and process-wide state shared by the entry points of the inpc_b200 library.
#include "common.cuh"
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

namespace inpc {

namespace {
thread_local char g_error[512] = "";

// Status slots: mapped pinned host memory, kStatusSlots x STATUS_WORDS words.  Every call that launches
// kernels with bounded waits takes the next slot (round-robin), clears it and hands its device address to
// those kernels; a kernel that gives up stores 1 into its word.  The host reads a slot without any device
// synchronisation.  A slot is reused after kStatusSlots further calls.
constexpr int kStatusSlots = 1024;
std::mutex g_status_mutex;
unsigned* g_status_host = nullptr;
unsigned* g_status_dev = nullptr;
long long g_status_next = 1;                       // ticket of the next call (0 = none)
const char* g_status_entry[kStatusSlots] = {nullptr};
thread_local long long g_thread_last_ticket = 0;   // last ticket this host thread took
constexpr int kRecent = 8;                         // tickets a thread keeps looking at when it makes its next calls
thread_local long long g_thread_recent[kRecent] = {0};
thread_local int g_thread_recent_pos = 0;

bool status_memory_ready() {
    if (g_status_dev) return true;
    void* h = nullptr;
    if (cudaHostAlloc(&h, sizeof(unsigned) * STATUS_WORDS * kStatusSlots, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
        cuda_fail(cudaGetLastError(), "cudaHostAlloc(status)");
        return false;
    }
    std::memset(h, 0, sizeof(unsigned) * STATUS_WORDS * kStatusSlots);
    void* d = nullptr;
    if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
        cuda_fail(cudaGetLastError(), "cudaHostGetDevicePointer(status)");
        cudaFreeHost(h);
        return false;
    }
    g_status_host = static_cast<unsigned*>(h);
    g_status_dev = static_cast<unsigned*>(d);
    return true;
}
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

unsigned* acquire_status(const char* entry, long long* ticket_out) {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!status_memory_ready()) return nullptr;
    const long long ticket = g_status_next++;
    const int slot = (int)(ticket % kStatusSlots);
    volatile unsigned* w = g_status_host + (size_t)slot * STATUS_WORDS;
    for (int k = 0; k < (int)STATUS_WORDS; ++k) w[k] = 0u;
    g_status_entry[slot] = entry;
    g_thread_last_ticket = ticket;
    g_thread_recent[g_thread_recent_pos] = ticket;
    g_thread_recent_pos = (g_thread_recent_pos + 1) % kRecent;
    if (ticket_out) *ticket_out = ticket;
    return g_status_dev + (size_t)slot * STATUS_WORDS;
}

int read_status(long long ticket, unsigned* words, const char** entry) {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (ticket <= 0 || ticket >= g_status_next || !g_status_host) { set_error("status ticket %lld was never issued", ticket); return INPC_E_INVALID; }
    if (g_status_next - ticket > kStatusSlots) { set_error("status ticket %lld is too old: its slot has been reused", ticket); return INPC_E_INVALID; }
    const int slot = (int)(ticket % kStatusSlots);
    const volatile unsigned* w = g_status_host + (size_t)slot * STATUS_WORDS;
    for (int k = 0; k < (int)STATUS_WORDS; ++k) words[k] = w[k];
    if (entry) *entry = g_status_entry[slot];
    return INPC_OK;
}

// Message + INPC_E_DEVICE if the words report a failure (sampler exhaustion is informational and does not count).
static int status_to_result(const unsigned* w, const char* entry) {
    const char* who = entry ? entry : "an earlier call";
    if (w[STATUS_LOOKBACK_TIMEOUT]) { set_error("%s: a radix-sort tile gave up waiting for a predecessor tile; the results of that call are invalid", who); return INPC_E_DEVICE; }
    if (w[STATUS_BULK_COPY_TIMEOUT]) { set_error("%s: a block gave up waiting for its bulk copy into shared memory; the results of that call are invalid", who); return INPC_E_DEVICE; }
    if (w[STATUS_INDEX_OUT_OF_RANGE]) { set_error("%s: a gather index was out of range (access skipped); the results of that call are invalid", who); return INPC_E_DEVICE; }
    return INPC_OK;
}

int check_previous_calls() {
    // the kernels of a recent call may still be running, so each of the last few tickets is looked at again
    // at every call until it has been reported once or has dropped out of the window
    for (int k = 0; k < kRecent; ++k) {
        const long long ticket = g_thread_recent[k];
        if (ticket <= 0) continue;
        unsigned w[STATUS_WORDS];
        const char* entry = nullptr;
        if (read_status(ticket, w, &entry) != INPC_OK) { g_thread_recent[k] = 0; continue; }   // slot already reused
        const int rc = status_to_result(w, entry);
        if (rc != INPC_OK) { g_thread_recent[k] = 0; return rc; }
    }
    return INPC_OK;
}

int sm_count() {
    static std::mutex m;
    static int cached[kMaxDevices] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::lock_guard<std::mutex> lock(m);
    if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) return cached[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (dev >= 0 && dev < kMaxDevices) cached[dev] = sms;
    return sms;
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

extern "C" long long inpc_last_call_ticket(void) { return inpc::g_thread_last_ticket; }

extern "C" int inpc_call_status(long long ticket, unsigned* words) {
    using namespace inpc;
    unsigned w[STATUS_WORDS];
    const char* entry = nullptr;
    const int rc = read_status(ticket, w, &entry);
    if (rc != INPC_OK) return rc;
    if (words)
        for (int k = 0; k < (int)STATUS_WORDS; ++k) words[k] = w[k];
    return status_to_result(w, entry);
}

extern "C" const char* inpc_last_error(void) { return inpc::g_error; }
extern "C" int inpc_version(void) { return 100; }
