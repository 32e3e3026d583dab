// Error reporting and process-wide state shared by the entry points of the inpc_b200 library.
#include "common.cuh"
#include <cstring>

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

}  // namespace inpc

extern "C" const char* inpc_last_error(void) { return inpc::g_error; }
extern "C" int inpc_version(void) { return 100; }
