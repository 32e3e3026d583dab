// Shared host/device helpers of the inpc_b200 library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <mutex>
#include "../../include/inpc_b200.h"

namespace inpc {

// ---- error reporting ---------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define INPC_CUDA_TRY(expr)                                        \
    do {                                                           \
        cudaError_t _e = (expr);                                   \
        if (_e != cudaSuccess) return ::inpc::cuda_fail(_e, #expr); \
    } while (0)

// After every kernel launch: counts it (inpc_launch_count) and turns a launch error into a status.
#define INPC_LAUNCH_CHECK(name)                                       \
    do {                                                              \
        ::inpc::count_launch();                                       \
        cudaError_t _e = cudaGetLastError();                          \
        if (_e != cudaSuccess) return ::inpc::cuda_fail(_e, name);     \
    } while (0)

void count_launch();

// Optional per-stage device timing (inpc_profile_enable): a StageScope records a CUDA event pair
// around the launches of one pipeline stage on the stream they are issued to.
enum Stage : int {
    STAGE_SAMPLE = 0,        // leaf weights, CDF, draws
    STAGE_PREPROCESS = 1,    // visibility count, scan, project + SH
    STAGE_SORT_DEPTH = 2,
    STAGE_INSTANCES = 3,     // per-point tile counts, scan, emission
    STAGE_SORT_TILE = 4,     // tile sort + ranges
    STAGE_BLEND_FWD = 5,
    STAGE_BLEND_BWD = 6,
    STAGE_PREPROCESS_BWD = 7,
    STAGE_COUNT = 8,
};
struct StageScope {
    int slot;
    cudaStream_t stream;
    StageScope(Stage stage, cudaStream_t s);
    ~StageScope();
};

// Device-visible status words in mapped pinned host memory: a kernel stores 1 into its word when a
// bounded wait runs out (plain store, no atomics over PCIe); the host reads them without a device
// synchronisation.
enum : unsigned {
    STATUS_LOOKBACK_TIMEOUT = 0,   // a radix-sort tile gave up waiting for a predecessor tile
    STATUS_SAMPLER_EXHAUSTED = 1,  // informational: some sample slots ran out of rejection attempts
    STATUS_BULK_COPY_TIMEOUT = 2,  // a block gave up waiting for its bulk copy into shared memory
    STATUS_INDEX_OUT_OF_RANGE = 3, // checked build only: a gather index was outside its array (the access was skipped)
    STATUS_WORDS = 4,
};
// Takes the next status slot for a call of `entry` (a string literal): returns the device address of its
// STATUS_WORDS cleared words, or nullptr (error set).  *ticket_out names the slot for read_status.
unsigned* acquire_status(const char* entry, long long* ticket_out = nullptr);
int read_status(long long ticket, unsigned* words, const char** entry);
// INPC_E_DEVICE (with a message naming the entry point) if the last status-carrying call this host thread
// made has reported a failure since; every entry point that launches work calls it first, so a failure
// surfaces at the thread's next call at the latest -- or earlier through inpc_call_status.
int check_previous_calls();

// ---- small utilities ---------------------------------------------------------------------
template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// Carves consecutive 256-byte-aligned arrays out of one blob.
struct Carver {
    char* base;
    size_t off = 0;
    explicit Carver(void* p) : base(static_cast<char*>(p)) {}
    template <typename T>
    T* take(size_t count) {
        off = align_up(off);
        T* p = reinterpret_cast<T*>(base + off);
        off += sizeof(T) * count;
        return p;
    }
    size_t used() const { return align_up(off); }
};

inline int bit_length(uint32_t v) {
    int b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

// ---- camera parameters passed by value to kernels -----------------------------------------
struct ViewParams {
    const float* w2c;   // device, 16 floats
    const float* cam;   // device, 3 floats
    int width, height;
    float fx, fy, cx, cy, near_plane, far_plane;
};

inline ViewParams to_params(const inpc_view* v) {
    ViewParams p;
    p.w2c = v->w2c; p.cam = v->cam_position;
    p.width = v->width; p.height = v->height;
    p.fx = v->fx; p.fy = v->fy; p.cx = v->cx; p.cy = v->cy;
    p.near_plane = v->near_plane; p.far_plane = v->far_plane;
    return p;
}

// ---- radix sort (radix_sort.cu) ------------------------------------------------------------
size_t sort_workspace_bytes(int64_t n);
int sort_pass_count(int end_bit);   // passes sort_pairs makes; the result is in the alternate buffers iff odd (and n > 1)
// `status`: device address of the STATUS_WORDS words a tile that gives up its look-back reports to.
int sort_pairs(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n,
               int end_bit, void* workspace, unsigned* status, int* result_in_alt, cudaStream_t stream);
// The number of pairs is *n_dev (device memory, <= n_max); the workspace is sized for n_max.  The result is in the
// alternate buffers iff sort_pass_count(end_bit) is odd, whatever the count turns out to be.
int sort_pairs_device_count(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n_max,
                            const unsigned long long* n_dev, int end_bit, void* workspace, unsigned* status, int* result_in_alt,
                            cudaStream_t stream);

// More than 48 KB of dynamic shared memory is an opt-in per kernel AND per device: `done` is the
// caller's per-kernel table of devices already set up.
constexpr int kMaxDevices = 64;
// Number of multiprocessors of the current device (looked up once per device; 148 if the query fails).
int sm_count();

template <typename Kernel>
int opt_in_dynamic_smem(Kernel kernel, size_t bytes, bool (&done)[kMaxDevices]) {
    static std::mutex table_mutex;   // one per kernel: host threads may reach the same kernel's table together
    std::lock_guard<std::mutex> lock(table_mutex);
    int dev = 0;
    INPC_CUDA_TRY(cudaGetDevice(&dev));
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    if (tracked && done[dev]) return INPC_OK;
    INPC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (tracked) done[dev] = true;
    return INPC_OK;
}

// ---- device helpers ------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31u; }

__device__ __forceinline__ unsigned warp_inclusive_scan(unsigned v) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane_id() >= (unsigned)o) v += t;
    }
    return v;
}

// ---- bulk asynchronous copies (the copy engine behind TMA, untiled form) ------------------------------
// global -> shared: one thread arms an mbarrier with the byte count and issues the copy; every thread
// that will read the data waits on the barrier's phase.  Source, destination and size must be
// multiples of 16 bytes.  The wait is bounded: a block that gives up reports it and the caller skips
// its work, the next entry point of the library then returns an error.
__device__ __forceinline__ unsigned shared_address(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarrier_init(unsigned long long* bar, unsigned arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(bar)), "r"(arrivals) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void bulk_load_to_shared(void* dst_shared, const void* src_global, unsigned bytes, unsigned long long* bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(shared_address(dst_shared)),
                 "l"(src_global), "r"(bytes), "r"(shared_address(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbarrier_wait_bounded(unsigned long long* bar, unsigned parity) {
    const unsigned addr = shared_address(bar);
    for (int spin = 0; spin < (1 << 20); ++spin) {
        unsigned done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// shared -> global: the writers of the shared data call `fence_shared_for_bulk()` before the block
// barrier, then one thread issues the store and waits until the source has been read.
__device__ __forceinline__ void fence_shared_for_bulk() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void bulk_store_from_shared(void* dst_global, const void* src_shared, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_global), "r"(shared_address(src_shared)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Block-wide exclusive scan of one unsigned per thread; `smem` needs (blockDim.x/32 + 1) words.
// Returns the exclusive prefix; *total receives the block sum (same value in every thread).
__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned* smem, unsigned* total) {
    const unsigned lane = lane_id(), warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    const unsigned inc = warp_inclusive_scan(v);
    if (lane == 31) smem[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned w = lane < nwarps ? smem[lane] : 0u;
        unsigned winc = warp_inclusive_scan(w);
        if (lane < nwarps) smem[lane] = winc - w;
        if (lane == 31) smem[nwarps] = winc;
    }
    __syncthreads();
    const unsigned r = smem[warp] + inc - v;
    *total = smem[nwarps];
    __syncthreads();
    return r;
}
#endif

}  // namespace inpc
