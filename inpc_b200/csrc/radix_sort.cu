// Onesweep least-significant-digit radix sort of (u32 key, u32 value) pairs for sm_100a.
//
// One up-front kernel builds the digit histograms of every pass in a single read of the keys; each
// pass is then ONE kernel that reads the pairs once and writes them once.  Inside a pass every tile
// ranks its keys stably (per-warp match-any ranking), publishes its per-digit counts and resolves
// its global offsets with a decoupled look-back over the tiles before it.  Tiles take their index
// from a ticket counter, so a tile a later one waits for is always already running; every wait is
// nevertheless bounded and reports through the status word instead of spinning for ever.
//
// Replaces cub::DeviceRadixSort::SortPairs as used in rasterization/src/bilinear/forward.cu:91-98
// (32-bit depth keys) and :132-139 (tile keys) of the reference.
#include "common.cuh"
#include <mutex>

namespace inpc {

namespace {

constexpr int kRadixBits = 9;            // widest digit of a pass: 27 key bits sort in 3 passes, 32 in 4 x 8
constexpr int kRadix = 1 << kRadixBits;  // capacity of every per-digit array
constexpr int kMaxPasses = 4;
constexpr int kThreads = 512;
constexpr int kItems = 16;
constexpr int kTile = kThreads * kItems;   // 8192 pairs per tile
constexpr int kWarps = kThreads / 32;
constexpr int kDigitsPerThread = (kRadix + kThreads - 1) / kThreads;   // digits a thread owns in the scan / look-back phase

constexpr unsigned kFlagAggregate = 1u << 30;
constexpr unsigned kFlagPrefix = 2u << 30;
constexpr unsigned kFlagMask = 3u << 30;
constexpr unsigned kValueMask = ~kFlagMask;
constexpr int kSpinLimit = 1 << 22;

struct PassTable {
    int n_passes;
    int shift[kMaxPasses];
    int bits[kMaxPasses];
};

// ---- histogram of every pass in one read ---------------------------------------------------
constexpr int kHistThreads = 512;
constexpr int kHistItemsPerBlock = kHistThreads * 4 * 8;   // 8 uint4 loads per thread

// `n_dev` (optional): the number of pairs lives on the device (the grid is then sized for an upper bound).
// The kernel is bound by its shared-memory atomics (up to four per key), not by how the keys arrive: a variant that
// brought them in with bulk asynchronous copies (cp.async.bulk into two 16 KB slabs per block, an mbarrier per slab)
// measured the same on B200 -- whole sort of 2^23 pairs, 32 / 27 / 24 key bits: 316 / 271 / 241 us against
// 314 / 267 / 239 us with the plain 16-byte loads below; 2^25 pairs, 25 bits: 794 against 799 us.
__global__ void __launch_bounds__(kHistThreads) radix_histogram_kernel(
    const uint32_t* __restrict__ keys, int64_t n_arg, const unsigned long long* __restrict__ n_dev, PassTable pt, unsigned* __restrict__ hist) {
    const int64_t n = n_dev ? (int64_t)*n_dev : n_arg;
    if ((int64_t)blockIdx.x * kHistItemsPerBlock >= n) return;
    __shared__ unsigned s_hist[kMaxPasses][kRadix];
    for (int i = threadIdx.x; i < kMaxPasses * kRadix; i += kHistThreads) (&s_hist[0][0])[i] = 0;
    __syncthreads();

    const int64_t block_base = (int64_t)blockIdx.x * kHistItemsPerBlock;
    const int64_t block_end = min(n, block_base + (int64_t)kHistItemsPerBlock);
    auto count = [&](uint32_t k) {
#pragma unroll
        for (int p = 0; p < kMaxPasses; ++p)
            if (p < pt.n_passes) atomicAdd(&s_hist[p][(k >> pt.shift[p]) & ((1u << pt.bits[p]) - 1u)], 1u);
    };
    // keys is 16-byte aligned (carved at 256 bytes) and block_base is a multiple of 4
    const uint4* keys4 = reinterpret_cast<const uint4*>(keys + block_base);
    const int64_t n_vec = (block_end - block_base) / 4;
    for (int64_t v = threadIdx.x; v < n_vec; v += kHistThreads) {
        const uint4 k = __ldg(keys4 + v);
        count(k.x); count(k.y); count(k.z); count(k.w);
    }
    for (int64_t i = block_base + n_vec * 4 + threadIdx.x; i < block_end; i += kHistThreads) count(keys[i]);
    __syncthreads();
    for (int i = threadIdx.x; i < kMaxPasses * kRadix; i += kHistThreads) {
        const unsigned c = (&s_hist[0][0])[i];
        if (c) atomicAdd(hist + i, c);
    }
}

// exclusive scan of each pass's 256 counters -> global digit bases
__global__ void __launch_bounds__(kRadix) radix_scan_histogram_kernel(const unsigned* __restrict__ hist,
                                                                      unsigned* __restrict__ base) {
    __shared__ unsigned s_scan[kRadix / 32 + 1];
    const int p = blockIdx.x;
    const unsigned c = hist[p * kRadix + threadIdx.x];
    unsigned total;
    const unsigned ex = block_exclusive_scan(c, s_scan, &total);
    base[p * kRadix + threadIdx.x] = ex;
}

// ---- one pass ---------------------------------------------------------------------------------
struct PassSmem {
    union {
        unsigned warp_hist[kWarps][kRadix];   // ranking phase
        uint32_t keys[kTile];                 // reorder phase (keys); the two never live at the same time
    };
    uint32_t values[kTile];
    unsigned bin_start[kRadix];    // tile-local exclusive start of each digit
    unsigned global_off[kRadix];   // global position of a digit's first key minus bin_start
    unsigned scan[kWarps + 1];
    unsigned tile_id;
};

// BITS > 0 fixes the digit width at compile time (the ballot loop of the ranking unrolls); BITS == 0
// takes it from `bits_arg`.
template <int BITS>
__global__ void __launch_bounds__(kThreads) radix_onesweep_pass_kernel(
    const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
    uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n_arg, const unsigned long long* __restrict__ n_dev,
    int shift, int bits_arg, const unsigned* __restrict__ digit_base, volatile unsigned* tile_state, unsigned* ticket,
    volatile unsigned* status, int spin_limit, unsigned mute_tile) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    PassSmem& s = *reinterpret_cast<PassSmem*>(smem_raw);

    const unsigned tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const int bits = BITS > 0 ? BITS : bits_arg;
    const unsigned digit_mask = (1u << bits) - 1u;

    if (tid == 0) s.tile_id = atomicAdd(ticket, 1u);
    for (int i = tid; i < kWarps * kRadix; i += kThreads) (&s.warp_hist[0][0])[i] = 0;
    __syncthreads();
    const unsigned tile = s.tile_id;
    // `mute_tile` (no tile in normal operation) leaves without publishing anything: the tiles behind it then
    // run into the limit of their look-back wait, which is how the tests exercise that path
    if (tile == mute_tile) return;
    const int64_t n = n_dev ? (int64_t)*n_dev : n_arg;
    const int64_t tile_base = (int64_t)tile * kTile;
    if (tile_base >= n) return;   // grid sized for an upper bound of n: nothing here, and no tile waits for this one
    const int valid = (int)min((int64_t)kTile, n - tile_base);

    // warp-striped load: warp w owns [w*32*kItems, (w+1)*32*kItems) of the tile, item i of lane l
    // is element i*32+l of that segment, so (warp, item, lane) order is the input order.
    uint32_t key[kItems];
    unsigned rank[kItems];
    const int seg = warp * 32 * kItems;
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const int local = seg + i * 32 + lane;
        key[i] = local < valid ? __ldg(keys_in + tile_base + local) : 0xFFFFFFFFu;
    }

    // stable rank within the warp's segment, per digit.  The lanes holding the same digit are found
    // with one ballot per digit bit (independent across items, so they pipeline); only the update of
    // the warp's digit counter is a serial chain.
    unsigned peers[kItems];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const unsigned d = (key[i] >> shift) & digit_mask;
        unsigned p = 0xffffffffu;
        if (BITS > 0) {
#pragma unroll
            for (int b = 0; b < BITS; ++b) {
                const bool one = (d >> b) & 1u;
                const unsigned m = __ballot_sync(0xffffffffu, one);
                p &= one ? m : ~m;
            }
        } else {
            for (int b = 0; b < bits; ++b) {
                const bool one = (d >> b) & 1u;
                const unsigned m = __ballot_sync(0xffffffffu, one);
                p &= one ? m : ~m;
            }
        }
        peers[i] = p;
    }
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const unsigned d = (key[i] >> shift) & digit_mask;
        const int leader = __ffs(peers[i]) - 1;
        unsigned base = 0;
        if ((int)lane == leader) {
            base = s.warp_hist[warp][d];
            s.warp_hist[warp][d] = base + __popc(peers[i]);
        }
        base = __shfl_sync(0xffffffffu, base, leader);
        rank[i] = base + __popc(peers[i] & ((1u << lane) - 1u));
        __syncwarp();
    }
    __syncthreads();

    // per digit: exclusive scan over warps, tile total.  Thread t owns digits t*kDigitsPerThread ...
    const unsigned radix = 1u << bits;
    unsigned total[kDigitsPerThread];
    unsigned thread_sum = 0;
#pragma unroll
    for (int q = 0; q < kDigitsPerThread; ++q) {
        const unsigned d = tid * kDigitsPerThread + q;
        total[q] = 0;
        if (d < radix) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const unsigned c = s.warp_hist[w][d];
                s.warp_hist[w][d] = total[q];
                total[q] += c;
            }
            // publish this tile's digit count before any waiting
            tile_state[(size_t)tile * kRadix + d] = total[q] | (tile == 0 ? kFlagPrefix : kFlagAggregate);
        }
        thread_sum += total[q];
    }
    unsigned block_total;
    unsigned start = block_exclusive_scan(thread_sum, s.scan, &block_total);
#pragma unroll
    for (int q = 0; q < kDigitsPerThread; ++q) {
        const unsigned d = tid * kDigitsPerThread + q;
        if (d >= radix) break;
        s.bin_start[d] = start;
        // decoupled look-back, a window of predecessors per round trip: the loads of a window are
        // independent, so their latencies overlap; entries are then consumed nearest-first
        unsigned exclusive = 0;
        if (tile > 0) {
            constexpr int kWindow = 8;
            int64_t j = (int64_t)tile - 1;
            bool gave_up = false, finished = false;
            while (j >= 0 && !finished && !gave_up) {
                unsigned v[kWindow];
#pragma unroll
                for (int k = 0; k < kWindow; ++k) {
                    v[k] = 2u << 30;   // beyond tile 0: an empty inclusive prefix
                    if (j - k >= 0) v[k] = tile_state[(size_t)(j - k) * kRadix + d];
                }
#pragma unroll
                for (int k = 0; k < kWindow; ++k) {
                    if (finished || gave_up) break;
                    unsigned x = v[k];
                    int spins = 0;
                    while ((x & kFlagMask) == 0u && spins < spin_limit) {   // not published yet: poll this one
                        __nanosleep(20);
                        x = tile_state[(size_t)(j - k) * kRadix + d];
                        ++spins;
                    }
                    if ((x & kFlagMask) == 0u) { gave_up = true; break; }
                    exclusive += x & kValueMask;
                    if (x & kFlagPrefix) finished = true;
                }
                j -= kWindow;
            }
            if (gave_up) status[STATUS_LOOKBACK_TIMEOUT] = 1u;
            tile_state[(size_t)tile * kRadix + d] = ((exclusive + total[q]) & kValueMask) | kFlagPrefix;
        }
        s.global_off[d] = digit_base[d] + exclusive - start;
        start += total[q];
    }
    __syncthreads();

    // tile-local position of every key; values follow the same permutation
    unsigned pos[kItems];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const unsigned d = (key[i] >> shift) & digit_mask;
        pos[i] = s.bin_start[d] + s.warp_hist[warp][d] + rank[i];
    }
    uint32_t val[kItems];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const int local = seg + i * 32 + lane;
        val[i] = local < valid ? __ldg(vals_in + tile_base + local) : 0u;
    }
    __syncthreads();   // warp_hist is dead from here on: its storage becomes the key staging area
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        s.keys[pos[i]] = key[i];
        s.values[pos[i]] = val[i];
    }
    __syncthreads();

    // coalesced write-out: consecutive staged slots of one digit go to consecutive addresses.
    // Padding keys (0xFFFFFFFF) rank behind every real key of the last tile, i.e. at slots >= valid.
    for (int q = tid; q < valid; q += kThreads) {
        const uint32_t k = s.keys[q];
        const unsigned d = (k >> shift) & digit_mask;
        const unsigned dst = s.global_off[d] + (unsigned)q;
        // always true in a healthy sort.  After a look-back that gave up, a later pass meets keys whose digits no
        // longer match the histogram taken up front, and its positions can then run past the end: drop those.
        if (dst < (unsigned)n) {
            keys_out[dst] = k;
            vals_out[dst] = s.values[q];
        }
    }
}

struct SortWorkspace {
    unsigned* hist;     // [kMaxPasses][kRadix]
    unsigned* ticket;   // [kMaxPasses]
    unsigned* base;     // [kMaxPasses][kRadix]
    unsigned* state;    // [kMaxPasses][tiles][kRadix]
    size_t zero_bytes;  // leading bytes that must be cleared per sort (hist + ticket)
    size_t state_bytes;
    size_t total;
};

SortWorkspace carve_sort_workspace(void* ws, int64_t n) {
    SortWorkspace w;
    const int64_t tiles = n > 0 ? ceil_div<int64_t>(n, kTile) : 1;
    Carver c(ws);
    w.hist = c.take<unsigned>(kMaxPasses * kRadix);
    w.ticket = c.take<unsigned>(64);
    w.zero_bytes = c.used();
    w.state = c.take<unsigned>((size_t)kMaxPasses * tiles * kRadix);
    w.state_bytes = c.used() - w.zero_bytes;
    w.base = c.take<unsigned>(kMaxPasses * kRadix);
    w.total = c.used();
    return w;
}


struct PassArgs {
    int64_t tiles;
    const uint32_t *kin, *vin;
    uint32_t *kout, *vout;
    int64_t n;
    const unsigned long long* n_dev;
    int shift, bits;
    const unsigned* base;
    unsigned *state, *ticket, *status;
    int spin_limit;        // polls a tile spends on one unpublished predecessor before it gives up
    unsigned mute_tile;    // tile that never publishes (tests only); 0xFFFFFFFF = none
};

template <int BITS>
int launch_onesweep_instance(const PassArgs& a, cudaStream_t stream) {
    static bool attr_set[kMaxDevices] = {false};
    static std::mutex attr_mutex;
    constexpr size_t kSmemBytes = sizeof(PassSmem);
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        const int rc = opt_in_dynamic_smem(radix_onesweep_pass_kernel<BITS>, kSmemBytes, attr_set);
        if (rc != INPC_OK) return rc;
    }
    radix_onesweep_pass_kernel<BITS><<<(unsigned)a.tiles, kThreads, kSmemBytes, stream>>>(a.kin, a.vin, a.kout, a.vout, a.n, a.n_dev, a.shift, a.bits, a.base,
                                                                                         a.state, a.ticket, a.status, a.spin_limit, a.mute_tile);
    INPC_LAUNCH_CHECK("radix_onesweep_pass_kernel");
    return INPC_OK;
}

// the digit widths the rasterizer's sorts use (depth keys 9/8, tile keys 7) get unrolled kernels
int launch_onesweep_pass(const PassArgs& a, cudaStream_t stream) {
    switch (a.bits) {
        case 7: return launch_onesweep_instance<7>(a, stream);
        case 8: return launch_onesweep_instance<8>(a, stream);
        case 9: return launch_onesweep_instance<9>(a, stream);
        default: return launch_onesweep_instance<0>(a, stream);
    }
}

}  // namespace

size_t sort_workspace_bytes(int64_t n) { return carve_sort_workspace(nullptr, n).total; }

int sort_pass_count(int end_bit) { return end_bit > 0 ? ceil_div(end_bit, kRadixBits) : 0; }

// Argument checks shared by the entry points; *nothing_to_do is set when the call is valid but makes no pass.
static int check_sort_args(const char* who, const uint32_t* keys, const uint32_t* keys_alt, const uint32_t* values, const uint32_t* values_alt,
                           int64_t n, int end_bit, bool* nothing_to_do) {
    *nothing_to_do = false;
    if (n < 0 || n >= (int64_t)1 << 30) { set_error("%s: n=%lld out of range [0, 2^30)", who, (long long)n); return INPC_E_INVALID; }
    if (end_bit < 0 || end_bit > 32) { set_error("%s: end_bit=%d out of range", who, end_bit); return INPC_E_INVALID; }
    if (n <= 1 || end_bit == 0) { *nothing_to_do = true; return INPC_OK; }
    if (!keys || !keys_alt || !values || !values_alt) { set_error("%s: null pointer", who); return INPC_E_INVALID; }
    if ((reinterpret_cast<uintptr_t>(keys) | reinterpret_cast<uintptr_t>(keys_alt)) & 15u) {
        set_error("%s: key buffers must be 16-byte aligned", who);
        return INPC_E_INVALID;
    }
    return INPC_OK;
}

// The sort proper: `workspace` holds sort_workspace_bytes(n) bytes, `status` is the device address of the
// status words a tile that gives up its look-back writes to.  Every entry point ends up here.
static int sort_pairs_with(const char* who, uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n, int end_bit,
                           void* workspace, unsigned* status, int* result_in_alt, cudaStream_t stream, int spin_limit = kSpinLimit,
                           unsigned mute_tile = 0xFFFFFFFFu, const unsigned long long* n_dev = nullptr) {
    if (result_in_alt) *result_in_alt = 0;
    if (!workspace || !status) { set_error("%s: null workspace", who); return INPC_E_INVALID; }

    PassTable pt;
    pt.n_passes = ceil_div(end_bit, kRadixBits);
    int bit = 0;
    for (int p = 0; p < kMaxPasses; ++p) { pt.shift[p] = 0; pt.bits[p] = 0; }
    for (int p = 0; p < pt.n_passes; ++p) {
        // spread the bits evenly over the passes (e.g. 12 bits -> 6 + 6): fewer digits per pass
        // means longer, better-coalesced output runs
        const int b = (end_bit - bit + (pt.n_passes - p) - 1) / (pt.n_passes - p);
        pt.shift[p] = bit;
        pt.bits[p] = b;
        bit += b;
    }

    SortWorkspace w = carve_sort_workspace(workspace, n);
    const int64_t tiles = ceil_div<int64_t>(n, kTile);
    // hist, tickets and the look-back state are contiguous at the front of the workspace; a workspace that
    // is reused keeps the previous call's contents, so everything this call reads is cleared first
    INPC_CUDA_TRY(cudaMemsetAsync(workspace, 0, w.zero_bytes + (size_t)pt.n_passes * tiles * kRadix * sizeof(unsigned), stream));

    const int hist_blocks = (int)ceil_div<int64_t>(n, kHistItemsPerBlock);
    radix_histogram_kernel<<<hist_blocks, kHistThreads, 0, stream>>>(keys, n, n_dev, pt, w.hist);
    INPC_LAUNCH_CHECK("radix_histogram_kernel");
    radix_scan_histogram_kernel<<<pt.n_passes, kRadix, 0, stream>>>(w.hist, w.base);
    INPC_LAUNCH_CHECK("radix_scan_histogram_kernel");

    PassArgs a;
    a.tiles = tiles; a.n = n; a.n_dev = n_dev; a.status = status;
    a.spin_limit = spin_limit; a.mute_tile = mute_tile;
    a.kin = keys; a.kout = keys_alt; a.vin = values; a.vout = values_alt;
    for (int p = 0; p < pt.n_passes; ++p) {
        a.shift = pt.shift[p]; a.bits = pt.bits[p];
        a.base = w.base + p * kRadix;
        a.state = w.state + (size_t)p * tiles * kRadix;
        a.ticket = w.ticket + p;
        const int rc = launch_onesweep_pass(a, stream);
        if (rc != INPC_OK) return rc;
        const uint32_t* t = a.kin; a.kin = a.kout; a.kout = const_cast<uint32_t*>(t);
        t = a.vin; a.vin = a.vout; a.vout = const_cast<uint32_t*>(t);
    }
    if (result_in_alt) *result_in_alt = pt.n_passes & 1;
    return INPC_OK;
}

int sort_pairs(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n,
               int end_bit, void* workspace, unsigned* status, int* result_in_alt, cudaStream_t stream) {
    if (result_in_alt) *result_in_alt = 0;
    bool nothing = false;
    const int rc = check_sort_args("sort_pairs", keys, keys_alt, values, values_alt, n, end_bit, &nothing);
    if (rc != INPC_OK || nothing) return rc;
    if (!workspace) { set_error("sort_pairs: null workspace"); return INPC_E_INVALID; }
    return sort_pairs_with("sort_pairs", keys, keys_alt, values, values_alt, n, end_bit, workspace, status, result_in_alt, stream);
}

// The same sort with the number of pairs in device memory (*n_dev <= n_max): grids and the look-back state are
// sized for n_max, the kernels read the count themselves, and the result is always in the alternate buffers iff
// the number of passes is odd.  No host synchronisation anywhere.
int sort_pairs_device_count(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n_max,
                            const unsigned long long* n_dev, int end_bit, void* workspace, unsigned* status, int* result_in_alt,
                            cudaStream_t stream) {
    if (result_in_alt) *result_in_alt = 0;
    if (n_max <= 0 || end_bit == 0) return INPC_OK;
    bool nothing = false;
    const int rc = check_sort_args("sort_pairs", keys, keys_alt, values, values_alt, n_max < 2 ? 2 : n_max, end_bit, &nothing);
    if (rc != INPC_OK) return rc;
    if (!workspace || !n_dev) { set_error("sort_pairs: null workspace or count"); return INPC_E_INVALID; }
    return sort_pairs_with("sort_pairs", keys, keys_alt, values, values_alt, n_max, end_bit, workspace, status, result_in_alt, stream, kSpinLimit,
                           0xFFFFFFFFu, n_dev);
}

}  // namespace inpc

// ---- sorting without any allocation -------------------------------------------------------------
// Scratch for inpc_sort_pairs_static lives in this fixed device array: every GPU that loads the library
// holds it (about 1 MB) until the process exits.  Layout = the ordinary sort workspace for
// kStaticMaxPairs pairs, followed by one 256-byte status area.
namespace inpc {
namespace {
constexpr int64_t kStaticMaxPairs = 1 << 20;
constexpr size_t kStaticTiles = (kStaticMaxPairs + kTile - 1) / kTile;
constexpr size_t kStaticWorkspaceBytes = (kMaxPasses * kRadix * 4 + 256)            // histograms + tickets
                                         + kMaxPasses * kStaticTiles * kRadix * 4   // look-back state
                                         + kMaxPasses * kRadix * 4;                 // digit bases
constexpr size_t kStaticScratchBytes = kStaticWorkspaceBytes + 256;
static_assert(kStaticWorkspaceBytes % 256 == 0, "status area must stay 256-byte aligned");

static __device__ __align__(256) unsigned char g_static_sort_scratch[kStaticScratchBytes];

std::mutex g_static_mutex;
void* g_static_scratch_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device

// Once per device, with that device current: resolve the array's device address.  In host code the
// array's name is only a handle for the runtime, not an address a kernel could use.
int static_scratch_for_current_device(void** out) {
    int dev = -1;
    INPC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) { set_error("device index %d outside the supported range", dev); return INPC_E_INVALID; }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_scratch_ptr[dev]) {
        void* p = nullptr;
        INPC_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_sort_scratch));
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return INPC_OK;
}
}  // namespace
}  // namespace inpc

extern "C" int inpc_sort_pairs_static(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt,
                                      int64_t n, int end_bit, int* result_in_alt, void* stream_) {
    using namespace inpc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (result_in_alt) *result_in_alt = 0;
    if (n > kStaticMaxPairs) {
        set_error("inpc_sort_pairs_static: n=%lld exceeds the fixed capacity of %lld pairs; use inpc_sort_pairs with a caller workspace",
                  (long long)n, (long long)kStaticMaxPairs);
        return INPC_E_CAPACITY;
    }
    // the hand-written size of the fixed array must be what the ordinary workspace layout needs at capacity
    if (sort_workspace_bytes(kStaticMaxPairs) != kStaticWorkspaceBytes) {
        set_error("inpc_sort_pairs_static: fixed scratch of %zu bytes does not match the workspace layout (%zu bytes)",
                  kStaticWorkspaceBytes, sort_workspace_bytes(kStaticMaxPairs));
        return INPC_E_INVALID;
    }
    bool nothing = false;
    int rc = check_sort_args("inpc_sort_pairs_static", keys, keys_alt, values, values_alt, n, end_bit, &nothing);
    if (rc != INPC_OK || nothing) return rc;
    void* scratch = nullptr;
    rc = static_scratch_for_current_device(&scratch);
    if (rc != INPC_OK) return rc;
    // the status words of this entry point live behind the workspace, inside the same fixed array
    unsigned* status = reinterpret_cast<unsigned*>(static_cast<unsigned char*>(scratch) + kStaticWorkspaceBytes);
    INPC_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(unsigned) * STATUS_WORDS, stream));
    return sort_pairs_with("inpc_sort_pairs_static", keys, keys_alt, values, values_alt, n, end_bit, scratch, status, result_in_alt, stream);
}

extern "C" size_t inpc_sort_workspace_bytes(int64_t n) { return inpc::sort_workspace_bytes(n < 0 ? 0 : n); }

extern "C" int inpc_sort_pairs(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt,
                               int64_t n, int end_bit, void* workspace, int* result_in_alt, void* stream) {
    using namespace inpc;
    if (result_in_alt) *result_in_alt = 0;
    bool nothing = false;
    int rc = check_sort_args("inpc_sort_pairs", keys, keys_alt, values, values_alt, n, end_bit, &nothing);
    if (rc != INPC_OK || nothing) return rc;
    if (!workspace) { set_error("inpc_sort_pairs: null workspace"); return INPC_E_INVALID; }
    rc = check_previous_calls();
    if (rc != INPC_OK) return rc;
    unsigned* status = acquire_status("inpc_sort_pairs");
    if (!status) return INPC_E_CUDA;
    return sort_pairs(keys, keys_alt, values, values_alt, n, end_bit, workspace, status, result_in_alt, static_cast<cudaStream_t>(stream));
}

// Test hook: inpc_sort_pairs with tile 0 of every pass leaving before it publishes its digit counts and a
// look-back limit of 2^10 polls.  The tiles behind it give up within microseconds, report through the call's
// status words, publish what they have and finish: every access stays inside the buffers (the write-out
// checks its destination against n), the output is simply not sorted.  Returns the call's status ticket in *ticket.
extern "C" int inpc_debug_sort_lookback_timeout(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt,
                                                int64_t n, int end_bit, void* workspace, long long* ticket, void* stream) {
    using namespace inpc;
    bool nothing = false;
    int rc = check_sort_args("inpc_debug_sort_lookback_timeout", keys, keys_alt, values, values_alt, n, end_bit, &nothing);
    if (rc != INPC_OK) return rc;
    if (nothing || !workspace || !ticket) { set_error("inpc_debug_sort_lookback_timeout: needs n > 1, end_bit > 0, a workspace and a ticket pointer"); return INPC_E_INVALID; }
    unsigned* status = acquire_status("inpc_debug_sort_lookback_timeout", ticket);
    if (!status) return INPC_E_CUDA;
    return sort_pairs_with("inpc_debug_sort_lookback_timeout", keys, keys_alt, values, values_alt, n, end_bit, workspace, status, nullptr,
                           static_cast<cudaStream_t>(stream), 1 << 10, 0u);
}

// Status words of the last inpc_sort_pairs_static call on the current device, copied out of the fixed array
// after `stream` has been synchronised (no allocation here either).
extern "C" int inpc_sort_pairs_static_status(void* stream_, unsigned* words) {
    using namespace inpc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!words) { set_error("inpc_sort_pairs_static_status: null argument"); return INPC_E_INVALID; }
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != INPC_OK) return rc;
    unsigned host[STATUS_WORDS];
    INPC_CUDA_TRY(cudaMemcpyAsync(host, static_cast<unsigned char*>(scratch) + kStaticWorkspaceBytes, sizeof(host), cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    for (int k = 0; k < (int)STATUS_WORDS; ++k) words[k] = host[k];
    if (host[STATUS_LOOKBACK_TIMEOUT]) {
        set_error("inpc_sort_pairs_static: a radix-sort tile gave up waiting for a predecessor tile; the results of that call are invalid");
        return INPC_E_DEVICE;
    }
    return INPC_OK;
}
