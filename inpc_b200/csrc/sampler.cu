// Probability-field sampler of the inpc_b200 library.
//
// Per-view leaf weights -> normalised fp32 CDF (deterministic block scans) -> per-slot draws from a
// counter-based Philox4x32-10 stream: one Philox block yields the CDF uniform and the three jitter
// uniforms of a draw.  Every output slot owns its own sub-stream (seed, call, slot, attempt), so the
// training sampler needs no atomics and is reproducible; the reference's rejection sampler hands out
// slots with an atomic ticket and is not (sampling/src/sampling_kernels.cu:104-125).
// Citations are paths below INPCCudaBackend/INPCCudaBackend/sampling/ of the reference.
#include "common.cuh"

namespace inpc {

namespace {

constexpr float kEps = 1e-8f;   // FLT_EPS of the reference's utils.h:8
constexpr int kThreads = 256;
constexpr int kMaxAttempts = 4096;

// ---- viewpoint weights: src/sampling_kernels.cu:9-64 ----------------------------------------
struct Rows {
    float r0[4], r1[4], r2[4];
};
__device__ __forceinline__ Rows load_rows(const float* __restrict__ w2c) {
    Rows m;
#pragma unroll
    for (int k = 0; k < 4; ++k) { m.r0[k] = __ldg(w2c + k); m.r1[k] = __ldg(w2c + 4 + k); m.r2[k] = __ldg(w2c + 8 + k); }
    return m;
}

// All sampler arithmetic spells out its fused multiply-adds, so that the CPU restatement used by the
// tests reproduces every value bit for bit.
__device__ __forceinline__ float affine(const float* r, float x, float y, float z) {
    return fmaf(r[2], z, fmaf(r[1], y, fmaf(r[0], x, r[3])));
}

__device__ __forceinline__ bool in_frustum(const Rows& m, const ViewParams& v, float px, float py, float pz, float* z_out) {
    const float vx = affine(m.r0, px, py, pz);
    const float vy = affine(m.r1, px, py, pz);
    const float z = affine(m.r2, px, py, pz);
    const float inv_z = 1.0f / (z + kEps);
    const float x = fmaf(vx * inv_z, v.fx, v.cx);
    const float y = fmaf(vy * inv_z, v.fy, v.cy);
    if (z_out) *z_out = z;
    return (z >= v.near_plane) & (z <= v.far_plane) & (x >= 0.0f) & (x < (float)v.width) & (y >= 0.0f) & (y < (float)v.height);
}

__global__ void __launch_bounds__(kThreads) viewpoint_weights_kernel(ViewParams v, int64_t n_cells,
                                                                     const float* __restrict__ centers,
                                                                     const int* __restrict__ levels,
                                                                     const float* __restrict__ weights,
                                                                     float initial_size, float* __restrict__ out,
                                                                     float4* __restrict__ leaf_pack) {
    const int64_t l = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (l >= n_cells) return;
    const Rows m = load_rows(v.w2c);
    const float cx = __ldg(centers + 3 * l), cy = __ldg(centers + 3 * l + 1), cz = __ldg(centers + 3 * l + 2);
    const int level = __ldg(levels + l);
    float z;
    bool valid = in_frustum(m, v, cx, cy, cz, &z);
    if (!valid) {
        const float half_size = initial_size / scalbnf(1.0f, level + 1);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float ox = (k & 4) ? 1.0f : -1.0f, oy = (k & 2) ? 1.0f : -1.0f, oz = (k & 1) ? 1.0f : -1.0f;
            valid |= in_frustum(m, v, fmaf(half_size, ox, cx), fmaf(half_size, oy, cy), fmaf(half_size, oz, cz), nullptr);
        }
    }
    float w = 0.0f;
    if (valid) {
        const float depth_scale = fmaxf(fabsf(z - v.near_plane) / v.far_plane, kEps);
        // 2^(level/2), exact: the reference's exp2f(level * 0.5f) agrees to within the 2 ulp of exp2f
        const float size_scale = scalbnf((level & 1) ? 1.41421356237309504880f : 1.0f, level >> 1);
        w = 1.0f / (depth_scale * size_scale) * __ldg(weights + l);
    }
    out[l] = w;
    // centre and edge length in one 16-byte record: a draw then needs one load per leaf instead of four
    if (leaf_pack) leaf_pack[l] = make_float4(cx, cy, cz, 1.0f / scalbnf(1.0f, level) * initial_size);
}

// ---- CDF: src/sampling.cu:97-125 (Sum, multiply by 1/sum, InclusiveSum) -------------------------
// The reference scans fp32 values with CUB, whose summation order is unspecified.  Here every weight
// is first expressed as a 39-bit fixed-point fraction of the largest weight; integer prefix sums are
// exact and associative, so the CDF is independent of how the scan is parallelised, monotone, and
// reproducible bit for bit anywhere (the CPU restatement is a plain loop):
//   q_i = trunc(w_i / w_max * 2^39),  P_i = q_0 + ... + q_i,  cdf_i = float(P_i / P_last),
//   sum = float(P_last * 2^-39 * w_max).
constexpr int kCdfThreads = 256;
constexpr int kCdfItems = 8;
constexpr int kCdfChunk = kCdfThreads * kCdfItems;
constexpr float kFixedOne = 549755813888.0f;   // 2^39
constexpr double kFixedInv = 1.0 / 549755813888.0;

// Non-finite and non-positive weights count as zero (an infinite one would make the quotient NaN, whose
// conversion to an integer is undefined).
__device__ __forceinline__ unsigned long long to_fixed(float w, float w_max) {
    return (w > 0.0f && w <= 3.402823466e38f) ? (unsigned long long)((w / w_max) * kFixedOne) : 0ull;
}

// largest weight via atomicMax on the bit pattern (valid for non-negative floats; order-free)
__global__ void __launch_bounds__(kCdfThreads) cdf_max_kernel(const float* __restrict__ w, int64_t n, unsigned* __restrict__ max_bits) {
    const int64_t base = (int64_t)blockIdx.x * kCdfChunk + (int64_t)threadIdx.x * kCdfItems;
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < kCdfItems; ++k)
        if (base + k < n) {
            const float v = __ldg(w + base + k);
            if (v <= 3.402823466e38f) m = fmaxf(m, v);   // NaN and +inf do not take part
        }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_down_sync(0xffffffffu, m, o));
    if (lane_id() == 0 && m > 0.0f) atomicMax(max_bits, __float_as_uint(m));
}

__device__ __forceinline__ unsigned long long warp_inclusive_scan_u64(unsigned long long v) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane_id() >= (unsigned)o) v += t;
    }
    return v;
}

// exclusive scan of one u64 per thread over the block; smem needs blockDim/32 + 1 entries
__device__ __forceinline__ unsigned long long block_exclusive_scan_u64(unsigned long long v, unsigned long long* smem,
                                                                     unsigned long long* total) {
    const unsigned lane = lane_id(), warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    const unsigned long long inc = warp_inclusive_scan_u64(v);
    if (lane == 31) smem[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        const unsigned long long wv = lane < nwarps ? smem[lane] : 0ull;
        const unsigned long long winc = warp_inclusive_scan_u64(wv);
        if (lane < nwarps) smem[lane] = winc - wv;
        if (lane == 31) smem[nwarps] = winc;
    }
    __syncthreads();
    const unsigned long long r = smem[warp] + inc - v;
    *total = smem[nwarps];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(kCdfThreads) cdf_chunk_sums_kernel(const float* __restrict__ w, int64_t n,
                                                                     const unsigned* __restrict__ max_bits,
                                                                     unsigned long long* __restrict__ chunk_sums) {
    __shared__ unsigned long long s[kCdfThreads / 32 + 1];
    const float w_max = __uint_as_float(__ldg(max_bits));
    const int64_t base = (int64_t)blockIdx.x * kCdfChunk + (int64_t)threadIdx.x * kCdfItems;
    unsigned long long acc = 0;
#pragma unroll
    for (int k = 0; k < kCdfItems; ++k)
        if (base + k < n) acc += to_fixed(__ldg(w + base + k), w_max);
    unsigned long long total;
    block_exclusive_scan_u64(acc, s, &total);
    if (threadIdx.x == 0) chunk_sums[blockIdx.x] = total;
}

// one block: exclusive scan of the chunk sums in place; total -> *total_out, fp32 sum -> *sum_out
__global__ void __launch_bounds__(1024) cdf_scan_chunks_kernel(unsigned long long* __restrict__ chunk_sums, int64_t n_chunks,
                                                               const unsigned* __restrict__ max_bits,
                                                               unsigned long long* __restrict__ total_out,
                                                               float* __restrict__ sum_out) {
    __shared__ unsigned long long s[1024 / 32 + 1];
    unsigned long long running = 0;
    for (int64_t base = 0; base < n_chunks; base += 1024) {
        const int64_t j = base + threadIdx.x;
        const unsigned long long c = j < n_chunks ? chunk_sums[j] : 0ull;
        unsigned long long total;
        const unsigned long long ex = block_exclusive_scan_u64(c, s, &total);
        if (j < n_chunks) chunk_sums[j] = running + ex;
        running += total;
    }
    if (threadIdx.x == 0) {
        *total_out = running;
        *sum_out = (float)((double)running * kFixedInv * (double)__uint_as_float(*max_bits));
    }
}

__global__ void __launch_bounds__(kCdfThreads) cdf_finalize_kernel(const float* __restrict__ w, int64_t n,
                                                                   const unsigned* __restrict__ max_bits,
                                                                   const unsigned long long* __restrict__ chunk_base,
                                                                   const unsigned long long* __restrict__ total_ptr,
                                                                   float* __restrict__ cdf) {
    __shared__ unsigned long long s[kCdfThreads / 32 + 1];
    const float w_max = __uint_as_float(__ldg(max_bits));
    const double total = (double)__ldg(total_ptr);
    const int64_t base = (int64_t)blockIdx.x * kCdfChunk + (int64_t)threadIdx.x * kCdfItems;
    unsigned long long q[kCdfItems];
    unsigned long long acc = 0;
#pragma unroll
    for (int k = 0; k < kCdfItems; ++k) {
        acc += base + k < n ? to_fixed(__ldg(w + base + k), w_max) : 0ull;
        q[k] = acc;
    }
    unsigned long long block_total;
    const unsigned long long before = __ldg(chunk_base + blockIdx.x) + block_exclusive_scan_u64(acc, s, &block_total);
#pragma unroll
    for (int k = 0; k < kCdfItems; ++k)
        if (base + k < n) cdf[base + k] = (float)((double)(before + q[k]) / total);
}

// ---- Philox4x32-10 ----------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
        k.x += 0x9E3779B9u;
        k.y += 0xBB67AE85u;
    }
    return c;
}

// 23 random mantissa bits -> [0,1), the mapping of include/pcg32.h:105-114
__device__ __forceinline__ float unit_float(unsigned r) { return __uint_as_float((r >> 9) | 0x3f800000u) - 1.0f; }

struct Draw {
    float u, jx, jy, jz;
    unsigned raw_u;   // the 32 bits u was made of
};
// stream layout: counter = (slot, attempt, call lo, call hi), key = seed (lo, hi)
__device__ __forceinline__ Draw philox_draw(unsigned long long seed, unsigned long long call, unsigned slot, unsigned attempt) {
    const uint4 o = philox4x32_10(make_uint4(slot, attempt, (unsigned)call, (unsigned)(call >> 32)),
                                  make_uint2((unsigned)seed, (unsigned)(seed >> 32)));
    Draw d;
    d.u = unit_float(o.x); d.jx = unit_float(o.y); d.jy = unit_float(o.z); d.jz = unit_float(o.w);
    d.raw_u = o.x;
    return d;
}

// first index with cdf[idx] >= u, clamped to n-1: include/sampling_utils.h:49-69
__device__ __forceinline__ unsigned lower_bound_clamped(const float* __restrict__ cdf, float u, unsigned n) {
    unsigned first = 0, count = n;
    while (count > 0) {
        const unsigned step = count >> 1;
        if (__ldg(cdf + first + step) < u) { first += step + 1; count -= step + 1; }
        else count = step;
    }
    return min(first, n - 1);
}

// Guide table: guide[b] = lower_bound(cdf, b / 2^k) for b = 0 .. 2^k.  The CDF is monotone (integer
// prefix sums), so the look-up for a uniform in bucket b only has to search [guide[b], guide[b+1]):
// about L / 2^k entries instead of log2(L) dependent loads, with bit-identical results.
__global__ void __launch_bounds__(kThreads) guide_table_kernel(const float* __restrict__ cdf, unsigned n_cells, int k,
                                                               unsigned* __restrict__ guide) {
    const unsigned b = blockIdx.x * kThreads + threadIdx.x;
    if (b > (1u << k)) return;
    // bucket edge as a float: (b << (23 - k)) * 2^-23, exact
    const float edge = (float)(b << (23 - k)) * 1.1920928955078125e-07f;
    unsigned first = 0, count = n_cells;
    while (count > 0) {
        const unsigned step = count >> 1;
        if (__ldg(cdf + first + step) < edge) { first += step + 1; count -= step + 1; }
        else count = step;
    }
    guide[b] = first;
}

// r: the raw 32 random bits the uniform is made of (u = (r >> 9) * 2^-23)
__device__ __forceinline__ unsigned guided_lower_bound(const float* __restrict__ cdf, const unsigned* __restrict__ guide, int k,
                                                       unsigned r, float u, unsigned n) {
    const unsigned b = (r >> 9) >> (23 - k);
    const uint2 g = make_uint2(__ldg(guide + b), __ldg(guide + b + 1));
    unsigned first = g.x, count = g.y - g.x;
    while (count > 0) {
        const unsigned step = count >> 1;
        if (__ldg(cdf + first + step) < u) { first += step + 1; count -= step + 1; }
        else count = step;
    }
    return min(first, n - 1);
}

__device__ __forceinline__ float leaf_scale(int level, float initial_size) {
    return 1.0f / scalbnf(1.0f, level) * initial_size;
}

// ---- training samples: same acceptance test as src/sampling_kernels.cu:98-113 -------------------
__global__ void __launch_bounds__(kThreads) training_samples_kernel(
    ViewParams v, unsigned long long seed, unsigned long long call, const float* __restrict__ cdf,
    const unsigned* __restrict__ guide, int guide_bits, const float* __restrict__ sum_ptr, unsigned n_cells,
    const float4* __restrict__ leaf_pack, int64_t n_samples, float* __restrict__ positions, long long* __restrict__ indices,
    volatile unsigned* status) {
    const int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (s >= n_samples) return;
    if (!(__ldg(sum_ptr) > 0.0f)) {
        // src/sampling.cu:107-111: zero positions, indices of -1
        positions[3 * s] = 0.0f; positions[3 * s + 1] = 0.0f; positions[3 * s + 2] = 0.0f;
        indices[s] = -1;
        return;
    }
    const Rows m = load_rows(v.w2c);
    unsigned leaf = 0;
    float x = 0.0f, y = 0.0f, z = 0.0f;
    bool ok = false;
    for (unsigned a = 0; a < (unsigned)kMaxAttempts && !ok; ++a) {
        const Draw d = philox_draw(seed, call, (unsigned)s, a);
        leaf = guided_lower_bound(cdf, guide, guide_bits, d.raw_u, d.u, n_cells);
        const float4 lp = __ldg(leaf_pack + leaf);
        x = fmaf(d.jx - 0.5f, lp.w, lp.x);
        y = fmaf(d.jy - 0.5f, lp.w, lp.y);
        z = fmaf(d.jz - 0.5f, lp.w, lp.z);
        const float vz = affine(m.r2, x, y, z);
        if (vz < v.near_plane || vz > v.far_plane) continue;
        const float inv_z = 1.0f / (vz + kEps);
        const float sx = fmaf(affine(m.r0, x, y, z) * inv_z, v.fx, v.cx);
        if (sx < 0.0f || sx >= (float)v.width) continue;
        const float sy = fmaf(affine(m.r1, x, y, z) * inv_z, v.fy, v.cy);
        if (sy < 0.0f || sy >= (float)v.height) continue;
        ok = true;
    }
    if (!ok) status[STATUS_SAMPLER_EXHAUSTED] = 1u;
    positions[3 * s] = x; positions[3 * s + 1] = y; positions[3 * s + 2] = z;
    indices[s] = (long long)leaf;
}

// ---- unconditional samples: src/sampling_kernels.cu:128-150 with the Philox stream ----------------
__global__ void __launch_bounds__(kThreads) samples_kernel(unsigned long long seed, unsigned long long call,
                                                           const float* __restrict__ cdf, const unsigned* __restrict__ guide,
                                                           int guide_bits, unsigned n_cells,
                                                           const float4* __restrict__ leaf_pack, int64_t n_samples,
                                                           float* __restrict__ positions) {
    const int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (s >= n_samples) return;
    const Draw d = philox_draw(seed, call, (unsigned)s, 0u);
    const unsigned leaf = guided_lower_bound(cdf, guide, guide_bits, d.raw_u, d.u, n_cells);
    const float4 lp = __ldg(leaf_pack + leaf);
    positions[3 * s] = fmaf(d.jx - 0.5f, lp.w, lp.x);
    positions[3 * s + 1] = fmaf(d.jy - 0.5f, lp.w, lp.y);
    positions[3 * s + 2] = fmaf(d.jz - 0.5f, lp.w, lp.z);
}

__global__ void __launch_bounds__(kThreads) draw_leaves_kernel(const float* __restrict__ cdf, unsigned n_cells,
                                                               const float* __restrict__ u, int64_t n,
                                                               long long* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    out[i] = (long long)lower_bound_clamped(cdf, __ldg(u + i), n_cells);
}

// ---- expected samples: src/sampling_kernels.cu:152-205 ----------------------------------------
__global__ void __launch_bounds__(kThreads) sample_counts_kernel(const float* __restrict__ vw, const float* __restrict__ sum_ptr,
                                                                 unsigned n_samples, int64_t n_cells, unsigned* __restrict__ counts) {
    const int64_t l = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (l >= n_cells) return;
    const float w = __ldg(vw + l);
    const float sum = __ldg(sum_ptr);
    int c = 0;
    if (w > 0.0f && sum > 0.0f) {
        const float norm = 1.0f / sum;
        c = max(__float2int_rn(w * norm * static_cast<float>(n_samples)), 1);
    }
    counts[l] = (unsigned)c;
}

constexpr int kIScanThreads = 1024;
// in-place inclusive scan of per-chunk sums is not needed: the counts array is small enough for a
// two-level scheme (chunk sums by one kernel, one block scans them, one kernel finalises).
__global__ void __launch_bounds__(kThreads) count_chunk_sums_kernel(const unsigned* __restrict__ counts, int64_t n,
                                                                    unsigned* __restrict__ chunk_sums) {
    __shared__ unsigned s[kThreads / 32];
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    unsigned c = i < n ? counts[i] : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
    if (lane_id() == 0) s[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned t = 0;
        for (int w = 0; w < kThreads / 32; ++w) t += s[w];
        chunk_sums[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(kIScanThreads) scan_chunk_sums_kernel(unsigned* __restrict__ chunk_sums, int64_t n_chunks,
                                                                        unsigned long long* __restrict__ total_out) {
    __shared__ unsigned s_scan[kIScanThreads / 32 + 1];
    unsigned long long running = 0;
    for (int64_t base = 0; base < n_chunks; base += kIScanThreads) {
        const int64_t j = base + threadIdx.x;
        const unsigned c = j < n_chunks ? chunk_sums[j] : 0u;
        unsigned total;
        const unsigned ex = block_exclusive_scan(c, s_scan, &total);
        if (j < n_chunks) chunk_sums[j] = (unsigned)running + ex;
        running += total;
    }
    if (threadIdx.x == 0) *total_out = running;
}

// offsets[l] = inclusive prefix of counts (the reference's sample_offsets)
__global__ void __launch_bounds__(kThreads) count_offsets_kernel(const unsigned* __restrict__ counts, int64_t n,
                                                                 const unsigned* __restrict__ chunk_base,
                                                                 unsigned* __restrict__ offsets) {
    __shared__ unsigned s_scan[kThreads / 32 + 1];
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const unsigned c = i < n ? counts[i] : 0u;
    unsigned total;
    const unsigned ex = block_exclusive_scan(c, s_scan, &total);
    if (i < n) offsets[i] = chunk_base[blockIdx.x] + ex + c;
}

// slot i jitters inside leaf upper_bound(offsets, i % n_created): the load-balanced form of the
// reference's per-leaf fill loop + gather
__global__ void __launch_bounds__(kThreads) expected_samples_kernel(unsigned long long seed, unsigned long long call,
                                                                    const unsigned* __restrict__ offsets, unsigned n_cells,
                                                                    const float* __restrict__ centers, const int* __restrict__ levels,
                                                                    float initial_size, int64_t n_total, unsigned n_created,
                                                                    float* __restrict__ positions) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n_total) return;
    const unsigned r = (unsigned)(i % n_created);
    // first leaf whose inclusive offset exceeds r
    unsigned first = 0, count = n_cells;
    while (count > 0) {
        const unsigned step = count >> 1;
        if (__ldg(offsets + first + step) <= r) { first += step + 1; count -= step + 1; }
        else count = step;
    }
    const unsigned leaf = min(first, n_cells - 1);
    const Draw d = philox_draw(seed, call, (unsigned)i, 0u);
    const float scale = leaf_scale(__ldg(levels + leaf), initial_size);
    positions[3 * i] = fmaf(d.jx - 0.5f, scale, __ldg(centers + 3 * (int64_t)leaf));
    positions[3 * i + 1] = fmaf(d.jy - 0.5f, scale, __ldg(centers + 3 * (int64_t)leaf + 1));
    positions[3 * i + 2] = fmaf(d.jz - 0.5f, scale, __ldg(centers + 3 * (int64_t)leaf + 2));
}

// ---- global point cloud: Modules/ProbabilityField.py:121-144 + utils.py:36-64 -----------------------
// counts[leaf] = number of the n multinomial draws that fell into the leaf (torch.multinomial +
// bincount in the reference; here the library's own Philox stream, one draw per slot)
__global__ void __launch_bounds__(kThreads) leaf_histogram_kernel(unsigned long long seed, unsigned long long call,
                                                                  const float* __restrict__ cdf, const unsigned* __restrict__ guide,
                                                                  int guide_bits, unsigned n_cells, int64_t n_samples,
                                                                  unsigned* __restrict__ counts) {
    const int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (s >= n_samples) return;
    const Draw d = philox_draw(seed, call, (unsigned)s, 0u);
    atomicAdd(counts + guided_lower_bound(cdf, guide, guide_bits, d.raw_u, d.u, n_cells), 1u);
}

// Element `index` (1-based) of the Halton sequence in `base`, with the reference's arithmetic
// (utils.py:36-46): double precision, one rounding per product, sum and division; the value is then
// stored as float32 (utils.py:52-55).
__device__ __forceinline__ float halton_element(unsigned index, unsigned base) {
    double result = 0.0;
    double f = __ddiv_rn(1.0, (double)base);
    unsigned i = index;
    while (i > 0u) {
        result = __dadd_rn(result, __dmul_rn(f, (double)(i % base)));
        i /= base;
        f = __ddiv_rn(f, (double)base);
    }
    return __double2float_rn(result);
}

// Sample i lies in leaf upper_bound(offsets, i) and is that leaf's h-th sample, h = i - first sample
// of the leaf: Halton point h+1 in bases (2, 3, 5) scaled into the cell; a leaf with a single sample
// puts it at its centre (ProbabilityField.py:131-140).
__global__ void __launch_bounds__(kThreads) halton_samples_kernel(const unsigned* __restrict__ counts, const unsigned* __restrict__ offsets,
                                                                  unsigned n_cells, const float* __restrict__ centers,
                                                                  const int* __restrict__ levels, float initial_size, int64_t n_total,
                                                                  float* __restrict__ positions) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n_total) return;
    unsigned first = 0, count = n_cells;
    while (count > 0) {
        const unsigned step = count >> 1;
        if (__ldg(offsets + first + step) <= (unsigned)i) { first += step + 1; count -= step + 1; }
        else count = step;
    }
    const unsigned leaf = min(first, n_cells - 1);
    const unsigned c = __ldg(counts + leaf);
    const unsigned h = (unsigned)i - (__ldg(offsets + leaf) - c);
    const float cx = __ldg(centers + 3 * (int64_t)leaf), cy = __ldg(centers + 3 * (int64_t)leaf + 1), cz = __ldg(centers + 3 * (int64_t)leaf + 2);
    if (c == 1u) {
        positions[3 * i] = cx; positions[3 * i + 1] = cy; positions[3 * i + 2] = cz;
        return;
    }
    // cell edge = initial_size / 2^level, exact in fp32 for the levels an octree has; every further
    // operation rounds on its own like the torch expression  centre - cell/2 + halton * cell
    const float cell = __fdiv_rn(initial_size, (float)(1u << __ldg(levels + leaf)));
    const float half = __fmul_rn(cell, 0.5f);
    positions[3 * i] = __fadd_rn(__fsub_rn(cx, half), __fmul_rn(halton_element(h + 1u, 2u), cell));
    positions[3 * i + 1] = __fadd_rn(__fsub_rn(cy, half), __fmul_rn(halton_element(h + 1u, 3u), cell));
    positions[3 * i + 2] = __fadd_rn(__fsub_rn(cz, half), __fmul_rn(halton_element(h + 1u, 5u), cell));
}

// 30-bit Morton code (10 bits per axis, x lowest) of a position inside the box [lo, lo + extent]^3
__device__ __forceinline__ unsigned spread_bits_10(unsigned v) {
    v &= 0x3FFu;
    v = (v | (v << 16)) & 0x030000FFu;
    v = (v | (v << 8)) & 0x0300F00Fu;
    v = (v | (v << 4)) & 0x030C30C3u;
    v = (v | (v << 2)) & 0x09249249u;
    return v;
}

__global__ void __launch_bounds__(kThreads) morton_codes_kernel(const float* __restrict__ positions, int64_t n, float lo_x, float lo_y,
                                                                float lo_z, float inv_extent, unsigned* __restrict__ codes,
                                                                unsigned* __restrict__ order) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    const float qx = (__ldg(positions + 3 * i) - lo_x) * inv_extent * 1024.0f;
    const float qy = (__ldg(positions + 3 * i + 1) - lo_y) * inv_extent * 1024.0f;
    const float qz = (__ldg(positions + 3 * i + 2) - lo_z) * inv_extent * 1024.0f;
    const unsigned x = (unsigned)fminf(fmaxf(qx, 0.0f), 1023.0f), y = (unsigned)fminf(fmaxf(qy, 0.0f), 1023.0f),
                   z = (unsigned)fminf(fmaxf(qz, 0.0f), 1023.0f);
    codes[i] = spread_bits_10(x) | (spread_bits_10(y) << 1) | (spread_bits_10(z) << 2);
    order[i] = (unsigned)i;
}

__global__ void __launch_bounds__(kThreads) gather_positions_kernel(const float* __restrict__ positions, const unsigned* __restrict__ order,
                                                                    int64_t n, float* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    const int64_t j = __ldg(order + i);
    out[3 * i] = __ldg(positions + 3 * j);
    out[3 * i + 1] = __ldg(positions + 3 * j + 1);
    out[3 * i + 2] = __ldg(positions + 3 * j + 2);
}

struct SamplerWs {
    float* vw;          // viewpoint weights (n_cells)
    float* cdf;         // (n_cells)
    unsigned long long* chunk_sums64;   // fixed-point chunk sums / bases
    unsigned long long* total64;        // fixed-point total
    unsigned* max_bits;                 // bit pattern of the largest weight
    float* sum;         // 1 float (+ padding)
    unsigned* counts;   // expected-sample counts (n_cells)
    unsigned* offsets;  // inclusive offsets (n_cells)
    unsigned* chunk_sums;
    unsigned long long* total;
    unsigned* guide;    // 2^guide_bits + 1 entries
    int guide_bits;
    float4* leaf_pack;  // (n_cells) centre + edge length
    size_t bytes;
};

int guide_bits_for(int64_t n_cells) {
    int k = 8;
    while (k < 20 && ((int64_t)1 << k) < n_cells) ++k;
    return k;
}

SamplerWs carve_sampler_ws(void* p, int64_t n_cells) {
    SamplerWs w;
    Carver c(p);
    const int64_t n = n_cells > 0 ? n_cells : 1;
    w.vw = c.take<float>(n);
    w.cdf = c.take<float>(n);
    w.chunk_sums64 = c.take<unsigned long long>(ceil_div<int64_t>(n, kCdfChunk));
    w.total64 = c.take<unsigned long long>(2);
    w.max_bits = c.take<unsigned>(4);
    w.sum = c.take<float>(4);
    w.counts = c.take<unsigned>(n);
    w.offsets = c.take<unsigned>(n);
    w.chunk_sums = c.take<unsigned>(ceil_div<int64_t>(n, kThreads));
    w.total = c.take<unsigned long long>(2);
    w.guide_bits = guide_bits_for(n);
    w.guide = c.take<unsigned>(((size_t)1 << w.guide_bits) + 2);
    w.leaf_pack = c.take<float4>(n);
    w.bytes = c.used();
    return w;
}

// weight sum only (expected-sample mode) or sum + CDF
int build_cdf(const float* weights, int64_t n_cells, float* cdf, float* sum_out, const SamplerWs& w, cudaStream_t stream) {
    const int64_t chunks = ceil_div<int64_t>(n_cells, kCdfChunk);
    INPC_CUDA_TRY(cudaMemsetAsync(w.max_bits, 0, sizeof(unsigned), stream));
    cdf_max_kernel<<<(unsigned)chunks, kCdfThreads, 0, stream>>>(weights, n_cells, w.max_bits);
    INPC_LAUNCH_CHECK("cdf_max_kernel");
    cdf_chunk_sums_kernel<<<(unsigned)chunks, kCdfThreads, 0, stream>>>(weights, n_cells, w.max_bits, w.chunk_sums64);
    INPC_LAUNCH_CHECK("cdf_chunk_sums_kernel");
    cdf_scan_chunks_kernel<<<1, 1024, 0, stream>>>(w.chunk_sums64, chunks, w.max_bits, w.total64, sum_out);
    INPC_LAUNCH_CHECK("cdf_scan_chunks_kernel");
    if (cdf) {
        cdf_finalize_kernel<<<(unsigned)chunks, kCdfThreads, 0, stream>>>(weights, n_cells, w.max_bits, w.chunk_sums64, w.total64, cdf);
        INPC_LAUNCH_CHECK("cdf_finalize_kernel");
        if (cdf == w.cdf) {
            guide_table_kernel<<<(unsigned)ceil_div<int64_t>(((int64_t)1 << w.guide_bits) + 1, kThreads), kThreads, 0, stream>>>(
                cdf, (unsigned)n_cells, w.guide_bits, w.guide);
            INPC_LAUNCH_CHECK("guide_table_kernel");
        }
    }
    return INPC_OK;
}

int check_cells(const inpc_view* view, int64_t n_cells, const void* a, const void* b, const void* c) {
    if (!view || !view->w2c) { set_error("sampler: view and view.w2c must be non-null"); return INPC_E_INVALID; }
    // 2^24 leaves is the reference octree's own cap (Modules/ProbabilityField.py:217-257); the 39-bit
    // fixed-point fractions of the CDF add up in 64 bits without wrapping for up to 2^25 of them
    if (n_cells <= 0 || n_cells > ((int64_t)1 << 24)) { set_error("sampler: n_cells=%lld out of range [1, 2^24]", (long long)n_cells); return INPC_E_INVALID; }
    if (!a || !b || !c) { set_error("sampler: null leaf array"); return INPC_E_INVALID; }
    return INPC_OK;
}

float* pinned_float() {
    static thread_local float* p = nullptr;
    if (!p && cudaHostAlloc(reinterpret_cast<void**>(&p), 64, cudaHostAllocDefault) != cudaSuccess) p = nullptr;
    return p;
}

}  // namespace

}  // namespace inpc

using namespace inpc;

struct inpc_sampler {
    unsigned long long seed;
    unsigned long long counter;
    long long training_ticket;   // status slot of the last inpc_generate_training_samples call (0: none)
};

extern "C" inpc_sampler* inpc_sampler_create(int64_t seed) {
    inpc_sampler* s = new inpc_sampler;
    s->seed = (unsigned long long)seed;
    s->counter = 0;
    s->training_ticket = 0;
    return s;
}
extern "C" void inpc_sampler_destroy(inpc_sampler* s) { delete s; }
// 1 if some slots of the sampler's last inpc_generate_training_samples call ran out of rejection attempts
// (they hold their last candidate, a position outside the view frustum), 0 if none did, -1 if that is no longer
// known (the status slot has been reused).  Meaningful once the call's stream has been synchronised.
extern "C" int inpc_sampler_exhausted(const inpc_sampler* s) {
    if (!s || s->training_ticket == 0) return 0;
    unsigned w[inpc::STATUS_WORDS];
    if (inpc::read_status(s->training_ticket, w, nullptr) != INPC_OK) return -1;
    return w[inpc::STATUS_SAMPLER_EXHAUSTED] ? 1 : 0;
}
extern "C" uint64_t inpc_sampler_get_counter(const inpc_sampler* s) { return s ? s->counter : 0; }
extern "C" void inpc_sampler_set_counter(inpc_sampler* s, uint64_t counter) { if (s) s->counter = counter; }

extern "C" size_t inpc_sampler_workspace_bytes(int64_t n_cells) { return carve_sampler_ws(nullptr, n_cells).bytes; }

extern "C" int inpc_compute_viewpoint_weights(const inpc_view* view, int64_t n_cells, const float* centers,
                                              const int32_t* levels, const float* weights, float initial_size,
                                              float* out, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_cells == 0) return INPC_OK;
    int rc = check_cells(view, n_cells, centers, levels, weights);
    if (rc != INPC_OK) return rc;
    if (!out) { set_error("inpc_compute_viewpoint_weights: null output"); return INPC_E_INVALID; }
    viewpoint_weights_kernel<<<(unsigned)ceil_div<int64_t>(n_cells, kThreads), kThreads, 0, stream>>>(
        to_params(view), n_cells, centers, levels, weights, initial_size, out, nullptr);
    INPC_LAUNCH_CHECK("viewpoint_weights_kernel");
    return INPC_OK;
}

extern "C" int inpc_build_cdf(const float* weights, int64_t n_cells, float* cdf, float* sum_out, void* workspace,
                              void* stream_) {
    if (n_cells <= 0 || !weights || !cdf || !sum_out || !workspace) { set_error("inpc_build_cdf: bad argument"); return INPC_E_INVALID; }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    return build_cdf(weights, n_cells, cdf, sum_out, w, static_cast<cudaStream_t>(stream_));
}

extern "C" int inpc_draw_leaves(const float* cdf, int64_t n_cells, const float* u, int64_t n, int64_t* out, void* stream_) {
    if (n == 0) return INPC_OK;
    if (n_cells <= 0 || n_cells >= ((int64_t)1 << 31) || !cdf || !u || !out || n < 0) { set_error("inpc_draw_leaves: bad argument"); return INPC_E_INVALID; }
    draw_leaves_kernel<<<(unsigned)ceil_div<int64_t>(n, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
        cdf, (unsigned)n_cells, u, n, reinterpret_cast<long long*>(out));
    INPC_LAUNCH_CHECK("draw_leaves_kernel");
    return INPC_OK;
}

extern "C" int inpc_generate_training_samples(inpc_sampler* s, const inpc_view* view, int64_t n_cells, const float* centers,
                                              const int32_t* levels, const float* weights, float initial_size,
                                              int64_t n_samples, float* positions, int64_t* indices, void* workspace,
                                              void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!s) { set_error("null sampler"); return INPC_E_INVALID; }
    if (n_samples == 0) return INPC_OK;
    int rc = check_cells(view, n_cells, centers, levels, weights);
    if (rc != INPC_OK) return rc;
    if (n_samples < 0 || n_samples >= ((int64_t)1 << 32) || !positions || !indices || !workspace) { set_error("inpc_generate_training_samples: bad argument"); return INPC_E_INVALID; }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    const ViewParams v = to_params(view);
    StageScope scope(STAGE_SAMPLE, stream);
    viewpoint_weights_kernel<<<(unsigned)ceil_div<int64_t>(n_cells, kThreads), kThreads, 0, stream>>>(v, n_cells, centers, levels, weights, initial_size, w.vw, w.leaf_pack);
    INPC_LAUNCH_CHECK("viewpoint_weights_kernel");
    rc = build_cdf(w.vw, n_cells, w.cdf, w.sum, w, stream);
    if (rc != INPC_OK) return rc;
    unsigned* status = acquire_status("inpc_generate_training_samples", &s->training_ticket);
    if (!status) return INPC_E_CUDA;
    training_samples_kernel<<<(unsigned)ceil_div<int64_t>(n_samples, kThreads), kThreads, 0, stream>>>(
        v, s->seed, s->counter, w.cdf, w.guide, w.guide_bits, w.sum, (unsigned)n_cells, w.leaf_pack, n_samples, positions,
        reinterpret_cast<long long*>(indices), status);
    INPC_LAUNCH_CHECK("training_samples_kernel");
    s->counter += 1;
    return INPC_OK;
}

extern "C" int inpc_generate_samples(inpc_sampler* s, const inpc_view* view, int64_t n_cells, const float* centers,
                                     const int32_t* levels, const float* weights, float initial_size, int64_t n_samples,
                                     float* positions, int64_t* n_written, void* workspace, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!s || !n_written) { set_error("null sampler or n_written"); return INPC_E_INVALID; }
    *n_written = 0;
    int rc = check_cells(view, n_cells, centers, levels, weights);
    if (rc != INPC_OK) return rc;
    if (n_samples < 0 || n_samples >= ((int64_t)1 << 32) || !workspace || (n_samples > 0 && !positions)) { set_error("inpc_generate_samples: bad argument"); return INPC_E_INVALID; }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    const ViewParams v = to_params(view);
    viewpoint_weights_kernel<<<(unsigned)ceil_div<int64_t>(n_cells, kThreads), kThreads, 0, stream>>>(v, n_cells, centers, levels, weights, initial_size, w.vw, w.leaf_pack);
    INPC_LAUNCH_CHECK("viewpoint_weights_kernel");
    rc = build_cdf(w.vw, n_cells, w.cdf, w.sum, w, stream);
    if (rc != INPC_OK) return rc;
    float* host = pinned_float();
    if (!host) return cuda_fail(cudaGetLastError(), "cudaHostAlloc");
    INPC_CUDA_TRY(cudaMemcpyAsync(host, w.sum, sizeof(float), cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    if (!(host[0] > 0.0f)) return INPC_OK;   // src/sampling_api.cu:154: empty result
    if (n_samples > 0) {
        samples_kernel<<<(unsigned)ceil_div<int64_t>(n_samples, kThreads), kThreads, 0, stream>>>(
            s->seed, s->counter, w.cdf, w.guide, w.guide_bits, (unsigned)n_cells, w.leaf_pack, n_samples, positions);
        INPC_LAUNCH_CHECK("samples_kernel");
    }
    s->counter += 1;
    *n_written = n_samples;
    return INPC_OK;
}

extern "C" int inpc_generate_expected_samples_count(inpc_sampler* s, const inpc_view* view, int64_t n_cells,
                                                    const float* centers, const int32_t* levels, const float* weights,
                                                    float initial_size, int64_t n_samples, int64_t* n_created,
                                                    void* workspace, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!s || !n_created) { set_error("null sampler or n_created"); return INPC_E_INVALID; }
    *n_created = 0;
    int rc = check_cells(view, n_cells, centers, levels, weights);
    if (rc != INPC_OK) return rc;
    if (n_samples < 0 || n_samples >= ((int64_t)1 << 32) || !workspace) { set_error("inpc_generate_expected_samples_count: bad argument"); return INPC_E_INVALID; }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    const ViewParams v = to_params(view);
    const unsigned blocks = (unsigned)ceil_div<int64_t>(n_cells, kThreads);
    viewpoint_weights_kernel<<<blocks, kThreads, 0, stream>>>(v, n_cells, centers, levels, weights, initial_size, w.vw, nullptr);
    INPC_LAUNCH_CHECK("viewpoint_weights_kernel");
    rc = build_cdf(w.vw, n_cells, nullptr, w.sum, w, stream);
    if (rc != INPC_OK) return rc;
    sample_counts_kernel<<<blocks, kThreads, 0, stream>>>(w.vw, w.sum, (unsigned)n_samples, n_cells, w.counts);
    INPC_LAUNCH_CHECK("sample_counts_kernel");
    count_chunk_sums_kernel<<<blocks, kThreads, 0, stream>>>(w.counts, n_cells, w.chunk_sums);
    INPC_LAUNCH_CHECK("count_chunk_sums_kernel");
    scan_chunk_sums_kernel<<<1, kIScanThreads, 0, stream>>>(w.chunk_sums, blocks, w.total);
    INPC_LAUNCH_CHECK("scan_chunk_sums_kernel");
    count_offsets_kernel<<<blocks, kThreads, 0, stream>>>(w.counts, n_cells, w.chunk_sums, w.offsets);
    INPC_LAUNCH_CHECK("count_offsets_kernel");
    unsigned long long* host = reinterpret_cast<unsigned long long*>(pinned_float());
    if (!host) return cuda_fail(cudaGetLastError(), "cudaHostAlloc");
    INPC_CUDA_TRY(cudaMemcpyAsync(host, w.total, sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    if (host[0] >= (1ull << 32)) { set_error("expected sample count %llu exceeds 2^32", host[0]); return INPC_E_CAPACITY; }
    *n_created = (int64_t)host[0];
    return INPC_OK;
}

extern "C" int inpc_generate_expected_samples_fill(inpc_sampler* s, int64_t n_cells, const float* centers,
                                                   const int32_t* levels, float initial_size, int64_t n_created,
                                                   int64_t n_multi, float* positions, void* workspace, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!s) { set_error("null sampler"); return INPC_E_INVALID; }
    const int64_t total = n_created * n_multi;
    if (n_cells <= 0 || n_created <= 0 || n_multi <= 0 || total >= ((int64_t)1 << 32) || !centers || !levels || !positions || !workspace) {
        set_error("inpc_generate_expected_samples_fill: bad argument");
        return INPC_E_INVALID;
    }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    expected_samples_kernel<<<(unsigned)ceil_div<int64_t>(total, kThreads), kThreads, 0, stream>>>(
        s->seed, s->counter, w.offsets, (unsigned)n_cells, centers, levels, initial_size, total, (unsigned)n_created, positions);
    INPC_LAUNCH_CHECK("expected_samples_kernel");
    s->counter += 1;
    return INPC_OK;
}

namespace {
// inclusive offsets of w.counts into w.offsets
int scan_counts(const SamplerWs& w, int64_t n_cells, cudaStream_t stream) {
    const unsigned blocks = (unsigned)ceil_div<int64_t>(n_cells, kThreads);
    count_chunk_sums_kernel<<<blocks, kThreads, 0, stream>>>(w.counts, n_cells, w.chunk_sums);
    INPC_LAUNCH_CHECK("count_chunk_sums_kernel");
    scan_chunk_sums_kernel<<<1, kIScanThreads, 0, stream>>>(w.chunk_sums, blocks, w.total);
    INPC_LAUNCH_CHECK("scan_chunk_sums_kernel");
    count_offsets_kernel<<<blocks, kThreads, 0, stream>>>(w.counts, n_cells, w.chunk_sums, w.offsets);
    INPC_LAUNCH_CHECK("count_offsets_kernel");
    return INPC_OK;
}
}  // namespace

extern "C" int inpc_draw_leaf_counts(inpc_sampler* s, int64_t n_cells, const float* weights, int64_t n_samples, uint32_t* counts,
                                     void* workspace, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!s || n_cells <= 0 || n_cells >= ((int64_t)1 << 31) || n_samples < 0 || n_samples >= ((int64_t)1 << 32) || !weights || !counts || !workspace) {
        set_error("inpc_draw_leaf_counts: bad argument");
        return INPC_E_INVALID;
    }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    int rc = build_cdf(weights, n_cells, w.cdf, w.sum, w, stream);
    if (rc != INPC_OK) return rc;
    INPC_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(uint32_t) * (size_t)n_cells, stream));
    float* host = pinned_float();
    if (!host) return cuda_fail(cudaGetLastError(), "cudaHostAlloc");
    INPC_CUDA_TRY(cudaMemcpyAsync(host, w.sum, sizeof(float), cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    if (!(host[0] > 0.0f)) { set_error("inpc_draw_leaf_counts: the weights sum to zero"); return INPC_E_INVALID; }
    if (n_samples > 0) {
        leaf_histogram_kernel<<<(unsigned)ceil_div<int64_t>(n_samples, kThreads), kThreads, 0, stream>>>(
            s->seed, s->counter, w.cdf, w.guide, w.guide_bits, (unsigned)n_cells, n_samples, counts);
        INPC_LAUNCH_CHECK("leaf_histogram_kernel");
    }
    s->counter += 1;
    return INPC_OK;
}

extern "C" int inpc_halton_samples(const uint32_t* counts, int64_t n_cells, const float* centers, const int32_t* levels, float initial_size,
                                   int64_t n_total, float* positions, void* workspace, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_total == 0) return INPC_OK;
    if (n_cells <= 0 || n_cells >= ((int64_t)1 << 31) || n_total < 0 || n_total >= ((int64_t)1 << 32) || !counts || !centers || !levels || !positions || !workspace) {
        set_error("inpc_halton_samples: bad argument");
        return INPC_E_INVALID;
    }
    SamplerWs w = carve_sampler_ws(workspace, n_cells);
    INPC_CUDA_TRY(cudaMemcpyAsync(w.counts, counts, sizeof(uint32_t) * (size_t)n_cells, cudaMemcpyDeviceToDevice, stream));
    const int rc = scan_counts(w, n_cells, stream);
    if (rc != INPC_OK) return rc;
    halton_samples_kernel<<<(unsigned)ceil_div<int64_t>(n_total, kThreads), kThreads, 0, stream>>>(w.counts, w.offsets, (unsigned)n_cells, centers, levels,
                                                                                                 initial_size, n_total, positions);
    INPC_LAUNCH_CHECK("halton_samples_kernel");
    return INPC_OK;
}

extern "C" size_t inpc_morton_workspace_bytes(int64_t n) {
    const size_t arr = align_up(sizeof(uint32_t) * (size_t)(n > 0 ? n : 1));
    return 4 * arr + sort_workspace_bytes(n) + 256;
}

extern "C" int inpc_morton_order(const float* positions, int64_t n, const float* box_lo, float box_extent, float* out, void* workspace,
                                 void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n == 0) return INPC_OK;
    if (n < 0 || n >= ((int64_t)1 << 30) || !positions || !box_lo || !(box_extent > 0.0f) || !out || !workspace || out == positions) {
        set_error("inpc_morton_order: bad argument");
        return INPC_E_INVALID;
    }
    Carver c(workspace);
    uint32_t* codes[2] = {c.take<uint32_t>(n), c.take<uint32_t>(n)};
    uint32_t* order[2] = {c.take<uint32_t>(n), c.take<uint32_t>(n)};
    c.off = align_up(c.off);
    void* sort_ws = c.base + c.off;
    morton_codes_kernel<<<(unsigned)ceil_div<int64_t>(n, kThreads), kThreads, 0, stream>>>(positions, n, box_lo[0], box_lo[1], box_lo[2],
                                                                                       1.0f / box_extent, codes[0], order[0]);
    INPC_LAUNCH_CHECK("morton_codes_kernel");
    int in_alt = 0;
    {
        const int rc_prev = check_previous_calls();
        if (rc_prev != INPC_OK) return rc_prev;
    }
    unsigned* status = acquire_status("inpc_morton_order");
    if (!status) return INPC_E_CUDA;
    const int rc = sort_pairs(codes[0], codes[1], order[0], order[1], n, 30, sort_ws, status, &in_alt, stream);
    if (rc != INPC_OK) return rc;
    gather_positions_kernel<<<(unsigned)ceil_div<int64_t>(n, kThreads), kThreads, 0, stream>>>(positions, order[in_alt], n, out);
    INPC_LAUNCH_CHECK("gather_positions_kernel");
    return INPC_OK;
}
