// Rasterizer of the inpc_b200 library: cull/project/SH-evaluate -> order by (tile, depth) ->
// front-to-back blend, forward, backward and inference, bilinear and gaussian splats.
//
// Data layout in HBM (all carved from two caller-allocated blobs):
//   per point   : PointRec 32 B {screen x, screen y, opacity, depth | 4 view-space feature channels}
//                 (one 32-byte sector per gather in the blend), tile bounds 8 B, conic 16 B (gaussian)
//   per visible : depth key + point id, ping-pong pair for the depth sort
//   per instance: tile key + point id, ping-pong pair for the tile sort
//   per tile    : [first, last+1) instance range
//
// The arithmetic follows the reference kernels expression by expression (cited per function, paths
// below INPCCudaBackend/INPCCudaBackend/rasterization/ of the reference); the organisation of the
// work does not: compaction is a deterministic two-pass scan instead of atomics, the sorts are the
// library's own onesweep, and the bilinear blend walks per-pixel bit masks of the staged batch
// instead of testing every staged point against every pixel.
#include "common.cuh"

#include <type_traits>

namespace inpc {

namespace {

constexpr float kTransmittanceEps = 1e-4f;      // include/bilinear/config.h:16
constexpr float kOneMinusAlphaEps = 1e-8f;      // include/bilinear/config.h:17
constexpr float kDilation = 0.16f;              // include/gaussian/config.h:19
constexpr float kTrainGaussThreshold = 0.01110899653f;   // src/gaussian/kernels.cu:452


// Checked build (-DINPC_CHECK_INDICES, `python -m inpc_b200._build --checked`): every point index read
// from a sorted list is range-checked before it is used for a gather; a bad one is counted, reported
// through a status word and replaced by 0, so the access itself never leaves its array.  The limit
// lives in a device variable the entry points set before they launch anything.
#ifdef INPC_CHECK_INDICES
__device__ unsigned long long g_check_n_points;
__device__ unsigned g_check_failures;
__device__ __forceinline__ uint32_t checked_point(uint32_t id) {
    if ((unsigned long long)id >= g_check_n_points) {
        atomicAdd(&g_check_failures, 1u);
        return 0u;
    }
    return id;
}
#else
__device__ __forceinline__ uint32_t checked_point(uint32_t id) { return id; }
#endif

enum { VAR_TRAIN = 0, VAR_RAW37 = 1, VAR_PREEXTRACTED = 2, VAR_ROWS = 3 };   // VAR_ROWS: features stay in the caller's (n, C) fp32 array

struct __align__(16) PointRec {
    float sx, sy, opacity, depth;
    float f[4];
};

struct RasterParams {
    ViewParams v;
    int tile;       // tile edge in pixels (8 or 16)
    float inv_tile; // its reciprocal: the edge is a power of two, so x * inv_tile == x / tile bit for bit
    int gw, gh;     // tile grid of one image
    int n_sets;     // images drawn by the call (1 except for batched multi-set inference): the grid has n_sets * gh rows
    float sigma_world, sigma_cutoff;
    const float* scales;   // optional per-point sigma (gaussian, pre-extracted)
};

// Input points of a call: one array triple, or (batched multi-set inference) up to kMaxSets of them laid end to end in
// a virtual index space in which every set starts at a multiple of 1024, so that a block of the two input passes never
// straddles two sets.  Set j is drawn into its own image: its tiles are rows [j * gh, (j + 1) * gh) of a stacked grid.
constexpr int kMaxSets = 8;
constexpr int64_t kSetAlign = 1024;
struct PointSets {
    int count;
    int64_t start[kMaxSets + 1];      // virtual index of every set's first point; start[count] = virtual total
    int64_t size[kMaxSets];
    const float* positions[kMaxSets];
    const void* features[kMaxSets];
    const float* opacities[kMaxSets];
};
__device__ __forceinline__ int set_of_block(const PointSets& ps, int64_t block_first) {
    int j = 0;
    while (j + 1 < ps.count && block_first >= ps.start[j + 1]) ++j;
    return j;
}

struct Projection {
    bool visible;
    float depth, sx, sy;
    unsigned x0, x1, y0, y1;
    float cx, cy, cz;   // conic
};

struct W2C {
    float r0[4], r1[4], r2[4];
};

__device__ __forceinline__ W2C load_w2c(const float* __restrict__ w2c) {
    W2C m;
#pragma unroll
    for (int k = 0; k < 4; ++k) { m.r0[k] = __ldg(w2c + k); m.r1[k] = __ldg(w2c + 4 + k); m.r2[k] = __ldg(w2c + 8 + k); }
    return m;
}

// One row of the world-to-camera transform applied to a point: r.x p.x + r.y p.y + r.z p.z + r.w with the
// roundings of the reference binary (src/bilinear/kernels.cu:43-49 as nvcc contracts it): the second
// product is rounded, the first and the third are fused onto it, the translation is added last.  Written
// with intrinsics so that depth keys and screen positions, which are compared bit for bit, do not depend
// on the compiler's choice of contraction.
__device__ __forceinline__ float affine_row(const float* r, float px, float py, float pz) {
    float t = __fmul_rn(r[1], py);
    t = __fmaf_rn(r[0], px, t);
    t = __fmaf_rn(r[2], pz, t);
    return __fadd_rn(t, r[3]);
}

// src/bilinear/kernels.cu:41-65 and src/gaussian/kernels.cu:41-90 (training), :145-186 (inference),
// :243-292 (pre-extracted): depth cull, perspective divide, pixel coordinates, tile bounds.
// `scales_index`: index into rp.scales; `set`: which image of the stacked tile grid the point is drawn into.
template <int MODE, int VARIANT>
__device__ __forceinline__ Projection project_point(const float px, const float py, const float pz, const W2C& m,
                                                    const RasterParams& rp, const int64_t i, const int set = 0) {
    Projection o;
    o.visible = false;
    o.x0 = o.x1 = o.y0 = o.y1 = 0;
    o.cx = o.cy = o.cz = 0.0f;
    const float depth = affine_row(m.r2, px, py, pz);
    o.depth = depth;
    o.sx = o.sy = 0.0f;
    if (depth < rp.v.near_plane || depth > rp.v.far_plane) return o;
    const float x = __fdiv_rn(affine_row(m.r0, px, py, pz), depth);
    const float y = __fdiv_rn(affine_row(m.r1, px, py, pz), depth);
    const float sx = __fmaf_rn(x, rp.v.fx, rp.v.cx);
    const float sy = __fmaf_rn(y, rp.v.fy, rp.v.cy);
    float ex = 0.5f, ey = 0.5f;
    if (MODE == INPC_MODE_GAUSSIAN) {
        float variance_world;
        float k = 3.0f;
        if (VARIANT == VAR_TRAIN) {
            constexpr float numerator = 0.3f * 0.3f * 0.5f * 0.5f;
            variance_world = numerator / (rp.v.fx * rp.v.fy);
        } else {
            k = rp.sigma_cutoff;
            if (VARIANT == VAR_PREEXTRACTED && rp.scales != nullptr) {
                const float s = __ldg(rp.scales + i);
                variance_world = s * s;
            } else {
                variance_world = rp.sigma_world * rp.sigma_world;
            }
        }
        const float fx = rp.v.fx, fy = rp.v.fy, cx = rp.v.cx, cy = rp.v.cy;
        const float J_00 = fx / depth;
        const float J_02 = -J_00 * fminf(fmaxf(x, -1.3f * cx / fx), 1.3f * cx / fx);
        const float J_11 = fy / depth;
        const float J_12 = -J_11 * fminf(fmaxf(y, -1.3f * cy / fy), 1.3f * cy / fy);
        float cov_x = variance_world * (J_00 * J_00 + J_02 * J_02);
        const float cov_y = variance_world * (J_02 * J_12);
        float cov_z = variance_world * (J_11 * J_11 + J_12 * J_12);
        cov_x += kDilation;
        cov_z += kDilation;
        const float det = cov_x * cov_z - cov_y * cov_y;
        if (det == 0.0f) return o;
        const float det_rcp = 1.0f / det;
        o.cx = cov_z * det_rcp;
        o.cy = -cov_y * det_rcp;
        o.cz = cov_x * det_rcp;
        ex = k * sqrtf(cov_x) - 0.5f;
        ey = k * sqrtf(cov_z) - 0.5f;
    }
    const float itf = rp.inv_tile;
    const unsigned gw = (unsigned)rp.gw, gh = (unsigned)rp.gh;
    o.x0 = min(gw, (unsigned)max(0, __float2int_rd((sx - ex) * itf)));
    o.x1 = min(gw, (unsigned)max(0, __float2int_ru((sx + ex) * itf)));
    o.y0 = min(gh, (unsigned)max(0, __float2int_rd((sy - ey) * itf)));
    o.y1 = min(gh, (unsigned)max(0, __float2int_ru((sy + ey) * itf)));
    o.sx = sx;
    o.sy = sy;
    o.visible = (o.x1 - o.x0) * (o.y1 - o.y0) != 0u;
    o.y0 += (unsigned)set * gh;   // rows of this set's image in the stacked grid (screen coordinates stay the set's own)
    o.y1 += (unsigned)set * gh;
    return o;
}

constexpr int kPreThreads = 256;
constexpr unsigned kCountShift = 30;   // bilinear: (tiles touched - 1) in key bits 30..31 when the depth offsets fit below

// Pass 1 of the deterministic compaction: per block, how many points survive culling and how many
// (point, tile) instances they create.
template <int MODE, int VARIANT>
__global__ void __launch_bounds__(kPreThreads) visibility_count_kernel(
    PointSets ps, RasterParams rp, unsigned* __restrict__ block_visible,
    unsigned* __restrict__ group_visible, unsigned long long* __restrict__ group_instances, unsigned* __restrict__ depth_min,
    unsigned* __restrict__ depth_max) {
    // this block's set; indices below are local to it
    const int set = set_of_block(ps, (int64_t)blockIdx.x * kPreThreads * 4);
    const float* __restrict__ positions = ps.positions[set];
    const int64_t n = ps.size[set];
    const int64_t n_virtual = ps.start[ps.count];
    // Every thread takes 4 consecutive points (three 16-byte loads when the array is aligned), so a
    // block covers 4 chunks of kPreThreads points; counts are kept per chunk because the projection
    // pass works on chunks of kPreThreads points.
    constexpr int kPerThread = 4;
    constexpr int kWarpsPerChunk = kPreThreads / kPerThread / 32;   // 2
    __shared__ unsigned s_v[kPreThreads / 32];
    __shared__ unsigned long long s_i[kPreThreads / 32];
    __shared__ unsigned s_lo[kPreThreads / 32], s_hi[kPreThreads / 32];
    const W2C m = load_w2c(rp.v.w2c);
    const int64_t first = ((int64_t)blockIdx.x * kPreThreads + threadIdx.x) * kPerThread - ps.start[set];   // local to the set
    float p[3 * kPerThread];
    if (first + kPerThread <= n && (reinterpret_cast<uintptr_t>(positions) & 15u) == 0) {
        const float4* src = reinterpret_cast<const float4*>(positions + 3 * first);
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const float4 v = __ldg(src + k);
            p[4 * k] = v.x; p[4 * k + 1] = v.y; p[4 * k + 2] = v.z; p[4 * k + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 3 * kPerThread; ++k) p[k] = first * 3 + k < 3 * n ? __ldg(positions + 3 * first + k) : 0.0f;
    }
    unsigned v = 0, lo = 0xFFFFFFFFu, hi = 0u;
    unsigned long long c = 0;
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
        if (first + k < n) {
            const Projection pr = project_point<MODE, VARIANT>(p[3 * k], p[3 * k + 1], p[3 * k + 2], m, rp, first + k, set);
            if (pr.visible) {
                v += 1u;
                c += (pr.x1 - pr.x0) * (pr.y1 - pr.y0);
                const unsigned bits = __float_as_uint(pr.depth);   // visible depths are positive: bit patterns order like the values
                lo = min(lo, bits);
                hi = max(hi, bits);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_down_sync(0xffffffffu, v, o);
        c += __shfl_down_sync(0xffffffffu, c, o);
        lo = min(lo, __shfl_down_sync(0xffffffffu, lo, o));
        hi = max(hi, __shfl_down_sync(0xffffffffu, hi, o));
    }
    const int warp = threadIdx.x >> 5;
    if (lane_id() == 0) { s_v[warp] = v; s_i[warp] = c; s_lo[warp] = lo; s_hi[warp] = hi; }
    __syncthreads();
    if (threadIdx.x < kPerThread) {
        // chunk `threadIdx.x` of this block
        const int64_t chunk = (int64_t)blockIdx.x * kPerThread + threadIdx.x;
        if (chunk * kPreThreads < n_virtual) {   // chunks of the padding behind a set count zero survivors
            unsigned tv = 0;
            unsigned long long ti = 0;
#pragma unroll
            for (int w = 0; w < kWarpsPerChunk; ++w) { tv += s_v[threadIdx.x * kWarpsPerChunk + w]; ti += s_i[threadIdx.x * kWarpsPerChunk + w]; }
            block_visible[chunk] = tv;
            (void)ti;
        }
    }
    if (threadIdx.x == 0) {
        unsigned tlo = 0xFFFFFFFFu, thi = 0u, tv = 0;
        unsigned long long ti = 0;
#pragma unroll
        for (int w = 0; w < kPreThreads / 32; ++w) { tlo = min(tlo, s_lo[w]); thi = max(thi, s_hi[w]); tv += s_v[w]; ti += s_i[w]; }
        // totals of this group of 4 chunks: the one-block scan runs over groups, four times fewer entries
        group_visible[blockIdx.x] = tv;
        group_instances[blockIdx.x] = ti;
        // (callers that know a bound on the depths beforehand pass no pointers; measured: no difference in time)
        if (depth_min && tlo <= thi) { atomicMin(depth_min, tlo); atomicMax(depth_max, thi); }
    }
}

// Exclusive scan of the per-group counts (groups of 4 chunks) by one block; totals land in counters[0]
// (visible) and counters[1] (instances), the depth range in counters[2..3].
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads) scan_block_counts_kernel(unsigned* __restrict__ block_visible,
                                                                         const unsigned long long* __restrict__ block_instances,
                                                                         int64_t n_blocks,
                                                                         unsigned* __restrict__ depth_min,
                                                                         unsigned* __restrict__ depth_max,
                                                                         unsigned long long* __restrict__ counters, int fixed_range,
                                                                         unsigned fixed_lo, unsigned fixed_hi) {
    constexpr int kItems = 8;
    __shared__ unsigned s_scan[kScanThreads / 32 + 1];
    __shared__ unsigned long long s_inst[kScanThreads / 32];
    unsigned running = 0;
    unsigned long long inst = 0;
    for (int64_t base = 0; base < n_blocks; base += (int64_t)kScanThreads * kItems) {
        const int64_t j0 = base + (int64_t)threadIdx.x * kItems;
        unsigned v[kItems];
        unsigned sum = 0;
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
            v[k] = j0 + k < n_blocks ? block_visible[j0 + k] : 0u;
            sum += v[k];
            if (j0 + k < n_blocks) inst += block_instances[j0 + k];
        }
        unsigned total;
        unsigned ex = running + block_exclusive_scan(sum, s_scan, &total);
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
            if (j0 + k < n_blocks) block_visible[j0 + k] = ex;
            ex += v[k];
        }
        running += total;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) inst += __shfl_down_sync(0xffffffffu, inst, o);
    if (lane_id() == 0) s_inst[threadIdx.x >> 5] = inst;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < kScanThreads / 32; ++w) t += s_inst[w];
        counters[0] = running;
        counters[1] = t;
        // the range of depth bit patterns the keys are offsets into: measured by the count pass, or given by the caller
        if (fixed_range) { *depth_min = fixed_lo; *depth_max = fixed_hi; }
        counters[2] = *depth_min;
        counters[3] = *depth_max;
    }
}

// SH degree 2 along the view ray -> 4 channels: include/sh_utils.cuh:6-23.  `h` points at 36 halves
// (coefficient-major, channel-minor) in shared memory.
__device__ __forceinline__ void sh_basis(const float px, const float py, const float pz, const float* __restrict__ cam,
                                         float* b) {
    const float vx = px - __ldg(cam), vy = py - __ldg(cam + 1), vz = pz - __ldg(cam + 2);
    const float inv = rsqrtf(vx * vx + vy * vy + vz * vz);
    const float x = vx * inv, y = vy * inv, z = vz * inv;
    const float xx = x * x, yy = y * y, zz = z * z;
    const float xy = x * y, yz = y * z, xz = x * z;
    b[0] = 0.28209479177387814f;
    b[1] = 0.48860251190291987f * y;
    b[2] = 0.48860251190291987f * z;
    b[3] = 0.48860251190291987f * x;
    b[4] = 1.0925484305920792f * xy;
    b[5] = 1.0925484305920792f * yz;
    b[6] = 0.94617469575755997f * zz - 0.31539156525251999f;
    b[7] = 1.0925484305920792f * xz;
    b[8] = 0.54627421529603959f * xx - 0.54627421529603959f * yy;
}

__device__ __forceinline__ float sh_eval_channel(const float* b, const __half* h, int c) {
    return b[0] * __half2float(h[c]) - b[1] * __half2float(h[4 + c]) + b[2] * __half2float(h[8 + c]) -
           b[3] * __half2float(h[12 + c]) + b[4] * __half2float(h[16 + c]) - b[5] * __half2float(h[20 + c]) +
           b[6] * __half2float(h[24 + c]) - b[7] * __half2float(h[28 + c]) + b[8] * __half2float(h[32 + c]);
}

// What the instance emission of the warp blend needs of a bilinear splat, in one word.  Columns: pixel column of the
// left pixel of its 2x2 footprint plus one (15 bits; a visible splat's footprint starts at pixel -1 at the earliest),
// whether it touches two tile columns (1 bit).  Rows: the first tile row it touches in the stacked grid (11 bits), the
// row of its upper pixel relative to that tile plus one (4 bits, 0..8), whether it touches two tile rows (1 bit).
// Rows are kept relative to the tile because the first row of an image other than the first is not row 0 of the
// grid.  4 bytes per point keep the array (33 MB for 2^23 points) resident in L2 while the emission gathers from
// it in depth order.
constexpr int kMaxCodedSide = 32760;       // widest image of this path, in pixels
constexpr int kMaxCodedTileRows = 2047;    // most tile rows of the (stacked) grid
__device__ __forceinline__ uint32_t pack_quad(const Projection& pr, int tile_rows_before) {
    const unsigned qx1 = (unsigned)(__float2int_rd(pr.sx - 0.5f) + 1);
    const unsigned ry1 = (unsigned)(__float2int_rd(pr.sy - 0.5f) - ((int)pr.y0 - tile_rows_before) * 8 + 1);
    return (qx1 & 0x7FFFu) | ((pr.x1 - pr.x0 - 1u) << 15) | ((pr.y0 & 0x7FFu) << 16) | ((ry1 & 0xFu) << 27) | ((pr.y1 - pr.y0 - 1u) << 31);
}

// Pass 2: project again (same arithmetic, same outcome), evaluate SH, write the point record and
// bounds, and append (depth key, point id) at the slot given by the block offset plus the rank of
// the point among the block's survivors — index order, hence reproducible.
// src/bilinear/kernels.cu:11-84, :106-184; src/gaussian/kernels.cu:11-111, :113-217, :219-324.
template <int MODE, int VARIANT>
__global__ void __launch_bounds__(kPreThreads) preprocess_kernel(
    PointSets ps, RasterParams rp, const unsigned* __restrict__ block_visible, const unsigned* __restrict__ group_offset,
    const unsigned* __restrict__ depth_min,
    const unsigned* __restrict__ depth_max, PointRec* __restrict__ rec, uint2* __restrict__ bounds, uint32_t* __restrict__ quad,
    float4* __restrict__ conic, uint32_t* __restrict__ depth_keys,
    uint32_t* __restrict__ point_ids, int pack_count, volatile unsigned* status) {
    constexpr int kHalves = VARIANT == VAR_RAW37 ? 37 : 36;
    constexpr int kSlabBytes = VARIANT == VAR_ROWS ? 16 : kPreThreads * kHalves * 2;   // multiple of 16 for both layouts
    __shared__ __align__(16) unsigned char s_feat[kSlabBytes];
    __shared__ unsigned s_scan[kPreThreads / 32 + 1];

    // this block's set: the input arrays are indexed by the point's position in its set (i), everything this pass
    // writes by its position in the virtual index space of the call (iv); the two coincide for a single set
    const int64_t block_first_v = (int64_t)blockIdx.x * kPreThreads;
    const int set = set_of_block(ps, block_first_v);
    const float* __restrict__ positions = ps.positions[set];
    const __half* __restrict__ features = static_cast<const __half*>(ps.features[set]);
    const float* __restrict__ opacities = ps.opacities[set];
    const int64_t n = ps.size[set];
    const bool bulk_ok = (reinterpret_cast<uintptr_t>(features) & 15u) == 0;
    const int64_t block_first = block_first_v - ps.start[set];
    const int in_block = (int)max((int64_t)0, min((int64_t)kPreThreads, n - block_first));
    __shared__ __align__(8) unsigned long long s_bar;
    // The block's feature slab is contiguous in global memory.  When base and size allow (multiples of
    // 16 bytes) one bulk asynchronous copy brings it in while the threads project their points;
    // otherwise (odd tail block, unaligned caller view) 16-byte loads through registers do.
    const bool bulk = VARIANT != VAR_ROWS && bulk_ok && in_block > 0 && ((in_block * kHalves * 2) & 15) == 0;
    if (bulk) {
        if (threadIdx.x == 0) mbarrier_init(&s_bar, 1);
        __syncthreads();
        if (threadIdx.x == 0)
            bulk_load_to_shared(s_feat, reinterpret_cast<const unsigned char*>(features) + block_first * (kHalves * 2),
                                (unsigned)(in_block * kHalves * 2), &s_bar);
    } else if (VARIANT != VAR_ROWS) {
        // coalesced 16-byte staging of the block's contiguous feature slab
        const unsigned char* src = reinterpret_cast<const unsigned char*>(features) + block_first * (kHalves * 2);
        const int bytes = in_block * kHalves * 2;
        const int n16 = bytes / 16;
        const uint4* src16 = reinterpret_cast<const uint4*>(src);
        uint4* dst16 = reinterpret_cast<uint4*>(s_feat);
        for (int k = threadIdx.x; k < n16; k += kPreThreads) dst16[k] = __ldg(src16 + k);
        for (int k = n16 * 16 + 2 * threadIdx.x; k < bytes; k += 2 * kPreThreads)
            *reinterpret_cast<unsigned short*>(s_feat + k) = __ldg(reinterpret_cast<const unsigned short*>(src + k));
    }
    const W2C m = load_w2c(rp.v.w2c);
    const int64_t i = block_first + threadIdx.x;
    const int64_t iv = block_first_v + threadIdx.x;
    Projection pr;
    pr.visible = false;
    float px = 0, py = 0, pz = 0;
    if (i < n) {
        px = __ldg(positions + 3 * i); py = __ldg(positions + 3 * i + 1); pz = __ldg(positions + 3 * i + 2);
        pr = project_point<MODE, VARIANT>(px, py, pz, m, rp, i, set);
    }
    bool slab_ready = true;
    if (bulk) slab_ready = mbarrier_wait_bounded(&s_bar, 0u);
    if (!slab_ready && status) status[STATUS_BULK_COPY_TIMEOUT] = 1u;
    __syncthreads();
    if (i >= n && iv < ps.start[ps.count]) bounds[iv] = make_uint2(0u, 0u);   // padding behind a set
    if (i < n && slab_ready) {
        if (pr.visible && VARIANT == VAR_ROWS) {
            // feature rows are gathered by the blend itself: the record carries the geometry only
            *reinterpret_cast<float4*>(rec + iv) = make_float4(pr.sx, pr.sy, __ldg(opacities + i), pr.depth);
            bounds[iv] = make_uint2(pr.x0 | (pr.x1 << 16), pr.y0 | (pr.y1 << 16));
        } else if (pr.visible) {
            const __half* h = reinterpret_cast<const __half*>(s_feat) + threadIdx.x * kHalves;
            float b[9];
            sh_basis(px, py, pz, rp.v.cam, b);
            PointRec r;
            r.sx = pr.sx; r.sy = pr.sy; r.depth = pr.depth;
            if (VARIANT == VAR_RAW37) {
                // opacity = 1 - exp(-exp(raw)) with the fast exponential: src/bilinear/kernels.cu:144
                r.opacity = 1.0f - __expf(-__expf(__half2float(h[0])));
                h += 1;
            } else {
                r.opacity = __ldg(opacities + i);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) r.f[c] = sh_eval_channel(b, h, c);
            float4* dst = reinterpret_cast<float4*>(rec + iv);
            dst[0] = make_float4(r.sx, r.sy, r.opacity, r.depth);
            dst[1] = make_float4(r.f[0], r.f[1], r.f[2], r.f[3]);
            bounds[iv] = make_uint2(pr.x0 | (pr.x1 << 16), pr.y0 | (pr.y1 << 16));
            if (quad) quad[iv] = pack_quad(pr, set * rp.gh);
            if (MODE == INPC_MODE_GAUSSIAN) conic[iv] = make_float4(pr.cx, pr.cy, pr.cz, 0.0f);
        } else {
            bounds[iv] = make_uint2(0u, 0u);
        }
    }
    unsigned total;
    const unsigned rank = block_exclusive_scan(pr.visible ? 1u : 0u, s_scan, &total);
    if (pr.visible) {
        // slot = survivors of all groups before + of the earlier chunks of this group + rank in this chunk
        unsigned slot = __ldg(group_offset + (blockIdx.x >> 2)) + rank;
        for (unsigned c = blockIdx.x & ~3u; c < blockIdx.x; ++c) slot += __ldg(block_visible + c);
        // sort key: offset of the depth's bit pattern from the smallest visible one (fewer radix passes).
        // A bilinear splat touches 1, 2 or 4 tiles; when the offsets leave the two top bits free that
        // count rides there (the sort ignores bits above its range and carries them along), which
        // saves the instance pass a gather.
        const unsigned lo = __ldg(depth_min);
        unsigned key = __float_as_uint(pr.depth) - lo;
        // pack_count: 1 yes, 0 no (the host knows a bound on the offsets), -1 decide from the measured depth range
        const bool pack = pack_count >= 0 ? pack_count != 0 : __ldg(depth_max) - lo < (1u << kCountShift);
        if (MODE == INPC_MODE_BILINEAR && pack)
            key |= ((pr.x1 - pr.x0) * (pr.y1 - pr.y0) - 1u) << kCountShift;
        depth_keys[slot] = key;
        point_ids[slot] = (uint32_t)iv;
    }
}

__device__ __forceinline__ unsigned tiles_of(const uint2 b) {
    return ((b.x >> 16) - (b.x & 0xffffu)) * ((b.y >> 16) - (b.y & 0xffffu));
}

// Instances per depth-sorted point, reduced per block (src/bilinear/kernels.cu:186-196 + the
// cub::DeviceScan::ExclusiveSum of src/bilinear/forward.cu:109-115, first half).
constexpr int kInstThreads = 1024;   // block sums over 1024 points keep the one-block scan short
template <bool PACKED>
__global__ void __launch_bounds__(kInstThreads / 4) instance_count_kernel(const uint32_t* __restrict__ sorted_keys,
                                                                          const uint32_t* __restrict__ sorted_ids,
                                                                          const uint2* __restrict__ bounds, int64_t n_visible_arg,
                                                                          const unsigned long long* __restrict__ n_visible_dev,
                                                                          unsigned* __restrict__ block_sums) {
    const int64_t n_visible = n_visible_dev ? (int64_t)*n_visible_dev : n_visible_arg;
    // a block of kInstThreads / 4 threads covers kInstThreads points, four consecutive ones per thread
    // (one 16-byte load when the keys carry the count)
    __shared__ unsigned s_w[kInstThreads / 4 / 32];
    const int64_t first = (int64_t)blockIdx.x * kInstThreads + 4 * (int64_t)threadIdx.x;
    unsigned c = 0;
    if (PACKED && first + 4 <= n_visible) {
        const uint4 k = __ldg(reinterpret_cast<const uint4*>(sorted_keys + first));   // the key buffers are 16-byte aligned
        c = (k.x >> kCountShift) + (k.y >> kCountShift) + (k.z >> kCountShift) + (k.w >> kCountShift) + 4u;
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int64_t s = first + q;
            if (s < n_visible) c += PACKED ? (__ldg(sorted_keys + s) >> kCountShift) + 1u : tiles_of(__ldg(bounds + checked_point(__ldg(sorted_ids + s))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
    if (lane_id() == 0) s_w[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned t = 0;
#pragma unroll
        for (int w = 0; w < kInstThreads / 4 / 32; ++w) t += s_w[w];
        block_sums[blockIdx.x] = t;
    }
}

constexpr int kScanItems = 8;
__global__ void __launch_bounds__(kScanThreads) scan_u32_kernel(unsigned* __restrict__ data, int64_t n) {
    __shared__ unsigned s_scan[kScanThreads / 32 + 1];
    unsigned running = 0;
    for (int64_t base = 0; base < n; base += (int64_t)kScanThreads * kScanItems) {
        const int64_t j0 = base + (int64_t)threadIdx.x * kScanItems;
        unsigned v[kScanItems];
        unsigned sum = 0;
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) {
            v[k] = j0 + k < n ? data[j0 + k] : 0u;
            sum += v[k];
        }
        unsigned total;
        unsigned ex = running + block_exclusive_scan(sum, s_scan, &total);
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) {
            if (j0 + k < n) data[j0 + k] = ex;
            ex += v[k];
        }
        running += total;
    }
}

// Instance key: the tile index in the low 24 bits, the only bits the tile sort looks at (it carries the
// bits above its range along).  For bilinear splats on 8x8 tiles the 8 bits above hold where the 2x2
// pixel footprint sits in the tile: column of its left pixel relative to the tile plus one (0..8) in
// bits 24..27, row of its upper pixel plus one in bits 28..31.  The blend then knows which pixels an
// instance can reach from the key alone, without fetching the point record.
constexpr unsigned kTileKeyBits = 24;
constexpr uint32_t kTileKeyMask = (1u << kTileKeyBits) - 1u;

// One (tile key, point id) pair per touched tile, row-major over the point's bounds, points in depth
// order (src/bilinear/kernels.cu:198-220).  CODED (bilinear, 8x8 tiles): bounds and footprint origin come
// from the packed word the projection pass left per point (see pack_quad), a 4-byte gather.
// (Four consecutive points per thread, with the four gathers in flight together, measured the same 0.12 ms for 2^23
// points: the kernel is bound by the throughput of the random 4-byte gathers, one 32-byte sector each, not by latency.)
template <bool CODED>
__global__ void __launch_bounds__(kInstThreads) emit_instances_kernel(const uint32_t* __restrict__ sorted_ids,
                                                                      const uint2* __restrict__ bounds, const uint32_t* __restrict__ quad,
                                                                      int64_t n_visible_arg, const unsigned long long* __restrict__ n_visible_dev,
                                                                      const unsigned* __restrict__ block_base, int gw,
                                                                      uint32_t* __restrict__ inst_keys,
                                                                      uint32_t* __restrict__ inst_ids) {
    __shared__ unsigned s_scan[kInstThreads / 32 + 1];
    const int64_t n_visible = n_visible_dev ? (int64_t)*n_visible_dev : n_visible_arg;
    if ((int64_t)blockIdx.x * kInstThreads >= n_visible) return;
    const int64_t s = (int64_t)blockIdx.x * kInstThreads + threadIdx.x;
    uint32_t id = 0;
    unsigned x0 = 0, x1 = 0, y0 = 0, y1 = 0;
    int qx = 0, qy = 0;
    if (s < n_visible) {
        id = checked_point(__ldg(sorted_ids + s));
        if (CODED) {
            // the tile bounds follow from the footprint origin: first tile = floor(origin / 8), never below 0
            const uint32_t q = __ldg(quad + id);
            qx = (int)(q & 0x7FFFu) - 1;
            x0 = qx < 0 ? 0u : (unsigned)qx >> 3;
            y0 = (q >> 16) & 0x7FFu;
            qy = (int)y0 * 8 + (int)((q >> 27) & 0xFu) - 1;   // row of the upper pixel in the stacked grid (or one above its image)
            x1 = x0 + 1u + ((q >> 15) & 1u);
            y1 = y0 + 1u + (q >> 31);
        } else {
            const uint2 b = __ldg(bounds + id);
            x0 = b.x & 0xffffu; x1 = b.x >> 16; y0 = b.y & 0xffffu; y1 = b.y >> 16;
        }
    }
    const unsigned c = (x1 - x0) * (y1 - y0);
    unsigned total;
    unsigned off = block_base[blockIdx.x] + block_exclusive_scan(c, s_scan, &total);
    for (unsigned ty = y0; ty < y1; ++ty)
        for (unsigned tx = x0; tx < x1; ++tx) {
            uint32_t key = ty * (unsigned)gw + tx;
            if (CODED) {
                const unsigned cx = (unsigned)min(max(qx - (int)tx * 8 + 1, 0), 8);
                const unsigned cy = (unsigned)min(max(qy - (int)ty * 8 + 1, 0), 8);
                key |= (cx << kTileKeyBits) | (cy << (kTileKeyBits + 4));
            }
            inst_keys[off] = key;
            inst_ids[off] = id;
            ++off;
        }
}

// Run boundaries of the sorted tile keys -> [first, last+1) per tile (src/bilinear/kernels.cu:222-239).
__global__ void __launch_bounds__(256) tile_ranges_kernel(const uint32_t* __restrict__ keys, int64_t n_instances_arg,
                                                          const unsigned long long* __restrict__ n_instances_dev,
                                                          uint2* __restrict__ ranges) {
    constexpr int kPer = 8;   // two 16-byte loads per thread (the key array is 256-byte aligned)
    const int64_t n_instances = n_instances_dev ? (int64_t)*n_instances_dev : n_instances_arg;
    const int64_t first = ((int64_t)blockIdx.x * 256 + threadIdx.x) * kPer;
    if (first >= n_instances) return;
    uint32_t prev = first > 0 ? __ldg(keys + first - 1) & kTileKeyMask : 0u;
    uint32_t k8[kPer];
    if (first + kPer <= n_instances) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(keys + first)), b = __ldg(reinterpret_cast<const uint4*>(keys + first) + 1);
        k8[0] = a.x; k8[1] = a.y; k8[2] = a.z; k8[3] = a.w; k8[4] = b.x; k8[5] = b.y; k8[6] = b.z; k8[7] = b.w;
    } else {
#pragma unroll
        for (int k = 0; k < kPer; ++k) k8[k] = first + k < n_instances ? __ldg(keys + first + k) : 0u;
    }
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
        const int64_t i = first + k;
        if (i >= n_instances) break;
        const uint32_t key = k8[k] & kTileKeyMask;
        if (i == 0) ranges[key].x = 0u;
        else if (key != prev) { ranges[prev].y = (unsigned)i; ranges[key].x = (unsigned)i; }
        if (i == n_instances - 1) ranges[key].y = (unsigned)n_instances;
        prev = key;
    }
}

// ------------------------------------------------------------------------------------------------
// Bilinear blend.
//
// (1) Per-pixel bit masks.  A point reaches only the 2x2 pixels whose centres lie within distance
// < 1 of it, so a block stages T*T instances at a time, every instance thread sets its bit in the
// masks of the (up to four) pixels it reaches, and every pixel thread then walks only its own set
// bits, in staged (= depth) order.  Per-fragment results that belong to the point (blending weight,
// gradients) go to a private shared-memory slot per (instance, footprint corner) and are reduced by
// the instance thread in a fixed order (the only shared-memory atomics are the ORs that build the masks),
// one global (vector) atomic per instance.  Two block barriers per batch.
//
// (2) Segments.  Front-to-back compositing is associative: (C, T) o (C', T') = (C + T C', T T').  A
// tile's instance list is cut into segments of at least 16 batches (at most 64 segments per tile) and
// every (tile, segment) pair is one block, so a tile that carries 100x the average load no longer
// sets the kernel's critical path.  For tiles with more than one segment a first pass computes each
// segment's per-pixel transmittance product, a per-tile prefix turns these into the transmittance at
// the start of every segment, and the main pass starts from that value (keeping the reference's
// early-termination rule); partial colours are added up per tile in segment order.  The backward
// pass starts every segment from the stored transmittance and colour prefix.
//
// Arithmetic per fragment: src/bilinear/kernels.cu:283-303 (forward), :361-415 (backward),
// :462-475 (inference).
// ------------------------------------------------------------------------------------------------
enum { BLEND_TRAIN = 0, BLEND_INFER = 1 };

struct __align__(16) Segment {
    uint32_t tile;
    uint32_t begin, end;   // instance range of this segment
    uint32_t info;         // index of the segment within its tile | number of segments of the tile << 16
};
constexpr int kMaxSegmentsPerTile = 64;
constexpr int kMinBatchesPerSegment = 16;

__device__ __forceinline__ unsigned segment_length(unsigned len, unsigned batch) {
    const unsigned s_min = batch * (unsigned)kMinBatchesPerSegment;
    const unsigned want = ceil_div(len, (unsigned)kMaxSegmentsPerTile);
    return max(s_min, ceil_div(want, batch) * batch);
}

// One block: number of segments per tile and their exclusive scan (tile_first), total in *n_segments.
__global__ void __launch_bounds__(kScanThreads) count_segments_kernel(const uint2* __restrict__ ranges, int n_tiles, int batch,
                                                                      uint32_t* __restrict__ tile_first,
                                                                      uint32_t* __restrict__ n_segments) {
    // four consecutive tiles per thread: short serial chains, two 16-byte loads
    constexpr int kItems = 4;
    __shared__ unsigned s_scan[kScanThreads / 32 + 1];
    unsigned running = 0;
    for (int base = 0; base < n_tiles; base += kScanThreads * kItems) {
        const int t0 = base + threadIdx.x * kItems;
        unsigned v[kItems];
        unsigned sum = 0;
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
            v[k] = 0u;
            if (t0 + k < n_tiles) {
                const uint2 r = __ldg(ranges + t0 + k);
                const unsigned len = r.y - r.x;
                v[k] = max(1u, ceil_div(len, segment_length(len, (unsigned)batch)));
            }
            sum += v[k];
        }
        unsigned total;
        unsigned ex = running + block_exclusive_scan(sum, s_scan, &total);
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
            if (t0 + k < n_tiles) tile_first[t0 + k] = ex;
            ex += v[k];
        }
        running += total;
    }
    if (threadIdx.x == 0) *n_segments = running;
}

// One thread per tile writes the tile's segment records.
__global__ void __launch_bounds__(256) emit_segments_kernel(const uint2* __restrict__ ranges, int n_tiles, int batch,
                                                            const uint32_t* __restrict__ tile_first, Segment* __restrict__ segs) {
    const int t = blockIdx.x * 256 + threadIdx.x;
    if (t >= n_tiles) return;
    const uint2 r = ranges[t];
    const unsigned len = r.y - r.x;
    const unsigned seg_len = segment_length(len, (unsigned)batch);
    const unsigned n = max(1u, ceil_div(len, seg_len));
    const unsigned first = tile_first[t];
    for (unsigned s = 0; s < n; ++s) {
        Segment g;
        g.tile = (uint32_t)t;
        g.begin = r.x + s * seg_len;
        g.end = min(r.y, g.begin + seg_len);
        g.info = s | (n << 16);
        segs[first + s] = g;
    }
}

// Stages instance `j` of the batch starting at `base`: record into shared memory, bit into the masks of
// the pixels it reaches.  Returns the point id.
template <int T, int B, bool NEED_F>
__device__ __forceinline__ uint32_t stage_instance(int j, int cnt, unsigned base, const uint32_t* __restrict__ inst_ids,
                                                   const PointRec* __restrict__ rec, int tile_x, int tile_y, float4* s_a,
                                                   float4* s_f, unsigned (*s_mask)[T * T]) {
    uint32_t id = 0;
    if (j < cnt) {
        id = checked_point(__ldg(inst_ids + base + j));
        const float4* r = reinterpret_cast<const float4*>(rec + id);
        const float4 a = __ldg(r);
        s_a[j] = a;
        if (NEED_F) s_f[j] = __ldg(r + 1);
        // first pixel column / row whose centre is within reach; the second is the next one
        const int qx = __float2int_rd(a.x - 0.5f) - tile_x * T;
        const int qy = __float2int_rd(a.y - 0.5f) - tile_y * T;
        const unsigned bit = 1u << (j & 31);
        unsigned* mrow = s_mask[j >> 5];
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
#pragma unroll
            for (int dx = 0; dx < 2; ++dx) {
                const int cx = qx + dx, cy = qy + dy;
                if (cx >= 0 && cx < T && cy >= 0 && cy < T) atomicOr(mrow + cy * T + cx, bit);
            }
    }
    return id;
}

// The same staging split in two, so that a batch's loads can be in flight while the batch before it is
// walked: `fetch` only issues the loads (instance id, then the record it names: two dependent trips to
// memory), `commit` writes the values to shared memory and sets the mask bits.
template <bool NEED_F>
struct Fetched {
    uint32_t id;
    float4 a, f;
};

template <bool NEED_F>
__device__ __forceinline__ Fetched<NEED_F> fetch_instance(int j, int cnt, unsigned base, const uint32_t* __restrict__ inst_ids,
                                                          const PointRec* __restrict__ rec) {
    Fetched<NEED_F> r;
    r.id = 0;
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.f = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < cnt) {
        r.id = checked_point(__ldg(inst_ids + base + j));
        const float4* p = reinterpret_cast<const float4*>(rec + r.id);
        r.a = __ldg(p);
        if (NEED_F) r.f = __ldg(p + 1);
    }
    return r;
}

template <int T, bool NEED_F>
__device__ __forceinline__ void commit_instance(int j, int cnt, const Fetched<NEED_F>& r, int tile_x, int tile_y, float4* s_a, float4* s_f,
                                                unsigned (*s_mask)[T * T]) {
    if (j < cnt) {
        s_a[j] = r.a;
        if (NEED_F) s_f[j] = r.f;
        const int qx = __float2int_rd(r.a.x - 0.5f) - tile_x * T;
        const int qy = __float2int_rd(r.a.y - 0.5f) - tile_y * T;
        const unsigned bit = 1u << (j & 31);
        unsigned* mrow = s_mask[j >> 5];
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
#pragma unroll
            for (int dx = 0; dx < 2; ++dx) {
                const int cx = qx + dx, cy = qy + dy;
                if (cx >= 0 && cx < T && cy >= 0 && cy < T) atomicOr(mrow + cy * T + cx, bit);
            }
    }
}

// Pass 1 (tiles with several segments only): per-pixel product of (1 - alpha) over one segment.
// A block is one (tile, segment): T*T threads = pixels, batches of B = T*T*IPT instances.
template <int T, int IPT>
__global__ void __launch_bounds__(T * T) blend_bilinear_transmittance_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, float* __restrict__ seg_T, int width, int height, int gw) {
    constexpr int P = T * T;
    constexpr int B = P * IPT;
    constexpr int WORDS = B / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu, n_seg = sg.info >> 16;
    if (n_seg == 1u || seg_idx == n_seg - 1u) return;   // the last segment's product is never needed

    __shared__ float4 s_a[B];
    __shared__ unsigned s_mask[WORDS][P];
    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
    __syncthreads();
    float Tr = 1.0f;
    bool done = !inside;
    // With 8x8 tiles the next batch's loads are issued before the current batch is walked (measured 3 %
    // faster); with 16x16 tiles the extra registers cost more than the overlap gains.
    constexpr bool kPrefetch = T == 8;
    Fetched<false> next[IPT];
    int cnt_next = (int)min((unsigned)B, sg.end - sg.begin);
    if (kPrefetch) {
#pragma unroll
        for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<false>(t + k * P, cnt_next, sg.begin, inst_ids, rec);
    }
    for (unsigned base = sg.begin; base < sg.end; base += B) {
        if (!kPrefetch) {
            cnt_next = (int)min((unsigned)B, sg.end - base);
#pragma unroll
            for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<false>(t + k * P, cnt_next, base, inst_ids, rec);
        }
        const int cnt = cnt_next;
#pragma unroll
        for (int k = 0; k < IPT; ++k) commit_instance<T, false>(t + k * P, cnt, next[k], tx, ty, s_a, nullptr, s_mask);
        if (kPrefetch) {
            cnt_next = base + B < sg.end ? (int)min((unsigned)B, sg.end - (base + B)) : 0;
#pragma unroll
            for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<false>(t + k * P, cnt_next, base + B, inst_ids, rec);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float dx = fabsf(a.x - pcx), dy = fabsf(a.y - pcy);
                if (dx >= 1.0f || dy >= 1.0f) continue;
                const float wgt = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                Tr *= 1.0f - a.z * wgt;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
        if (__syncthreads_count(done) == P) break;
    }
    seg_T[(size_t)blockIdx.x * P + t] = Tr;
}

// Per tile with several segments: products of the segments before -> transmittance at segment start.
template <int T>
__global__ void __launch_bounds__(T * T) blend_prefix_kernel(const Segment* __restrict__ segs, const uint32_t* __restrict__ tile_first,
                                                             float* __restrict__ seg_T) {
    constexpr int P = T * T;
    const unsigned first = tile_first[blockIdx.x];
    const unsigned n_seg = segs[first].info >> 16;
    if (n_seg == 1u) return;
    const int t = threadIdx.x;
    float run = 1.0f;
    for (unsigned s0 = 0; s0 < n_seg; s0 += 8) {
        float loc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const unsigned s = s0 + k;
            loc[k] = s + 1u < n_seg ? seg_T[(size_t)(first + s) * P + t] : 1.0f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const unsigned s = s0 + k;
            if (s < n_seg) seg_T[(size_t)(first + s) * P + t] = run;
            run *= loc[k];
        }
    }
}

template <int T, int IPT, int KIND>
__global__ void __launch_bounds__(T * T) blend_bilinear_forward_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, float* __restrict__ seg_T, float4* __restrict__ seg_C, float* __restrict__ seg_Z,
    float* __restrict__ image, float* __restrict__ depth_image, float* __restrict__ alpha_image,
    float* __restrict__ blending_weights, int width, int height, int gw) {
    constexpr int P = T * T;
    constexpr int B = P * IPT;
    constexpr int WORDS = B / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu, n_seg = sg.info >> 16;

    __shared__ float4 s_a[B];
    __shared__ float4 s_f[B];
    __shared__ unsigned s_mask[WORDS][P];
    __shared__ float s_slot[KIND == BLEND_TRAIN ? 4 : 1][KIND == BLEND_TRAIN ? B : 1];

    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
    const size_t state_idx = (size_t)blockIdx.x * P + t;

#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
    if (KIND == BLEND_TRAIN) {
#pragma unroll
        for (int k = 0; k < IPT; ++k)
#pragma unroll
            for (int q = 0; q < 4; ++q) s_slot[q][t + k * P] = 0.0f;
    }
    float C0 = 0.0f, C1 = 0.0f, C2 = 0.0f, C3 = 0.0f, Z = 0.0f;
    float Tr = 1.0f;
    if (seg_idx > 0u && inside) Tr = seg_T[state_idx];
    bool done = !inside || Tr < kTransmittanceEps;
    __syncthreads();

    uint32_t id[IPT];
    int cnt = 0;
    auto flush_weights = [&]() {
        // blending weights of the instances this thread staged last: the (up to) four fragments of each
        // in fixed order; the slots are cleared for the next batch
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            const int j = t + k * P;
            if (j < cnt) {
                const float sum = ((s_slot[0][j] + s_slot[1][j]) + s_slot[2][j]) + s_slot[3][j];
                if (sum > 0.0f) atomicAdd(blending_weights + id[k], sum);
                s_slot[0][j] = 0.0f; s_slot[1][j] = 0.0f; s_slot[2][j] = 0.0f; s_slot[3][j] = 0.0f;
            }
        }
    };
    // With 8x8 tiles the next batch's loads are issued before the current batch is walked (measured 3 %
    // faster); with 16x16 tiles the extra registers cost more than the overlap gains.
    constexpr bool kPrefetch = T == 8;
    Fetched<true> next[IPT];
    int cnt_next = (int)min((unsigned)B, sg.end - sg.begin);
    if (kPrefetch) {
#pragma unroll
        for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<true>(t + k * P, cnt_next, sg.begin, inst_ids, rec);
    }
    for (unsigned base = sg.begin; base < sg.end; base += B) {
        if (KIND == BLEND_TRAIN) flush_weights();
        if (!kPrefetch) {
            cnt_next = (int)min((unsigned)B, sg.end - base);
#pragma unroll
            for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<true>(t + k * P, cnt_next, base, inst_ids, rec);
        }
        cnt = cnt_next;
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            id[k] = next[k].id;
            commit_instance<T, true>(t + k * P, cnt, next[k], tx, ty, s_a, s_f, s_mask);
        }
        if (kPrefetch) {
            cnt_next = base + B < sg.end ? (int)min((unsigned)B, sg.end - (base + B)) : 0;
#pragma unroll
            for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<true>(t + k * P, cnt_next, base + B, inst_ids, rec);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float dx = fabsf(a.x - pcx), dy = fabsf(a.y - pcy);
                if (dx >= 1.0f || dy >= 1.0f) continue;
                const float wgt = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                const float al = a.z * wgt;
                const float bw = Tr * al;
                if (KIND == BLEND_TRAIN) {
                    // corner of the point's 2x2 footprint this pixel is: exactly one writer per slot
                    if (bw > 0.0f) s_slot[(pcx > a.x ? 1 : 0) + (pcy > a.y ? 2 : 0)][j] = bw * wgt;
                }
                const float4 f = s_f[j];
                C0 += bw * f.x; C1 += bw * f.y; C2 += bw * f.z; C3 += bw * f.w;
                if (KIND == BLEND_INFER) Z += bw * a.w;
                Tr *= 1.0f - al;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
        if (__syncthreads_count(done) == P) break;
    }
    if (KIND == BLEND_TRAIN) flush_weights();

    if (n_seg == 1u) {
        if (inside) {
            const int64_t n_px = (int64_t)width * height;
            const int64_t pi = (int64_t)py * width + px;
            image[pi] = C0;
            image[n_px + pi] = C1;
            image[2 * n_px + pi] = C2;
            image[3 * n_px + pi] = C3;
            if (KIND == BLEND_INFER) {
                const float A = 1.0f - Tr;
                depth_image[pi] = A > 0.0f ? Z / A : 0.0f;
                alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : A;
            } else {
                alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
            }
        }
    } else {
        // partial colour of this segment; the per-tile combine adds the segments up in order
        seg_C[state_idx] = make_float4(C0, C1, C2, C3);
        if (KIND == BLEND_INFER) {
            seg_Z[state_idx] = Z;
            seg_T[state_idx] = Tr;
        } else if (seg_idx == n_seg - 1u && inside) {
            alpha_image[(int64_t)py * width + px] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
        }
    }
}

// Per tile with several segments: image = sum of the segment colours in order.  For training the
// running sum before each segment is written back (the backward pass starts from it).
template <int T, int KIND>
__global__ void __launch_bounds__(T * T) blend_combine_kernel(const Segment* __restrict__ segs, const uint32_t* __restrict__ tile_first,
                                                              float4* __restrict__ seg_C, const float* __restrict__ seg_Z,
                                                              const float* __restrict__ seg_T, float* __restrict__ image,
                                                              float* __restrict__ depth_image, float* __restrict__ alpha_image,
                                                              int width, int height, int gw) {
    constexpr int P = T * T;
    const unsigned first = tile_first[blockIdx.x];
    const unsigned n_seg = segs[first].info >> 16;
    if (n_seg == 1u) return;
    const int t = threadIdx.x;
    const int tx = (int)(blockIdx.x % (unsigned)gw), ty = (int)(blockIdx.x / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
    float z = 0.0f;
    // transmittance where the pixel stopped: the end value of the first segment that fell below the
    // threshold (later segments start below it and only carry the product of everything skipped)
    float t_final = 1.0f;
    bool stopped = false;
    for (unsigned s0 = 0; s0 < n_seg; s0 += 4) {
        float4 c[4];
        float zz[4], tt[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const unsigned s = s0 + k;
            c[k] = s < n_seg ? seg_C[(size_t)(first + s) * P + t] : make_float4(0.f, 0.f, 0.f, 0.f);
            zz[k] = (KIND == BLEND_INFER && s < n_seg) ? seg_Z[(size_t)(first + s) * P + t] : 0.0f;
            tt[k] = (KIND == BLEND_INFER && s < n_seg) ? seg_T[(size_t)(first + s) * P + t] : 1.0f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const unsigned s = s0 + k;
            if (KIND == BLEND_TRAIN && s < n_seg) seg_C[(size_t)(first + s) * P + t] = run;
            run.x += c[k].x; run.y += c[k].y; run.z += c[k].z; run.w += c[k].w;
            z += zz[k];
            if (KIND == BLEND_INFER && s < n_seg && !stopped) {
                t_final = tt[k];
                stopped = t_final < kTransmittanceEps;
            }
        }
    }
    if (px < width && py < height) {
        const int64_t n_px = (int64_t)width * height;
        const int64_t pi = (int64_t)py * width + px;
        image[pi] = run.x;
        image[n_px + pi] = run.y;
        image[2 * n_px + pi] = run.z;
        image[3 * n_px + pi] = run.w;
        if (KIND == BLEND_INFER) {
            const float Tr = t_final;
            const float A = 1.0f - Tr;
            depth_image[pi] = A > 0.0f ? z / A : 0.0f;
            alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : A;
        }
    }
}

template <int T, int IPT>
__global__ void __launch_bounds__(T * T) blend_bilinear_backward_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, const float* __restrict__ seg_T, const float4* __restrict__ seg_C,
    const float* __restrict__ grad_image, const float* __restrict__ grad_alpha, const float* __restrict__ image,
    const float* __restrict__ alpha_image, float4* __restrict__ grad_feat_view, float* __restrict__ grad_opacity,
    int width, int height, int gw) {
    constexpr int P = T * T;
    constexpr int B = P * IPT;
    constexpr int WORDS = B / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu;
    if (sg.begin == sg.end) return;

    extern __shared__ __align__(16) unsigned char blend_smem[];
    float4* s_a = reinterpret_cast<float4*>(blend_smem);            // [B]
    float4* s_f = s_a + B;                                          // [B]
    float4* s_gf = s_f + B;                                         // [4][B] per footprint corner: feature gradient
    float* s_go = reinterpret_cast<float*>(s_gf + 4 * B);           // [4][B] per footprint corner: opacity gradient
    unsigned (*s_mask)[P] = reinterpret_cast<unsigned (*)[P]>(s_go + 4 * B);   // [WORDS][P]

    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
    const size_t state_idx = (size_t)blockIdx.x * P + t;

#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
#pragma unroll
    for (int k = 0; k < IPT; ++k)
#pragma unroll
        for (int q = 0; q < 4; ++q) { s_gf[q * B + t + k * P] = make_float4(0.f, 0.f, 0.f, 0.f); s_go[q * B + t + k * P] = 0.0f; }

    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), Cfin = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 Crun = make_float4(0.f, 0.f, 0.f, 0.f);
    float K = 0.0f, Tr = 1.0f;
    if (inside) {
        const int64_t n_px = (int64_t)width * height;
        const int64_t pi = (int64_t)py * width + px;
        g = make_float4(__ldg(grad_image + pi), __ldg(grad_image + n_px + pi), __ldg(grad_image + 2 * n_px + pi),
                        __ldg(grad_image + 3 * n_px + pi));
        Cfin = make_float4(__ldg(image + pi), __ldg(image + n_px + pi), __ldg(image + 2 * n_px + pi),
                           __ldg(image + 3 * n_px + pi));
        K = __ldg(grad_alpha + pi) * (1.0f - __ldg(alpha_image + pi));
        if (seg_idx > 0u) { Tr = seg_T[state_idx]; Crun = seg_C[state_idx]; }
    }
    bool done = !inside || Tr < kTransmittanceEps;
    __syncthreads();

    uint32_t id[IPT];
    int cnt = 0;
    auto flush_gradients = [&]() {
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            const int j = t + k * P;
            if (j < cnt) {
                float4 sf = s_gf[j];
                float so = s_go[j];
#pragma unroll
                for (int q = 1; q < 4; ++q) {
                    const float4 v = s_gf[q * B + j];
                    sf.x += v.x; sf.y += v.y; sf.z += v.z; sf.w += v.w;
                    so += s_go[q * B + j];
                }
                if (sf.x != 0.0f || sf.y != 0.0f || sf.z != 0.0f || sf.w != 0.0f) atomicAdd(grad_feat_view + id[k], sf);
                if (so != 0.0f) atomicAdd(grad_opacity + id[k], so);
#pragma unroll
                for (int q = 0; q < 4; ++q) { s_gf[q * B + j] = make_float4(0.f, 0.f, 0.f, 0.f); s_go[q * B + j] = 0.0f; }
            }
        }
    };
    // With 8x8 tiles the next batch's loads are issued before the current batch is walked (measured 3 %
    // faster); with 16x16 tiles the extra registers cost more than the overlap gains.
    constexpr bool kPrefetch = T == 8;
    Fetched<true> next[IPT];
    int cnt_next = (int)min((unsigned)B, sg.end - sg.begin);
    if (kPrefetch) {
#pragma unroll
        for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<true>(t + k * P, cnt_next, sg.begin, inst_ids, rec);
    }
    for (unsigned base = sg.begin; base < sg.end; base += B) {
        flush_gradients();
        if (!kPrefetch) {
            cnt_next = (int)min((unsigned)B, sg.end - base);
#pragma unroll
            for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<true>(t + k * P, cnt_next, base, inst_ids, rec);
        }
        cnt = cnt_next;
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            id[k] = next[k].id;
            commit_instance<T, true>(t + k * P, cnt, next[k], tx, ty, s_a, s_f, s_mask);
        }
        if (kPrefetch) {
            cnt_next = base + B < sg.end ? (int)min((unsigned)B, sg.end - (base + B)) : 0;
#pragma unroll
            for (int k = 0; k < IPT; ++k) next[k] = fetch_instance<true>(t + k * P, cnt_next, base + B, inst_ids, rec);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float dx = fabsf(a.x - pcx), dy = fabsf(a.y - pcy);
                if (dx >= 1.0f || dy >= 1.0f) continue;
                const float wgt = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                const float al = a.z * wgt;
                const float bw = Tr * al;
                const int q = (pcx > a.x ? 1 : 0) + (pcy > a.y ? 2 : 0);
                if (bw > 0.0f) s_gf[q * B + j] = make_float4(bw * g.x, bw * g.y, bw * g.z, bw * g.w);
                const float4 f = s_f[j];
                Crun.x += bw * f.x; Crun.y += bw * f.y; Crun.z += bw * f.z; Crun.w += bw * f.w;
                const float oma = 1.0f - al;
                const float rcp = 1.0f / fmaxf(oma, kOneMinusAlphaEps);
                const float from_features = (Tr * f.x + (Crun.x - Cfin.x) * rcp) * g.x +
                                            (Tr * f.y + (Crun.y - Cfin.y) * rcp) * g.y +
                                            (Tr * f.z + (Crun.z - Cfin.z) * rcp) * g.z +
                                            (Tr * f.w + (Crun.w - Cfin.w) * rcp) * g.w;
                const float dalpha = from_features + K * rcp;
                const float dop = dalpha * wgt;
                if (dop != 0.0f) s_go[q * B + j] = dop;
                Tr *= oma;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
        if (__syncthreads_count(done) == P) break;
    }
    flush_gradients();
}

template <int T, int IPT>
constexpr size_t backward_smem_bytes() {
    return (size_t)T * T * IPT * (16 + 16 + 4 * 16 + 4 * 4) + (size_t)(T * T * IPT / 32) * T * T * 4;
}

// ------------------------------------------------------------------------------------------------
// Bilinear blend on 8x8 tiles, one warp per work item (the default path).
//
// (1) Dead instances.  A pixel stops taking fragments once its transmittance has fallen below the
// threshold, and in a dense scene most instances of a tile's list lie behind pixels that have already
// stopped.  Such an instance has no effect whatsoever, so it is discarded from its sort key alone --
// the key says which pixels of the tile it reaches (see kTileKeyBits), a mask of stopped pixels lives
// in registers -- and its 32-byte record is never fetched.  A warp streams the keys of its item (128
// per step, loaded one step ahead), pushes the point ids of the instances that may still contribute
// into a ring in shared memory and blends them in batches of 32, the records of the next batch being
// in flight while the current one is blended.  The mask used by the filter lags the blend by a batch;
// that only lets a few extra instances through, whose fragments are then dropped.
//
// (2) A batch.  The geometry of a fragment (bilinear weight, alpha) depends on nothing that came
// before it, the blend itself is a serial chain per pixel.  So lane j first evaluates the (up to) four
// fragments of staged instance j, then the fragments are brought into per-pixel order in shared
// memory (bit masks per pixel give every fragment its rank, a scan of the counts gives every pixel
// its offset), and only then does every lane run down the short list of its own pixel: load alpha
// and features, accumulate, update the transmittance.  What a fragment saw (its transmittance) goes
// back to the instance lane, which forms the per-point sums in fixed corner order.  The arithmetic
// and its order are those of a plain front-to-back loop per pixel.
//
// (3) Segments.  Front-to-back compositing is associative: (C, T) o (C', T') = (C + T C', T T').  A
// tile's list is cut into a first segment of kFirstSegment instances and later ones of kLaterSegment, and every (tile half, segment) is one
// item, so a tile with 100x the average load does not set the critical path.  Pass FIRST blends
// segment 0 of every tile exactly; the pixels that dense clusters hit stop there.  Pass PRODUCT
// computes, for the later segments, the per-pixel product of (1 - alpha) over the segment, starting
// from (and filtering by) the state segment 0 left, so the work it repeats is small; a per-tile
// prefix turns the products into the transmittance at segment start; pass REST blends the later
// segments from that state; a per-tile combine adds the segment colours in order (and leaves the
// colour prefix for the backward pass, whose items are then independent).
//
// An item covers the upper or lower 8x4 half of a tile, one pixel per lane; both halves stream the same
// list and each keeps what reaches its own pixels.
//
// The forward passes write the compacted lists they blended (point ids in depth order, per item) for
// the backward pass, which therefore neither filters nor reads keys.
//
// Arithmetic per fragment: src/bilinear/kernels.cu:283-303 (forward), :361-415 (backward),
// :462-475 (inference).
// ------------------------------------------------------------------------------------------------
constexpr int kWarpBlendWarps = 8;        // warps per block; every warp works on items of its own
constexpr int kQueueCap = 256;            // ring of candidate point ids per warp: >= 31 left over + 128 of one filter step
constexpr int kFilterKeys = 4;            // keys per lane and filter step
// Measured on B200 (2^23 clustered samples, 1237x822; forward / backward stage in microseconds), first + later segment:
// 1024 + 4096: 422 / 276, 1024 + 2048: 439 / 268, 512 + 4096: 437 / 297, 512 + 2048: 458 / 274, 1024 + 1024: 488 / 291,
// 512 + 1024: 518 / 283, 256 + 2048: 469 / 283.  Per-item timestamps of the same run: every pass is full (about 3000 of
// the 3552 resident warps busy) for its first half and then drains for as long again while the longest items finish at
// 1.0 - 1.4 us per batch; shorter segments shorten that tail but add more work (more lists to filter, more states to
// carry) than they save.
constexpr unsigned kFirstSegment = 1024;    // instances in a tile's first segment
constexpr unsigned kLaterSegment = 4096;    // ... and in every later one
constexpr int kBatchFragments = 128;      // 32 instances x 4 fragments
enum { PASS_FIRST = 0, PASS_PRODUCT = 1, PASS_REST = 2 };

// Pixels of the tile (bit = row * 8 + column) that the instance with this key reaches.
__device__ __forceinline__ unsigned long long key_pixels(unsigned code) {
    const unsigned cx = code & 15u, cy = code >> 4;
    const unsigned m = ((3u << cx) >> 1) & 0xFFu;                        // columns cx - 1 and cx, clipped to the tile
    const unsigned long long two = (unsigned long long)(m | (m << 8));   // the same columns in two consecutive rows
    if (cx > 8u || cy > 8u) return 0ull;
    return cy == 0u ? two >> 8 : two << (8u * (cy - 1u));                // rows cy - 1 and cy, clipped likewise
}

__device__ __forceinline__ unsigned warp_segments(unsigned len) {
    return len <= kFirstSegment ? 1u : 1u + ceil_div(len - kFirstSegment, kLaterSegment);
}

// Work lists of the warp blend.  Step 1 (one block per 1024 tiles): segments and non-empty tiles of the block's tiles.
// Step 2 (one block): exclusive scan of those block sums; counts[0] = non-empty tiles, counts[1] = segments behind a
// tile's first.  Step 3 (same blocks as step 1): every tile's position from its block's base and a scan inside the
// block, and its items.  (One block scanning all tiles took 177 us for the 129,600 tiles of a 3840x2160 image.)
constexpr int kItemThreads = 256;
constexpr int kItemTilesPerThread = 4;
constexpr int kItemTilesPerBlock = kItemThreads * kItemTilesPerThread;

__device__ __forceinline__ void load_tile_segments(const uint2* __restrict__ ranges, int n_tiles, int t0, unsigned (&ns)[kItemTilesPerThread],
                                                   uint2 (&rg)[kItemTilesPerThread]) {
#pragma unroll
    for (int k = 0; k < kItemTilesPerThread; k += 2) {
        // two ranges per 16-byte load (t0 is even, the array 256-byte aligned)
        uint4 r = make_uint4(0u, 0u, 0u, 0u);
        if (t0 + k + 1 < n_tiles) r = __ldg(reinterpret_cast<const uint4*>(ranges + t0 + k));
        else if (t0 + k < n_tiles) { const uint2 r0 = __ldg(ranges + t0 + k); r.x = r0.x; r.y = r0.y; }
        rg[k] = make_uint2(r.x, r.y);
        rg[k + 1] = make_uint2(r.z, r.w);
        ns[k] = r.y > r.x ? warp_segments(r.y - r.x) : 0u;
        ns[k + 1] = r.w > r.z ? warp_segments(r.w - r.z) : 0u;
    }
}

__global__ void __launch_bounds__(kItemThreads) warp_items_count_kernel(const uint2* __restrict__ ranges, int n_tiles, uint2* __restrict__ block_sums) {
    __shared__ unsigned s_seg[kItemThreads / 32], s_tiles[kItemThreads / 32];
    unsigned ns[kItemTilesPerThread];
    uint2 rg[kItemTilesPerThread];
    load_tile_segments(ranges, n_tiles, blockIdx.x * kItemTilesPerBlock + threadIdx.x * kItemTilesPerThread, ns, rg);
    unsigned seg = 0, tiles = 0;
#pragma unroll
    for (int k = 0; k < kItemTilesPerThread; ++k) { seg += ns[k]; tiles += ns[k] ? 1u : 0u; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        seg += __shfl_down_sync(0xffffffffu, seg, o);
        tiles += __shfl_down_sync(0xffffffffu, tiles, o);
    }
    if (lane_id() == 0) { s_seg[threadIdx.x >> 5] = seg; s_tiles[threadIdx.x >> 5] = tiles; }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned a = 0, c = 0;
#pragma unroll
        for (int w = 0; w < kItemThreads / 32; ++w) { a += s_seg[w]; c += s_tiles[w]; }
        block_sums[blockIdx.x] = make_uint2(a, c);
    }
}

__global__ void __launch_bounds__(kScanThreads) warp_items_scan_kernel(uint2* __restrict__ block_sums, int n_blocks, uint32_t* __restrict__ counts) {
    __shared__ unsigned s_scan[kScanThreads / 32 + 1];
    unsigned run_seg = 0, run_tiles = 0;
    for (int base = 0; base < n_blocks; base += kScanThreads) {
        const int j = base + threadIdx.x;
        const uint2 v = j < n_blocks ? block_sums[j] : make_uint2(0u, 0u);
        unsigned total_seg, total_tiles;
        const unsigned ex_seg = run_seg + block_exclusive_scan(v.x, s_scan, &total_seg);
        const unsigned ex_tiles = run_tiles + block_exclusive_scan(v.y, s_scan, &total_tiles);
        if (j < n_blocks) block_sums[j] = make_uint2(ex_seg, ex_tiles);
        run_seg += total_seg;
        run_tiles += total_tiles;
    }
    if (threadIdx.x == 0) { counts[0] = run_tiles; counts[1] = run_seg - run_tiles; }
}

// Everything a warp needs to know about a (tile, segment), in one 32-byte record: the blend kernels read it with
// two 16-byte loads, one item ahead of the one they work on, instead of chasing tile -> range -> first segment.
struct __align__(16) WarpItem {
    uint32_t tile, seg;       // which tile, which of its segments
    uint32_t begin, end;      // instance range of the segment
    uint32_t first, n_seg;    // slot of the tile's segment 0 in the per-segment arrays; segments of the tile
    uint32_t pad0, pad1;
};

__device__ __forceinline__ WarpItem load_item(const WarpItem* p) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p)), b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    WarpItem w;
    w.tile = a.x; w.seg = a.y; w.begin = a.z; w.end = a.w; w.first = b.x; w.n_seg = b.y; w.pad0 = 0; w.pad1 = 0;
    return w;
}

// Step 3: items0 = segment 0 of the non-empty tiles, items1 = every later segment, tile by tile.
__global__ void __launch_bounds__(kItemThreads) warp_items_fill_kernel(const uint2* __restrict__ ranges, int n_tiles,
                                                                      const uint2* __restrict__ block_base, WarpItem* __restrict__ items0,
                                                                      WarpItem* __restrict__ items1) {
    __shared__ unsigned s_scan[kItemThreads / 32 + 1];
    unsigned ns[kItemTilesPerThread];
    uint2 rg[kItemTilesPerThread];
    const int t0 = blockIdx.x * kItemTilesPerBlock + threadIdx.x * kItemTilesPerThread;
    load_tile_segments(ranges, n_tiles, t0, ns, rg);
    unsigned seg = 0, tiles = 0;
#pragma unroll
    for (int k = 0; k < kItemTilesPerThread; ++k) { seg += ns[k]; tiles += ns[k] ? 1u : 0u; }
    const uint2 base = __ldg(block_base + blockIdx.x);
    unsigned total;
    unsigned first = base.x + block_exclusive_scan(seg, s_scan, &total);     // segments of the tiles before this one
    unsigned rank = base.y + block_exclusive_scan(tiles, s_scan, &total);    // non-empty tiles before this one
#pragma unroll
    for (int k = 0; k < kItemTilesPerThread; ++k) {
        if (ns[k] == 0u) continue;
        const uint2 r = rg[k];
        for (unsigned sg = 0; sg < ns[k]; ++sg) {
            const unsigned begin = sg == 0 ? r.x : r.x + kFirstSegment + (sg - 1u) * kLaterSegment;
            const unsigned end = min(r.y, begin + (sg == 0 ? kFirstSegment : kLaterSegment));
            // later segments: position = segments before this tile minus tiles before it
            WarpItem* dst = sg == 0 ? items0 + rank : items1 + (first - rank + sg - 1u);
            reinterpret_cast<uint4*>(dst)[0] = make_uint4((uint32_t)(t0 + k), sg, begin, end);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(first, ns[k], 0u, 0u);
        }
        first += ns[k];
        rank += 1u;
    }
}

// Asynchronous copies (global -> shared, 16 bytes, not through registers) and their completion groups.
__device__ __forceinline__ void async_copy_16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void async_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void async_copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A warp walks its list one batch of 32 instances at a time, and a batch cannot start before its 32 records have
// arrived (gathers from DRAM or, for the other half of the tile and for neighbouring tiles, from L1: hence the
// L1-caching form of the copy -- the form that bypasses L1 made the blend of a dense 2^25-point scene 30 % slower).
// The records of the next batch travel while the current one is blended, copied asynchronously into a two-stage ring
// in shared memory rather than through registers, and the per-pixel loops read a fragment's features from that
// ring instead of from a copy per fragment.  Measured with four stages (three batches in flight): the same
// single-view time, but 6 % less throughput with four views in flight on four streams (4985 against 5315
// Mpoints/s), since the larger rings leave room for fewer blocks of other views' kernels on an SM.
constexpr int kGatherDepthFilter = 2;     // stages of the ring, a power of two: first segments and products,
constexpr int kGatherDepthRest = 2;       // later segments,
constexpr int kGatherDepthBackward = 2;   // backward pass
constexpr int kIdsAhead = 3;      // later segments: batches whose point ids are loaded ahead of their gather

// Shared memory of one warp of the forward passes.
template <bool BLEND, bool WEIGHTS, int DEPTH>
struct __align__(16) WarpForwardSmem {
    float4 ring_a[DEPTH][32];                        // records of the batches in flight: position, alpha, depth ...
    float4 ring_f[BLEND ? DEPTH : 1][32];            // ... and features
    float2 frag[kBatchFragments];                    // fragments in per-pixel order: alpha, lane of the staged instance
    float frag_seen[WEIGHTS ? kBatchFragments : 1];  // transmittance the fragment met (0: it was dropped)
    uint32_t ring_id[DEPTH][32];                     // point ids of the batches in flight (0xFFFFFFFF: no instance)
    unsigned mask[32];                               // per pixel: staged instances with a fragment there
    unsigned off[32];                                // per pixel: first slot of its fragment list
    uint32_t queue[kQueueCap];
};

template <int PASS, int KIND>
constexpr size_t warp_forward_smem_bytes() {
    return 256 * sizeof(unsigned long long) +
           kWarpBlendWarps * sizeof(WarpForwardSmem<PASS != PASS_PRODUCT, PASS != PASS_PRODUCT && KIND == BLEND_TRAIN,
                                                    PASS == PASS_REST ? kGatherDepthRest : kGatherDepthFilter>);
}

template <int PASS, int KIND>
__global__ void __launch_bounds__(kWarpBlendWarps * 32, PASS == PASS_PRODUCT ? 4 : 3) blend_bilinear_warp_forward_kernel(
    const WarpItem* __restrict__ items, const uint32_t* __restrict__ counts, unsigned* __restrict__ ticket, const uint32_t* __restrict__ inst_keys,
    const uint32_t* __restrict__ inst_ids, const PointRec* __restrict__ rec, float* __restrict__ seg_T, float4* __restrict__ seg_C,
    float* __restrict__ seg_Z, float* __restrict__ seg_E, float* __restrict__ image, float* __restrict__ depth_image,
    float* __restrict__ alpha_image, float* __restrict__ blending_weights, uint32_t* kept0, uint32_t* kept1,
    uint32_t* __restrict__ n_kept, int width, int height, int gw, int gh) {
    constexpr unsigned kFull = 0xffffffffu;
    constexpr unsigned kNoInstance = 0xffffffffu;
    constexpr bool kBlend = PASS != PASS_PRODUCT;               // colours and weights; PRODUCT only multiplies
    constexpr bool kWeights = kBlend && KIND == BLEND_TRAIN;
    constexpr bool kDepth = kBlend && KIND == BLEND_INFER;
    constexpr int kGatherDepth = PASS == PASS_REST ? kGatherDepthRest : kGatherDepthFilter;
    using Smem = WarpForwardSmem<kBlend, kWeights, kGatherDepth>;
    extern __shared__ __align__(16) unsigned char blend_smem[];
    unsigned long long* s_reach = reinterpret_cast<unsigned long long*>(blend_smem);     // key code -> pixels reached
    Smem& sm = reinterpret_cast<Smem*>(blend_smem + 256 * sizeof(unsigned long long))[threadIdx.x >> 5];
    const unsigned lane = lane_id();
    const unsigned lt_mask = (1u << lane) - 1u;
    s_reach[threadIdx.x] = key_pixels(threadIdx.x);
    sm.mask[lane] = 0u;   // the masks start at zero and every batch leaves them at zero again
    sm.off[lane] = 0u;    // (the product pass uses both arrays as per-pixel accumulators)
    __syncthreads();
    const unsigned n_items = __ldg(counts + (PASS == PASS_FIRST ? 0 : 1)) * 2u;
    // Items are handed out one at a time through a ticket counter: consecutive items cost about the same (neighbouring
    // tiles, or consecutive segments of one tile), so a warp that reserved items ahead would sit on work that idle warps
    // could take (measured: holding two tickets ahead to prefetch the records made every pass 10-70 % slower).
    // ... unless there are very many of them: a single counter hands out one ticket every 2.7 ns at best (measured:
    // 259,200 items of a 3840x2160 image took 700 us whatever the occupancy), so with many small items a warp takes
    // several consecutive ones per visit.
    const unsigned per_visit = max(1u, min(8u, n_items / (gridDim.x * kWarpBlendWarps * 8u)));
    unsigned next_item = 0, visit_end = 0;
    for (;;) {
        if (next_item == visit_end) {
            unsigned first_item = 0;
            if (lane == 0) first_item = atomicAdd(ticket, per_visit);
            first_item = __shfl_sync(kFull, first_item, 0);
            if (first_item >= n_items) break;
            next_item = first_item;
            visit_end = min(first_item + per_visit, n_items);
        }
        const unsigned item = next_item++;
        const WarpItem it = load_item(items + (item >> 1));
        const unsigned tile = it.tile, seg = it.seg, n_seg = it.n_seg, first = it.first;
        const int half = (int)(item & 1u);
        const size_t sidx = (size_t)(first + seg) * 2u + half;      // this item's slot in the per-segment arrays
        const size_t sidx0 = (size_t)first * 2u + half;             // segment 0 of the same tile half
        const uint2 rg = make_uint2(it.begin, it.end);
        // rows [j gh, (j + 1) gh) of the tile grid are image j of the call (one image except for batched inference)
        const int tx = (int)(tile % (unsigned)gw), ty_all = (int)(tile / (unsigned)gw);
        const int set = ty_all / gh, ty = ty_all - set * gh;
        const int px0 = tx * 8, py0 = ty * 8 + 4 * half;            // first pixel of this half
        const int px = px0 + (int)(lane & 7u), py = py0 + (int)(lane >> 3);
        const bool inside = px < width && py < height;

        float Tr = 1.0f, Z = 0.0f, C0 = 0.0f, C1 = 0.0f, C2 = 0.0f, C3 = 0.0f;
        double log_sum = 0.0, log_stop = 0.0;   // PRODUCT: -log2 of the product so far, and where the pixel counts as stopped
        bool done = !inside;
        if (PASS == PASS_PRODUCT) {
            // the state segment 0 left: a pixel that has stopped there stays stopped; for the others the
            // product is taken until T0 * product falls below the threshold (the true transmittance at
            // that point is smaller still, so everything behind is dead whatever the product says).  The margin
            // keeps a pixel open when the sum's rounding could be what carries it over the line.
            const float T0 = seg_T[sidx0 * 32 + lane];
            done = done || T0 < kTransmittanceEps;
            log_stop = done ? 0.0 : log2((double)T0 / (double)kTransmittanceEps) + 1e-4;
        } else if (PASS == PASS_REST) {
            Tr = seg_T[sidx * 32 + lane];
            done = done || Tr < kTransmittanceEps;
        }
        unsigned done_w = __ballot_sync(kFull, done);   // bit l = pixel of lane l has stopped (warp-uniform)

        uint32_t* kept = half ? kept1 : kept0;
        unsigned n_out = 0;
        if (done_w != kFull) {   // else: nothing in this list can have an effect, and it is not even read
            // ---- where the instances come from.  FIRST and PRODUCT filter the item's keys (loaded one step ahead of
            // their use); REST blends the list PRODUCT compacted for this item (a superset of what is still alive at
            // the true transmittance, see above), its ids loaded kIdsAhead batches ahead of their gather.
            unsigned pos = rg.x;           // next key to load
            bool loaded = false;
            uint32_t kq[kFilterKeys], iq[kFilterKeys];
            auto load_step = [&]() {
#pragma unroll
                for (int k = 0; k < kFilterKeys; ++k) {
                    const unsigned idx = pos + 32u * k + lane;
                    const bool ok = idx < rg.y;
                    kq[k] = ok ? __ldg(inst_keys + idx) : 0xFFFFFFFFu;   // code 0xFF reaches nothing
                    iq[k] = ok ? __ldg(inst_ids + idx) : 0u;
                }
                pos = min(pos + 32u * kFilterKeys, rg.y);
                loaded = true;
            };
            unsigned q_head = 0, q_tail = 0;   // candidates [q_head, q_tail) wait for their gather
            // (measured: a second filter step of keys in flight gains 10 % in the PRODUCT pass and loses as much in FIRST)
            auto fill = [&]() {
                while (PASS != PASS_REST && q_tail - q_head < 32u && loaded) {
                    uint32_t ck[kFilterKeys], ci[kFilterKeys];
#pragma unroll
                    for (int k = 0; k < kFilterKeys; ++k) { ck[k] = kq[k]; ci[k] = iq[k]; }
                    loaded = false;
                    if (pos < rg.y) load_step();
#pragma unroll
                    for (int k = 0; k < kFilterKeys; ++k) {
                        const unsigned long long reach = s_reach[ck[k] >> kTileKeyBits];
                        const bool keep = ((unsigned)(reach >> (32 * half)) & ~done_w) != 0u;
                        const unsigned b = __ballot_sync(kFull, keep);
                        if (keep) sm.queue[(q_tail + __popc(b & lt_mask)) & (kQueueCap - 1)] = ci[k];
                        q_tail += __popc(b);
                    }
                }
                __syncwarp();
            };
            uint32_t idf[kIdsAhead];
            if (PASS == PASS_REST) {
                q_tail = n_kept[sidx];     // length of PRODUCT's list; the list itself starts at kept[rg.x]
#pragma unroll
                for (int k = 0; k < kIdsAhead; ++k) idf[k] = 32u * k + lane < q_tail ? kept[rg.x + 32u * k + lane] : 0u;
            } else if (pos < rg.y) {
                load_step();
            }
            // the next (up to) 32 candidates become a batch: their records start to travel into `stage` of the ring
            auto gather = [&](unsigned stage) {
                const unsigned n = min(32u, q_tail - q_head);
                uint32_t id = kNoInstance;
                if (lane < n) {
                    id = checked_point(PASS == PASS_REST ? idf[0] : sm.queue[(q_head + lane) & (kQueueCap - 1)]);
                    const float4* p = reinterpret_cast<const float4*>(rec + id);
                    async_copy_16(&sm.ring_a[stage][lane], p);
                    if (kBlend) async_copy_16(&sm.ring_f[stage][lane], p + 1);
                }
                sm.ring_id[stage][lane] = id;
                async_copy_commit();   // one group per batch, empty or not: the waits below count groups
                if (PASS == PASS_REST) {
#pragma unroll
                    for (int k = 0; k + 1 < kIdsAhead; ++k) idf[k] = idf[k + 1];
                    const unsigned nxt = q_head + 32u * kIdsAhead + lane;
                    idf[kIdsAhead - 1] = nxt < q_tail ? kept[rg.x + nxt] : 0u;
                }
                q_head += n;
            };
            fill();
#pragma unroll
            for (int st = 0; st + 1 < kGatherDepth; ++st) {
                gather((unsigned)st);
                fill();
            }
            for (unsigned batch = 0;; ++batch) {
                gather((batch + kGatherDepth - 1) & (kGatherDepth - 1));
                async_copy_wait<kGatherDepth - 1>();   // all but the newest kGatherDepth - 1 groups: this batch has arrived
                const unsigned stage = batch & (kGatherDepth - 1);
                const uint32_t id_cur = sm.ring_id[stage][lane];
                const bool staged = id_cur != kNoInstance;
                if (__ballot_sync(kFull, staged) == 0u) break;   // batches are filled in order: nothing is left
                const float4 a_cur = sm.ring_a[stage][lane];
                fill();
                // ---- lane j: the fragments of staged instance j
                const int qx = __float2int_rd(a_cur.x - 0.5f) - px0;
                const int qy = __float2int_rd(a_cur.y - 0.5f) - py0;
                float al[4], wg[4];
                int pix[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int cx = qx + (c & 1), cy = qy + (c >> 1);
                    const float pcx = (float)(px0 + cx) + 0.5f, pcy = (float)(py0 + cy) + 0.5f;
                    const float dx = fabsf(a_cur.x - pcx), dy = fabsf(a_cur.y - pcy);
                    wg[c] = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                    al[c] = a_cur.z * wg[c];
                    const int p = cy * 8 + cx;
                    const bool ok = staged && cx >= 0 && cx < 8 && cy >= 0 && cy < 4 && dx < 1.0f && dy < 1.0f &&
                                    !((done_w >> (p & 31)) & 1u);
                    pix[c] = ok ? p : -1;
                    if (PASS != PASS_PRODUCT) {
                        if (ok) atomicOr(sm.mask + p, 1u << lane);
                    } else if (ok) {
                        // A product does not care about order.  Its factors are added up as -log2(1 - alpha) in fixed
                        // point (integer part and 24 fractional bits in two words per pixel): integer atomics commute, so
                        // the sum is the same on every run, and none of the per-pixel ordering below is needed.
                        const float x = 1.0f - al[c];
                        const float t = x > 0.0f ? fminf(-log2f(x), 64.0f) : 64.0f;   // 2^-64: far below the threshold
                        const float ti = floorf(t);
                        atomicAdd(sm.mask + p, __float2uint_rn((t - ti) * 16777216.0f));
                        if (ti > 0.0f) atomicAdd(sm.off + p, (unsigned)ti);
                    }
                }
                if (PASS == PASS_PRODUCT || kWeights) {   // inference keeps no lists for a backward pass
                    // What reaches a pixel that has not stopped goes into the list of this item: FIRST's list is the
                    // backward pass's, PRODUCT's is blended by REST, REST's (what is still alive at the true
                    // transmittance; written in place, behind the part of PRODUCT's list already read) the backward
                    // pass's again.  The filter runs several batches ahead of the blend, so some of what it let
                    // through is dead by now and is dropped here.
                    const bool live = (pix[0] & pix[1] & pix[2] & pix[3]) >= 0;
                    const unsigned b = __ballot_sync(kFull, live);
                    if (live) kept[rg.x + n_out + __popc(b & lt_mask)] = id_cur;
                    n_out += __popc(b);
                }
                __syncwarp();
                if (PASS == PASS_PRODUCT) {
                    const unsigned frac = sm.mask[lane], whole = sm.off[lane];
                    if (frac | whole) {
                        sm.mask[lane] = 0u;
                        sm.off[lane] = 0u;
                        log_sum += (double)whole + (double)frac * (1.0 / 16777216.0);
                    }
                    done = done || log_sum > log_stop;
                    done_w = __ballot_sync(kFull, done);
                    __syncwarp();
                    if (done_w == kFull) break;   // every pixel has stopped: the rest of the list has no effect
                    continue;
                }
                // ---- per-pixel order: offset of every pixel's list, slot of every fragment
                const unsigned my_mask = sm.mask[lane];
                const unsigned cnt = __popc(my_mask);
                const unsigned off = warp_inclusive_scan(cnt) - cnt;
                sm.off[lane] = off;
                __syncwarp();
                int slot[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    slot[c] = 0;
                    if (pix[c] >= 0) {
                        slot[c] = (int)(sm.off[pix[c]] + __popc(sm.mask[pix[c]] & lt_mask));
                        sm.frag[slot[c]] = make_float2(al[c], __uint_as_float(lane));
                    }
                }
                __syncwarp();
                // ---- every lane runs down the list of its own pixel, front to back
                if (my_mask) sm.mask[lane] = 0u;
                // The chain from one fragment to the next is one multiply (the transmittance); everything else of a step
                // hangs off it.  The steps are therefore written without branches -- a stopped pixel selects its old
                // values -- and in chunks whose loads are issued together, so that consecutive steps overlap in the
                // pipeline instead of each waiting for its own shared-memory loads.
                constexpr int kChunk = 4;
                for (unsigned k0 = off; k0 < off + cnt; k0 += kChunk) {
                    float a[kChunk];
                    float4 f[kChunk];
                    float zd[kChunk];
#pragma unroll
                    for (int u = 0; u < kChunk; ++u) {
                        const unsigned k = min(k0 + u, off + cnt - 1u);   // the tail repeats the last slot: masked out below
                        const float2 e = sm.frag[k];
                        a[u] = e.x;
                        if (kBlend) f[u] = sm.ring_f[stage][__float_as_uint(e.y)];
                        if (kDepth) zd[u] = sm.ring_a[stage][__float_as_uint(e.y)].w;
                    }
#pragma unroll
                    for (int u = 0; u < kChunk; ++u) {
                        const bool live = !done && k0 + u < off + cnt;
                        if (kBlend) {
                            const float bw = Tr * a[u];
                            if (kWeights && k0 + u < off + cnt) sm.frag_seen[k0 + u] = live ? Tr : 0.0f;
                            C0 = live ? C0 + bw * f[u].x : C0;
                            C1 = live ? C1 + bw * f[u].y : C1;
                            C2 = live ? C2 + bw * f[u].z : C2;
                            C3 = live ? C3 + bw * f[u].w : C3;
                            if (kDepth) Z = live ? Z + bw * zd[u] : Z;
                            Tr = live ? Tr * (1.0f - a[u]) : Tr;
                            done = done || Tr < kTransmittanceEps;
                        }
                    }
                }
                __syncwarp();
                if (kWeights) {
                    // blending weight of every staged instance: its (up to) four fragments in fixed corner order
                    if (staged) {
                        float v[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float bw = pix[c] >= 0 ? sm.frag_seen[slot[c]] * al[c] : 0.0f;
                            v[c] = bw > 0.0f ? bw * wg[c] : 0.0f;
                        }
                        const float sum = ((v[0] + v[1]) + v[2]) + v[3];
                        if (sum > 0.0f) atomicAdd(blending_weights + id_cur, sum);
                    }
                }
                done_w = __ballot_sync(kFull, done);
                __syncwarp();
                if (done_w == kFull) break;   // every pixel has stopped: the rest of the list has no effect
            }
            async_copy_wait<0>();   // whatever is still travelling lands before the next item reuses the ring
            __syncwarp();
        }
        if ((PASS == PASS_PRODUCT || kWeights) && lane == 0) n_kept[sidx] = n_out;

        if (PASS == PASS_PRODUCT) {
            seg_T[sidx * 32 + lane] = (float)exp2(-log_sum);   // this segment's product
            continue;
        }
        const int64_t n_px = (int64_t)width * height;
        const int64_t pi = (int64_t)py * width + px;
        float* image_s = image + (int64_t)set * 4 * n_px;
        float* alpha_s = alpha_image + (int64_t)set * n_px;
        if (n_seg == 1u) {
            if (inside) {
                image_s[pi] = C0;
                image_s[n_px + pi] = C1;
                image_s[2 * n_px + pi] = C2;
                image_s[3 * n_px + pi] = C3;
                if (KIND == BLEND_INFER) {
                    const float A = 1.0f - Tr;
                    depth_image[(int64_t)set * n_px + pi] = A > 0.0f ? Z / A : 0.0f;
                    alpha_s[pi] = Tr < kTransmittanceEps ? 1.0f : A;
                } else {
                    alpha_s[pi] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
                }
            }
        } else {
            // partial colour of this segment; the per-tile combine adds the segments up in order
            const size_t si = sidx * 32 + lane;
            seg_C[si] = make_float4(C0, C1, C2, C3);
            if (PASS == PASS_FIRST) seg_T[si] = Tr;   // the exact state behind segment 0
            if (KIND == BLEND_INFER) {
                seg_Z[si] = Z;
                seg_E[si] = Tr;
            } else if (seg + 1u == n_seg && inside) {
                alpha_s[pi] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
            }
        }
    }
}

// Per tile half with several segments, between the PRODUCT and REST passes: seg_T of segment s >= 1 becomes
// the transmittance at its start = (state behind segment 0) * product of the segments 1 .. s-1.
__global__ void __launch_bounds__(kWarpBlendWarps * 32) warp_blend_prefix_kernel(const WarpItem* __restrict__ items0, const uint32_t* __restrict__ counts,
                                                                                 float* __restrict__ seg_T) {
    const unsigned lane = lane_id();
    const unsigned n_parts = __ldg(counts) * 2u;
    for (unsigned w = blockIdx.x * kWarpBlendWarps + (threadIdx.x >> 5); w < n_parts; w += gridDim.x * kWarpBlendWarps) {
        const WarpItem it = load_item(items0 + (w >> 1));
        const unsigned half = w & 1u;
        const unsigned n_seg = it.n_seg;
        if (n_seg == 1u) continue;
        const unsigned first = it.first;
        float* base = seg_T + ((size_t)first * 2u + half) * 32 + lane;   // segment g of this half: base[g * 64]
        float run = base[0];
        for (unsigned g0 = 1; g0 < n_seg; g0 += 8) {
            float product[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) product[k] = g0 + k + 1u < n_seg ? base[(size_t)(g0 + k) * 64] : 1.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (g0 + k < n_seg) base[(size_t)(g0 + k) * 64] = run;
                run *= product[k];
            }
        }
    }
}

// Per tile half with several segments, after the REST pass: image = sum of the segment colours in order.
// For training the running sum before each segment replaces the segment's own colour (the backward pass
// starts from it).  Inference: expected depth, and the transmittance where the pixel stopped = the end value
// of the first segment that fell below the threshold.
template <int KIND>
__global__ void __launch_bounds__(kWarpBlendWarps * 32) warp_blend_combine_kernel(
    const WarpItem* __restrict__ items0, const uint32_t* __restrict__ counts, float4* __restrict__ seg_C, const float* __restrict__ seg_Z,
    const float* __restrict__ seg_E,
    float* __restrict__ image, float* __restrict__ depth_image, float* __restrict__ alpha_image, int width, int height, int gw, int gh) {
    const unsigned lane = lane_id();
    const unsigned n_parts = __ldg(counts) * 2u;
    for (unsigned w = blockIdx.x * kWarpBlendWarps + (threadIdx.x >> 5); w < n_parts; w += gridDim.x * kWarpBlendWarps) {
        const WarpItem it = load_item(items0 + (w >> 1));
        const unsigned half = w & 1u;
        const unsigned tile = it.tile, n_seg = it.n_seg, first = it.first;
        if (n_seg == 1u) continue;
        const int tx = (int)(tile % (unsigned)gw), ty_all = (int)(tile / (unsigned)gw);
        const int set = ty_all / gh, ty = ty_all - set * gh;
        const int px = tx * 8 + (int)(lane & 7u);
        const int py = ty * 8 + 4 * (int)half + (int)(lane >> 3);
        const size_t base = ((size_t)first * 2u + half) * 32 + lane;   // segment g of this half: base + g * 64
        float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
        float z = 0.0f, t_final = 1.0f;
        bool stopped = false;
        for (unsigned g0 = 0; g0 < n_seg; g0 += 4) {
            float4 c[4];
            float zz[4], ee[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const bool ok = g0 + k < n_seg;
                const size_t si = base + (size_t)(g0 + k) * 64;
                c[k] = ok ? seg_C[si] : make_float4(0.f, 0.f, 0.f, 0.f);
                zz[k] = (KIND == BLEND_INFER && ok) ? seg_Z[si] : 0.0f;
                ee[k] = (KIND == BLEND_INFER && ok) ? seg_E[si] : 1.0f;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const bool ok = g0 + k < n_seg;
                if (KIND == BLEND_TRAIN && ok) seg_C[base + (size_t)(g0 + k) * 64] = run;
                run.x += c[k].x; run.y += c[k].y; run.z += c[k].z; run.w += c[k].w;
                z += zz[k];
                if (KIND == BLEND_INFER && ok && !stopped) { t_final = ee[k]; stopped = t_final < kTransmittanceEps; }
            }
        }
        if (px < width && py < height) {
            const int64_t n_px = (int64_t)width * height;
            const int64_t pi = (int64_t)py * width + px;
            float* image_s = image + (int64_t)set * 4 * n_px;
            image_s[pi] = run.x;
            image_s[n_px + pi] = run.y;
            image_s[2 * n_px + pi] = run.z;
            image_s[3 * n_px + pi] = run.w;
            if (KIND == BLEND_INFER) {
                const float A = 1.0f - t_final;
                depth_image[(int64_t)set * n_px + pi] = A > 0.0f ? z / A : 0.0f;
                alpha_image[(int64_t)set * n_px + pi] = t_final < kTransmittanceEps ? 1.0f : A;
            }
        }
    }
}

// Shared memory of one warp of the backward pass.
struct __align__(16) WarpBackwardSmem {
    float4 ring_a[kGatherDepthBackward][32];   // records of the batches in flight (see the forward pass): position, alpha ...
    float4 ring_f[kGatherDepthBackward][32];   // ... and features
    float4 pixel_grad[32];                  // image gradient of the half's pixels
    float4 frag_diff[kBatchFragments];      // per fragment: colour accumulated up to and including it, minus the final colour
    float2 frag[kBatchFragments];           // fragments in per-pixel order: alpha, lane of the staged instance
    float frag_seen[kBatchFragments];       // transmittance the fragment met (negative: it was dropped)
    float pixel_k[32];                      // grad_alpha * (1 - alpha) of the half's pixels
    uint32_t ring_id[kGatherDepthBackward][32];   // point ids of the batches in flight (0xFFFFFFFF: no instance)
    unsigned mask[32];
    unsigned off[32];
};
constexpr size_t kWarpBackwardSmemBytes = kWarpBlendWarps * sizeof(WarpBackwardSmem);

__global__ void __launch_bounds__(kWarpBlendWarps * 32, 3) blend_bilinear_warp_backward_kernel(
    const WarpItem* __restrict__ items0, const WarpItem* __restrict__ items1, const uint32_t* __restrict__ counts,
    unsigned* __restrict__ ticket, const uint32_t* __restrict__ kept0,
    const uint32_t* __restrict__ kept1, const uint32_t* __restrict__ n_kept, const PointRec* __restrict__ rec,
    const float* __restrict__ seg_T, const float4* __restrict__ seg_C, const float* __restrict__ grad_image,
    const float* __restrict__ grad_alpha, const float* __restrict__ image, const float* __restrict__ alpha_image,
    float4* __restrict__ slot_grad, unsigned* __restrict__ slot_mask, int width, int height, int gw) {
    constexpr unsigned kFull = 0xffffffffu;
    constexpr unsigned kNoInstance = 0xffffffffu;
    constexpr int kGatherDepth = kGatherDepthBackward;
    extern __shared__ __align__(16) unsigned char blend_smem[];
    const unsigned lane = lane_id();
    const unsigned lt_mask = (1u << lane) - 1u;
    WarpBackwardSmem& sm = reinterpret_cast<WarpBackwardSmem*>(blend_smem)[threadIdx.x >> 5];
    sm.mask[lane] = 0u;
    __syncwarp();
    const unsigned n_first = __ldg(counts) * 2u;
    const unsigned n_items = n_first + __ldg(counts + 1) * 2u;
    const unsigned n_rest = n_items - n_first;

    // items one at a time through a ticket counter, the later segments first (they belong to the longest lists)
    // (several consecutive ones per visit when there are very many, see the forward pass)
    const unsigned per_visit = max(1u, min(8u, n_items / (gridDim.x * kWarpBlendWarps * 8u)));
    unsigned next_item = 0, visit_end = 0;
    for (;;) {
        if (next_item == visit_end) {
            unsigned first_item = 0;
            if (lane == 0) first_item = atomicAdd(ticket, per_visit);
            first_item = __shfl_sync(kFull, first_item, 0);
            if (first_item >= n_items) break;
            next_item = first_item;
            visit_end = min(first_item + per_visit, n_items);
        }
        const unsigned item = next_item++;
        const WarpItem it = load_item(item < n_rest ? items1 + (item >> 1) : items0 + ((item - n_rest) >> 1));
        const int half = (int)((item < n_rest ? item : item - n_rest) & 1u);
        const unsigned n_list = __ldg(n_kept + (size_t)(it.first + it.seg) * 2u + half);
        const unsigned tile = it.tile, seg = it.seg, n_seg = it.n_seg;
        const size_t sidx = (size_t)(it.first + seg) * 2u + half;
        if (n_list == 0u) continue;
        const uint32_t* list = (half ? kept1 : kept0) + it.begin;
        const int tx = (int)(tile % (unsigned)gw), ty = (int)(tile / (unsigned)gw);
        const int px0 = tx * 8, py0 = ty * 8 + 4 * half;
        const int px = px0 + (int)(lane & 7u), py = py0 + (int)(lane >> 3);

        float4 g = make_float4(0.f, 0.f, 0.f, 0.f), Cfin = g, Crun = g;
        float K = 0.0f, Tr = 1.0f;
        bool done = !(px < width && py < height);
        if (!done) {
            const int64_t n_px = (int64_t)width * height;
            const int64_t pi = (int64_t)py * width + px;
            g = make_float4(__ldg(grad_image + pi), __ldg(grad_image + n_px + pi), __ldg(grad_image + 2 * n_px + pi),
                            __ldg(grad_image + 3 * n_px + pi));
            Cfin = make_float4(__ldg(image + pi), __ldg(image + n_px + pi), __ldg(image + 2 * n_px + pi),
                               __ldg(image + 3 * n_px + pi));
            K = __ldg(grad_alpha + pi) * (1.0f - __ldg(alpha_image + pi));
            if (seg > 0u) Tr = seg_T[sidx * 32 + lane];
            if (n_seg > 1u) Crun = seg_C[sidx * 32 + lane];
            done = Tr < kTransmittanceEps;
        }
        __syncwarp();   // the previous item's readers of pixel_grad are through
        sm.pixel_grad[lane] = g;
        sm.pixel_k[lane] = K;
        unsigned done_w = __ballot_sync(kFull, done);

        // ids kIdsAhead batches ahead of their gather, records kGatherDepth - 1 batches ahead of their use
        uint32_t idf[kIdsAhead];
#pragma unroll
        for (int k = 0; k < kIdsAhead; ++k) idf[k] = 32u * k + lane < n_list ? __ldg(list + 32u * k + lane) : 0u;
        unsigned issued = 0;   // instances whose gather has started
        auto gather = [&](unsigned stage) {
            const unsigned n = min(32u, n_list - issued);
            uint32_t id = kNoInstance;
            if (lane < n) {
                id = checked_point(idf[0]);
                const float4* p = reinterpret_cast<const float4*>(rec + id);
                async_copy_16(&sm.ring_a[stage][lane], p);
                async_copy_16(&sm.ring_f[stage][lane], p + 1);
            }
            sm.ring_id[stage][lane] = id;
            async_copy_commit();   // one group per batch, empty or not
#pragma unroll
            for (int k = 0; k + 1 < kIdsAhead; ++k) idf[k] = idf[k + 1];
            const unsigned nxt = issued + 32u * kIdsAhead + lane;
            idf[kIdsAhead - 1] = nxt < n_list ? __ldg(list + nxt) : 0u;
            issued += n;
        };
#pragma unroll
        for (int st = 0; st + 1 < kGatherDepth; ++st) gather((unsigned)st);
        for (unsigned batch = 0;; ++batch) {
            gather((batch + kGatherDepth - 1) & (kGatherDepth - 1));
            async_copy_wait<kGatherDepth - 1>();
            const unsigned stage = batch & (kGatherDepth - 1);
            const uint32_t id_cur = sm.ring_id[stage][lane];
            const bool staged = id_cur != kNoInstance;
            if (__ballot_sync(kFull, staged) == 0u) break;
            const float4 a_cur = sm.ring_a[stage][lane];
            // ---- lane j: the fragments of staged instance j
            const int qx = __float2int_rd(a_cur.x - 0.5f) - px0;
            const int qy = __float2int_rd(a_cur.y - 0.5f) - py0;
            float al[4], wg[4];
            int pix[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int cx = qx + (c & 1), cy = qy + (c >> 1);
                const float pcx = (float)(px0 + cx) + 0.5f, pcy = (float)(py0 + cy) + 0.5f;
                const float dx = fabsf(a_cur.x - pcx), dy = fabsf(a_cur.y - pcy);
                wg[c] = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                al[c] = a_cur.z * wg[c];
                const int p = cy * 8 + cx;
                const bool ok = staged && cx >= 0 && cx < 8 && cy >= 0 && cy < 4 && dx < 1.0f && dy < 1.0f &&
                                !((done_w >> (p & 31)) & 1u);
                pix[c] = ok ? p : -1;
                if (ok) atomicOr(sm.mask + p, 1u << lane);
            }
            __syncwarp();
            const unsigned my_mask = sm.mask[lane];
            const unsigned cnt = __popc(my_mask);
            const unsigned off = warp_inclusive_scan(cnt) - cnt;
            sm.off[lane] = off;
            __syncwarp();
            int slot[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                slot[c] = 0;
                if (pix[c] >= 0) {
                    slot[c] = (int)(sm.off[pix[c]] + __popc(sm.mask[pix[c]] & lt_mask));
                    sm.frag[slot[c]] = make_float2(al[c], __uint_as_float(lane));
                }
            }
            __syncwarp();
            if (my_mask) sm.mask[lane] = 0u;
            // The serial part, per pixel: only what one fragment hands to the next (transmittance, running colour) is
            // computed here, where the lanes with short lists idle; each fragment's state is left in shared memory
            // and the gradient arithmetic follows below, per instance, with every staged lane busy.  Branch-free
            // steps in chunks whose loads are issued together (see the forward pass).
            constexpr int kChunk = 4;
            for (unsigned k0 = off; k0 < off + cnt; k0 += kChunk) {
                float a[kChunk];
                float4 f[kChunk];
#pragma unroll
                for (int u = 0; u < kChunk; ++u) {
                    const unsigned k = min(k0 + u, off + cnt - 1u);
                    const float2 e = sm.frag[k];
                    a[u] = e.x;
                    f[u] = sm.ring_f[stage][__float_as_uint(e.y)];
                }
#pragma unroll
                for (int u = 0; u < kChunk; ++u) {
                    const bool in_list = k0 + u < off + cnt;
                    const bool live = !done && in_list;
                    const float bw = Tr * a[u];
                    const float4 cr = make_float4(Crun.x + bw * f[u].x, Crun.y + bw * f[u].y, Crun.z + bw * f[u].z, Crun.w + bw * f[u].w);
                    if (in_list) {
                        sm.frag_seen[k0 + u] = live ? Tr : -1.0f;
                        sm.frag_diff[k0 + u] = make_float4(cr.x - Cfin.x, cr.y - Cfin.y, cr.z - Cfin.z, cr.w - Cfin.w);
                    }
                    Crun = live ? cr : Crun;
                    Tr = live ? Tr * (1.0f - a[u]) : Tr;
                    done = done || Tr < kTransmittanceEps;
                }
            }
            __syncwarp();
            // gradients of every staged instance: its (up to) four fragments in fixed corner order
            if (staged) {
                const float4 fo = sm.ring_f[stage][lane];
                float4 sf = make_float4(0.f, 0.f, 0.f, 0.f);
                float so = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    float o = 0.0f;
                    if (pix[c] >= 0) {
                        const float seen = sm.frag_seen[slot[c]];
                        if (seen >= 0.0f) {
                            const float4 d = sm.frag_diff[slot[c]];
                            const float4 pg = sm.pixel_grad[pix[c]];
                            const float rcp = 1.0f / fmaxf(1.0f - al[c], kOneMinusAlphaEps);
                            const float bw = seen * al[c];
                            const float from_features = (seen * fo.x + d.x * rcp) * pg.x + (seen * fo.y + d.y * rcp) * pg.y +
                                                        (seen * fo.z + d.z * rcp) * pg.z + (seen * fo.w + d.w * rcp) * pg.w;
                            o = (from_features + sm.pixel_k[pix[c]] * rcp) * wg[c];
                            if (bw > 0.0f) v = make_float4(bw * pg.x, bw * pg.y, bw * pg.z, bw * pg.w);
                        }
                    }
                    if (c == 0) { sf = v; so = o; }
                    else { sf.x += v.x; sf.y += v.y; sf.z += v.z; sf.w += v.w; so += o; }
                }
                // A splat's 2x2 pixels lie in at most two tile columns and two (tile row, half) groups, and which of
                // them this item is follows from where the footprint starts: it holds the left column unless the
                // footprint starts left of it, and the upper row unless it starts above it.  So every (point, slot)
                // has exactly one writer in the whole launch: the sums go there with plain stores, a bit marks the
                // slot as written, and the per-point pass adds the slots in fixed order -- no floating-point
                // atomics, the same gradient bits on every run.
                if (sf.x != 0.0f || sf.y != 0.0f || sf.z != 0.0f || sf.w != 0.0f || so != 0.0f) {
                    const unsigned slot_of_point = (qx < 0 ? 1u : 0u) + (qy < 0 ? 2u : 0u);
                    // one aligned 32-byte record per slot: a whole memory sector, written without reading it first
                    float4* e = slot_grad + ((size_t)id_cur * 4u + slot_of_point) * 2u;
                    e[0] = sf;
                    e[1] = make_float4(so, 0.0f, 0.0f, 0.0f);
                    atomicOr(slot_mask + id_cur, 1u << slot_of_point);
                }
            }
            done_w = __ballot_sync(kFull, done);
            __syncwarp();
            if (done_w == kFull) break;
        }
        async_copy_wait<0>();   // whatever is still travelling lands before the next item reuses the ring
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------------
// Bilinear blend over feature rows: every point carries C = 4 * C4 fp32 channels in the caller's
// (n, C) array and they are blended as they are, into a (C, H, W) image.  The walk, the stopping
// rule and the segment composition are those of the kernels above (src/bilinear/kernels.cu:241-420
// with the channel count as a parameter); the reference itself only has the 36-half -> 4-channel
// layout.  The transmittance pre-pass and the per-tile prefix do not look at features and are
// shared.  One instance per pixel thread and batch.
// ------------------------------------------------------------------------------------------------
template <int T, int C4>
constexpr size_t rows_forward_smem_bytes() {
    return (size_t)T * T * (16 + 16 * C4 + 4 * 4) + (size_t)(T * T / 32) * T * T * 4;
}

template <int T, int C4, int KIND>
__global__ void __launch_bounds__(T * T) blend_rows_forward_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, const float4* __restrict__ features, float* __restrict__ seg_T,
    float4* __restrict__ seg_C, float* __restrict__ seg_Z, float* __restrict__ image, float* __restrict__ depth_image,
    float* __restrict__ alpha_image, float* __restrict__ blending_weights, int width, int height, int gw) {
    constexpr int P = T * T;
    constexpr int WORDS = P / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu, n_seg = sg.info >> 16;

    extern __shared__ __align__(16) unsigned char blend_smem[];
    float4* s_a = reinterpret_cast<float4*>(blend_smem);                        // [P]
    float4* s_f = s_a + P;                                                      // [C4][P]
    float* s_slot = reinterpret_cast<float*>(s_f + C4 * P);                     // [4][P] blending weight per footprint corner
    unsigned (*s_mask)[P] = reinterpret_cast<unsigned (*)[P]>(s_slot + 4 * P);  // [WORDS][P]

    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
    const size_t state_idx = (size_t)blockIdx.x * P + t;

#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
#pragma unroll
    for (int q = 0; q < 4; ++q) s_slot[q * P + t] = 0.0f;
    float4 acc[C4];
#pragma unroll
    for (int c = 0; c < C4; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    float Z = 0.0f, Tr = 1.0f;
    if (seg_idx > 0u && inside) Tr = seg_T[state_idx];
    bool done = !inside || Tr < kTransmittanceEps;
    __syncthreads();

    uint32_t id = 0;
    int cnt = 0;
    auto flush_weights = [&]() {
        if (t < cnt) {
            const float sum = ((s_slot[t] + s_slot[P + t]) + s_slot[2 * P + t]) + s_slot[3 * P + t];
            if (sum > 0.0f) atomicAdd(blending_weights + id, sum);
            s_slot[t] = 0.0f; s_slot[P + t] = 0.0f; s_slot[2 * P + t] = 0.0f; s_slot[3 * P + t] = 0.0f;
        }
    };
    for (unsigned base = sg.begin; base < sg.end; base += P) {
        if (KIND == BLEND_TRAIN) flush_weights();
        cnt = (int)min((unsigned)P, sg.end - base);
        id = stage_instance<T, P, false>(t, cnt, base, inst_ids, rec, tx, ty, s_a, nullptr, s_mask);
        if (t < cnt) {
            const float4* row = features + (size_t)id * C4;
#pragma unroll
            for (int c = 0; c < C4; ++c) s_f[c * P + t] = __ldg(row + c);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float dx = fabsf(a.x - pcx), dy = fabsf(a.y - pcy);
                if (dx >= 1.0f || dy >= 1.0f) continue;
                const float wgt = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                const float al = a.z * wgt;
                const float bw = Tr * al;
                if (KIND == BLEND_TRAIN) {
                    if (bw > 0.0f) s_slot[((pcx > a.x ? 1 : 0) + (pcy > a.y ? 2 : 0)) * P + j] = bw * wgt;
                }
#pragma unroll
                for (int c = 0; c < C4; ++c) {
                    const float4 f = s_f[c * P + j];
                    acc[c].x += bw * f.x; acc[c].y += bw * f.y; acc[c].z += bw * f.z; acc[c].w += bw * f.w;
                }
                if (KIND == BLEND_INFER) Z += bw * a.w;
                Tr *= 1.0f - al;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
        if (__syncthreads_count(done) == P) break;
    }
    if (KIND == BLEND_TRAIN) flush_weights();

    if (n_seg == 1u) {
        if (inside) {
            const int64_t n_px = (int64_t)width * height;
            const int64_t pi = (int64_t)py * width + px;
#pragma unroll
            for (int c = 0; c < C4; ++c) {
                image[(4 * c) * n_px + pi] = acc[c].x;
                image[(4 * c + 1) * n_px + pi] = acc[c].y;
                image[(4 * c + 2) * n_px + pi] = acc[c].z;
                image[(4 * c + 3) * n_px + pi] = acc[c].w;
            }
            if (KIND == BLEND_INFER) {
                const float A = 1.0f - Tr;
                depth_image[pi] = A > 0.0f ? Z / A : 0.0f;
                alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : A;
            } else {
                alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < C4; ++c) seg_C[((size_t)blockIdx.x * C4 + c) * P + t] = acc[c];
        if (KIND == BLEND_INFER) {
            seg_Z[state_idx] = Z;
            seg_T[state_idx] = Tr;
        } else if (seg_idx == n_seg - 1u && inside) {
            alpha_image[(int64_t)py * width + px] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
        }
    }
}

// Per tile with several segments, feature-row layout: image = sum of the segment colours in order;
// for training the running sum before each segment replaces the segment's own colour.
template <int T, int C4, int KIND>
__global__ void __launch_bounds__(T * T) blend_rows_combine_kernel(const Segment* __restrict__ segs, const uint32_t* __restrict__ tile_first,
                                                                   float4* __restrict__ seg_C, const float* __restrict__ seg_Z,
                                                                   const float* __restrict__ seg_T, float* __restrict__ image,
                                                                   float* __restrict__ depth_image, float* __restrict__ alpha_image,
                                                                   int width, int height, int gw) {
    constexpr int P = T * T;
    const unsigned first = tile_first[blockIdx.x];
    const unsigned n_seg = segs[first].info >> 16;
    if (n_seg == 1u) return;
    const int t = threadIdx.x;
    const int tx = (int)(blockIdx.x % (unsigned)gw), ty = (int)(blockIdx.x / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const int64_t n_px = (int64_t)width * height;
    const int64_t pi = (int64_t)py * width + px;
#pragma unroll 1
    for (int c = 0; c < C4; ++c) {
        float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
        for (unsigned s = 0; s < n_seg; ++s) {
            float4* slot = seg_C + ((size_t)(first + s) * C4 + c) * P + t;
            const float4 v = *slot;
            if (KIND == BLEND_TRAIN) *slot = run;
            run.x += v.x; run.y += v.y; run.z += v.z; run.w += v.w;
        }
        if (inside) {
            image[(4 * c) * n_px + pi] = run.x;
            image[(4 * c + 1) * n_px + pi] = run.y;
            image[(4 * c + 2) * n_px + pi] = run.z;
            image[(4 * c + 3) * n_px + pi] = run.w;
        }
    }
    if (KIND == BLEND_INFER) {
        float z = 0.0f, t_final = 1.0f;
        bool stopped = false;
        for (unsigned s = 0; s < n_seg; ++s) {
            z += seg_Z[(size_t)(first + s) * P + t];
            if (!stopped) {
                t_final = seg_T[(size_t)(first + s) * P + t];
                stopped = t_final < kTransmittanceEps;
            }
        }
        if (inside) {
            const float A = 1.0f - t_final;
            depth_image[pi] = A > 0.0f ? z / A : 0.0f;
            alpha_image[pi] = t_final < kTransmittanceEps ? 1.0f : A;
        }
    }
}

template <int T, int C4>
constexpr size_t rows_backward_smem_bytes() {
    return (size_t)T * T * (16 + 16 * C4 + 16 * C4 + 4 * 4 + 4 * 4) + (size_t)(T * T / 32) * T * T * 4;
}

// Backward over feature rows.  Per fragment only scalars are kept: with G = <g, .> over the channels,
// dL/dalpha = Tr * G(f) + (G(C_run) - G(C_final)) / (1 - alpha) + K / (1 - alpha), and G(C_run) is a
// running scalar.  The blending weight of each (instance, footprint corner) goes to a shared-memory
// slot; the thread that staged the instance then forms sum_corner bw * g(pixel of that corner) from
// the tile's pixel gradients in shared memory and issues one vector atomic per four channels.
template <int T, int C4>
__global__ void __launch_bounds__(T * T) blend_rows_backward_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, const float4* __restrict__ features, const float* __restrict__ seg_T,
    const float4* __restrict__ seg_C, const float* __restrict__ grad_image, const float* __restrict__ grad_alpha,
    const float* __restrict__ image, const float* __restrict__ alpha_image, float4* __restrict__ grad_features,
    float* __restrict__ grad_opacity, int width, int height, int gw) {
    constexpr int P = T * T;
    constexpr int WORDS = P / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu;
    if (sg.begin == sg.end) return;

    extern __shared__ __align__(16) unsigned char blend_smem[];
    float4* s_a = reinterpret_cast<float4*>(blend_smem);                      // [P]
    float4* s_f = s_a + P;                                                    // [C4][P] staged feature rows
    float4* s_g = s_f + C4 * P;                                               // [C4][P] image gradient of the tile's pixels
    float* s_bw = reinterpret_cast<float*>(s_g + C4 * P);                     // [4][P]
    float* s_go = s_bw + 4 * P;                                               // [4][P]
    unsigned (*s_mask)[P] = reinterpret_cast<unsigned (*)[P]>(s_go + 4 * P);  // [WORDS][P]

    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
    const size_t state_idx = (size_t)blockIdx.x * P + t;

#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
#pragma unroll
    for (int q = 0; q < 4; ++q) { s_bw[q * P + t] = 0.0f; s_go[q * P + t] = 0.0f; }

    float4 g[C4];
    float G_final = 0.0f, G_run = 0.0f, K = 0.0f, Tr = 1.0f;
#pragma unroll
    for (int c = 0; c < C4; ++c) g[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (inside) {
        const int64_t n_px = (int64_t)width * height;
        const int64_t pi = (int64_t)py * width + px;
#pragma unroll
        for (int c = 0; c < C4; ++c) {
            g[c] = make_float4(__ldg(grad_image + (4 * c) * n_px + pi), __ldg(grad_image + (4 * c + 1) * n_px + pi),
                               __ldg(grad_image + (4 * c + 2) * n_px + pi), __ldg(grad_image + (4 * c + 3) * n_px + pi));
            G_final += __ldg(image + (4 * c) * n_px + pi) * g[c].x + __ldg(image + (4 * c + 1) * n_px + pi) * g[c].y +
                       __ldg(image + (4 * c + 2) * n_px + pi) * g[c].z + __ldg(image + (4 * c + 3) * n_px + pi) * g[c].w;
        }
        K = __ldg(grad_alpha + pi) * (1.0f - __ldg(alpha_image + pi));
        if (seg_idx > 0u) {
            Tr = seg_T[state_idx];
#pragma unroll
            for (int c = 0; c < C4; ++c) {
                const float4 v = seg_C[((size_t)blockIdx.x * C4 + c) * P + t];
                G_run += v.x * g[c].x + v.y * g[c].y + v.z * g[c].z + v.w * g[c].w;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < C4; ++c) s_g[c * P + t] = g[c];
    bool done = !inside || Tr < kTransmittanceEps;
    __syncthreads();

    uint32_t id = 0;
    int cnt = 0;
    auto flush_gradients = [&]() {
        if (t < cnt) {
            const float4 a = s_a[t];
            const int qx = __float2int_rd(a.x - 0.5f) - tx * T;
            const int qy = __float2int_rd(a.y - 0.5f) - ty * T;
            float bw[4];
            float so = 0.0f;
            bool any = false;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                bw[q] = s_bw[q * P + t];
                so += s_go[q * P + t];
                any = any || bw[q] != 0.0f;
                s_bw[q * P + t] = 0.0f;
                s_go[q * P + t] = 0.0f;
            }
            if (any) {
                // a corner slot is only ever written by the pixel thread of that corner, so a filled
                // slot names a pixel of this tile
                float4* dst = grad_features + (size_t)id * C4;
#pragma unroll
                for (int c = 0; c < C4; ++c) {
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (bw[q] != 0.0f) {
                            const float4 v = s_g[c * P + (qy + (q >> 1)) * T + qx + (q & 1)];
                            sum.x += bw[q] * v.x; sum.y += bw[q] * v.y; sum.z += bw[q] * v.z; sum.w += bw[q] * v.w;
                        }
                    }
                    if (sum.x != 0.0f || sum.y != 0.0f || sum.z != 0.0f || sum.w != 0.0f) atomicAdd(dst + c, sum);
                }
            }
            if (so != 0.0f) atomicAdd(grad_opacity + id, so);
        }
    };
    for (unsigned base = sg.begin; base < sg.end; base += P) {
        flush_gradients();
        cnt = (int)min((unsigned)P, sg.end - base);
        id = stage_instance<T, P, false>(t, cnt, base, inst_ids, rec, tx, ty, s_a, nullptr, s_mask);
        if (t < cnt) {
            const float4* row = features + (size_t)id * C4;
#pragma unroll
            for (int c = 0; c < C4; ++c) s_f[c * P + t] = __ldg(row + c);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float dx = fabsf(a.x - pcx), dy = fabsf(a.y - pcy);
                if (dx >= 1.0f || dy >= 1.0f) continue;
                const float wgt = __saturatef(1.0f - dx) * __saturatef(1.0f - dy);
                const float al = a.z * wgt;
                const float bw = Tr * al;
                const int q = (pcx > a.x ? 1 : 0) + (pcy > a.y ? 2 : 0);
                if (bw > 0.0f) s_bw[q * P + j] = bw;
                float fg = 0.0f;
#pragma unroll
                for (int c = 0; c < C4; ++c) {
                    const float4 f = s_f[c * P + j];
                    fg += f.x * g[c].x + f.y * g[c].y + f.z * g[c].z + f.w * g[c].w;
                }
                G_run += bw * fg;
                const float oma = 1.0f - al;
                const float rcp = 1.0f / fmaxf(oma, kOneMinusAlphaEps);
                const float dalpha = Tr * fg + (G_run - G_final) * rcp + K * rcp;
                const float dop = dalpha * wgt;
                if (dop != 0.0f) s_go[q * P + j] = dop;
                Tr *= oma;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
        if (__syncthreads_count(done) == P) break;
    }
    flush_gradients();
}

// ------------------------------------------------------------------------------------------------
// Gaussian blend (src/gaussian/kernels.cu:401-474 forward, :476-579 backward, :581-660 inference).
// A footprint is an ellipse of a few pixels, not a fixed 2x2: the staging thread sets its instance's bit
// for the pixels of the ellipse's bounding box inside the tile (slightly widened, so a superset of the
// pixels that pass the reference's tests), and every pixel thread walks only its set bits and applies
// the reference's tests and arithmetic unchanged.  Per-point sums (blending weight, gradients) are
// accumulated with shared-memory atomics per staged instance and leave with one global atomic per
// instance (the reference issues global atomics per fragment).
// ------------------------------------------------------------------------------------------------
template <int T>
__device__ __forceinline__ void gaussian_mask_bits(int j, const float4& a, const float4& c, float neg_log_threshold, int tile_x, int tile_y,
                                                   unsigned (*s_mask)[T * T]) {
    // points with  -0.5 d^T Conic d >= -L  lie within |dx| <= sqrt(2 L cov_xx), |dy| <= sqrt(2 L cov_yy),
    // cov = Conic^-1
    const float det = c.x * c.z - c.y * c.y;
    int x0 = 0, x1 = T - 1, y0 = 0, y1 = T - 1;
    if (det > 0.0f) {
        const float s = 2.0f * neg_log_threshold / det;
        const float rx = sqrtf(fmaxf(s * c.z, 0.0f)) * 1.001f + 0.01f;
        const float ry = sqrtf(fmaxf(s * c.x, 0.0f)) * 1.001f + 0.01f;
        x0 = max(0, __float2int_ru(a.x - rx - 0.5f) - tile_x * T);
        x1 = min(T - 1, __float2int_rd(a.x + rx - 0.5f) - tile_x * T);
        y0 = max(0, __float2int_ru(a.y - ry - 0.5f) - tile_y * T);
        y1 = min(T - 1, __float2int_rd(a.y + ry - 0.5f) - tile_y * T);
    }
    const unsigned bit = 1u << (j & 31);
    unsigned* mrow = s_mask[j >> 5];
    for (int y = y0; y <= y1; ++y)
        for (int x = x0; x <= x1; ++x) atomicOr(mrow + y * T + x, bit);
}

// Pass 1 of the segmented gaussian blend (tiles with several segments only): per-pixel product of
// (1 - alpha) over one segment; FAST selects the exponential of the inference kernels.
template <int T, bool FAST>
__global__ void __launch_bounds__(T * T) blend_gaussian_transmittance_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, const float4* __restrict__ conic, float* __restrict__ seg_T, int width, int height, int gw,
    float threshold, float neg_log_threshold) {
    constexpr int B = T * T;
    constexpr int WORDS = B / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu, n_seg = sg.info >> 16;
    if (n_seg == 1u || seg_idx == n_seg - 1u) return;
    __shared__ float4 s_a[B];
    __shared__ float4 s_c[B];
    __shared__ unsigned s_mask[WORDS][B];
    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
    float Tr = 1.0f;
    bool done = !(px < width && py < height);
    for (unsigned base = sg.begin; base < sg.end; base += B) {
        if (__syncthreads_count(done) == B) break;
        const int cnt = (int)min((unsigned)B, sg.end - base);
        if (t < cnt) {
            const uint32_t id = checked_point(__ldg(inst_ids + base + t));
            const float4 a = __ldg(reinterpret_cast<const float4*>(rec + id));
            const float4 c = __ldg(conic + id);
            s_a[t] = a;
            s_c[t] = c;
            gaussian_mask_bits<T>(t, a, c, neg_log_threshold, tx, ty, s_mask);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float4 c = s_c[j];
                const float dx = a.x - pcx, dy = a.y - pcy;
                const float e = -0.5f * (c.x * dx * dx + c.z * dy * dy) - c.y * dx * dy;
                if (e > 0.0f) continue;
                const float G = FAST ? __expf(e) : expf(e);
                if (G < threshold) continue;
                Tr *= 1.0f - a.z * G;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
    }
    seg_T[(size_t)blockIdx.x * B + t] = Tr;
}

// Main pass: one block per (tile, segment), starting from the segment's incoming transmittance.
template <int T, int KIND>
__global__ void __launch_bounds__(T * T) blend_gaussian_forward_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, const float4* __restrict__ conic, float* __restrict__ seg_T, float4* __restrict__ seg_C,
    float* __restrict__ seg_Z, float* __restrict__ image, float* __restrict__ depth_image,
    float* __restrict__ alpha_image, float* __restrict__ blending_weights, int width, int height, int gw,
    float threshold, float neg_log_threshold) {
    constexpr int B = T * T;
    constexpr int WORDS = B / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu, n_seg = sg.info >> 16;
    __shared__ float4 s_a[B];
    __shared__ float4 s_f[B];
    __shared__ float4 s_c[B];
    __shared__ uint32_t s_id[B];
    __shared__ unsigned s_mask[WORDS][B];
    __shared__ float s_bw[KIND == BLEND_TRAIN ? B : 1];
    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
    const size_t state_idx = (size_t)blockIdx.x * B + t;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
    if (KIND == BLEND_TRAIN) s_bw[t] = 0.0f;
    float C0 = 0.f, C1 = 0.f, C2 = 0.f, C3 = 0.f, Z = 0.f, Tr = 1.0f;
    if (seg_idx > 0u && inside) Tr = seg_T[state_idx];
    bool done = !inside || Tr < kTransmittanceEps;
    int cnt = 0;
    auto flush_weights = [&]() {
        if (t < cnt) {
            const float sum = s_bw[t];
            if (sum > 0.0f) atomicAdd(blending_weights + s_id[t], sum);
            s_bw[t] = 0.0f;
        }
    };
    for (unsigned base = sg.begin; base < sg.end; base += B) {
        if (__syncthreads_count(done) == B) break;     // also: every thread has finished the batch before
        if (KIND == BLEND_TRAIN) flush_weights();
        cnt = (int)min((unsigned)B, sg.end - base);
        if (t < cnt) {
            const uint32_t id = checked_point(__ldg(inst_ids + base + t));
            const float4* r = reinterpret_cast<const float4*>(rec + id);
            const float4 a = __ldg(r);
            const float4 c = __ldg(conic + id);
            s_a[t] = a;
            s_f[t] = __ldg(r + 1);
            s_c[t] = c;
            s_id[t] = id;
            gaussian_mask_bits<T>(t, a, c, neg_log_threshold, tx, ty, s_mask);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float4 c = s_c[j];
                const float dx = a.x - pcx, dy = a.y - pcy;
                const float e = -0.5f * (c.x * dx * dx + c.z * dy * dy) - c.y * dx * dy;
                if (e > 0.0f) continue;
                const float G = KIND == BLEND_INFER ? __expf(e) : expf(e);
                if (G < threshold) continue;
                const float al = a.z * G;
                const float bw = Tr * al;
                if (KIND == BLEND_TRAIN) {
                    if (bw > 0.0f) atomicAdd(&s_bw[j], G * bw);
                }
                const float4 f = s_f[j];
                C0 += bw * f.x; C1 += bw * f.y; C2 += bw * f.z; C3 += bw * f.w;
                if (KIND == BLEND_INFER) Z += bw * a.w;
                Tr *= 1.0f - al;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
    }
    if (KIND == BLEND_TRAIN) {
        __syncthreads();
        flush_weights();
    }
    if (n_seg == 1u) {
        if (inside) {
            const int64_t n_px = (int64_t)width * height;
            const int64_t pi = (int64_t)py * width + px;
            image[pi] = C0;
            image[n_px + pi] = C1;
            image[2 * n_px + pi] = C2;
            image[3 * n_px + pi] = C3;
            if (KIND == BLEND_INFER) {
                const float A = 1.0f - Tr;
                depth_image[pi] = A > 0.0f ? Z / A : 0.0f;
                alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : A;
            } else {
                alpha_image[pi] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
            }
        }
    } else {
        seg_C[state_idx] = make_float4(C0, C1, C2, C3);
        if (KIND == BLEND_INFER) {
            seg_Z[state_idx] = Z;
            seg_T[state_idx] = Tr;
        } else if (seg_idx == n_seg - 1u && inside) {
            alpha_image[(int64_t)py * width + px] = Tr < kTransmittanceEps ? 1.0f : 1.0f - Tr;
        }
    }
}

template <int T>
__global__ void __launch_bounds__(T * T) blend_gaussian_backward_kernel(
    const Segment* __restrict__ segs, const uint32_t* __restrict__ n_segments, const uint32_t* __restrict__ inst_ids,
    const PointRec* __restrict__ rec, const float4* __restrict__ conic, const float* __restrict__ seg_T,
    const float4* __restrict__ seg_C, const float* __restrict__ grad_image, const float* __restrict__ grad_alpha,
    const float* __restrict__ image, const float* __restrict__ alpha_image, float4* __restrict__ grad_feat_view,
    float* __restrict__ grad_opacity, int width, int height, int gw) {
    constexpr int B = T * T;
    constexpr int WORDS = B / 32;
    if (blockIdx.x >= *n_segments) return;
    const Segment sg = segs[blockIdx.x];
    const unsigned seg_idx = sg.info & 0xffffu;
    if (sg.begin == sg.end) return;
    __shared__ float4 s_a[B];
    __shared__ float4 s_f[B];
    __shared__ float4 s_c[B];
    __shared__ uint32_t s_id[B];
    __shared__ unsigned s_mask[WORDS][B];
    __shared__ float s_gf[4][B];   // per staged instance: view-space feature gradient ...
    __shared__ float s_go[B];      // ... and opacity gradient, summed with shared-memory atomics
    const int t = threadIdx.x;
    const int tx = (int)(sg.tile % (unsigned)gw), ty = (int)(sg.tile / (unsigned)gw);
    const size_t state_idx = (size_t)blockIdx.x * B + t;
    const int px = tx * T + t % T, py = ty * T + t / T;
    const bool inside = px < width && py < height;
    const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_mask[w][t] = 0u;
#pragma unroll
    for (int q = 0; q < 4; ++q) s_gf[q][t] = 0.0f;
    s_go[t] = 0.0f;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), Cfin = make_float4(0.f, 0.f, 0.f, 0.f);
    float K = 0.0f;
    if (inside) {
        const int64_t n_px = (int64_t)width * height;
        const int64_t pi = (int64_t)py * width + px;
        g = make_float4(__ldg(grad_image + pi), __ldg(grad_image + n_px + pi), __ldg(grad_image + 2 * n_px + pi),
                        __ldg(grad_image + 3 * n_px + pi));
        Cfin = make_float4(__ldg(image + pi), __ldg(image + n_px + pi), __ldg(image + 2 * n_px + pi),
                           __ldg(image + 3 * n_px + pi));
        K = __ldg(grad_alpha + pi) * (1.0f - __ldg(alpha_image + pi));
    }
    float4 Crun = make_float4(0.f, 0.f, 0.f, 0.f);
    float Tr = 1.0f;
    if (inside && seg_idx > 0u) { Tr = seg_T[state_idx]; Crun = seg_C[state_idx]; }
    bool done = !inside || Tr < kTransmittanceEps;
    int cnt = 0;
    auto flush_gradients = [&]() {
        if (t < cnt) {
            const float4 sf = make_float4(s_gf[0][t], s_gf[1][t], s_gf[2][t], s_gf[3][t]);
            const float so = s_go[t];
            const uint32_t id = s_id[t];
            if (sf.x != 0.0f || sf.y != 0.0f || sf.z != 0.0f || sf.w != 0.0f) atomicAdd(grad_feat_view + id, sf);
            if (so != 0.0f) atomicAdd(grad_opacity + id, so);
            s_gf[0][t] = 0.0f; s_gf[1][t] = 0.0f; s_gf[2][t] = 0.0f; s_gf[3][t] = 0.0f;
            s_go[t] = 0.0f;
        }
    };
    constexpr float kNegLogThreshold = 4.5f;   // -ln(kTrainGaussThreshold)
    for (unsigned base = sg.begin; base < sg.end; base += B) {
        if (__syncthreads_count(done) == B) break;
        flush_gradients();
        cnt = (int)min((unsigned)B, sg.end - base);
        if (t < cnt) {
            const uint32_t id = checked_point(__ldg(inst_ids + base + t));
            const float4* r = reinterpret_cast<const float4*>(rec + id);
            const float4 a = __ldg(r);
            const float4 c = __ldg(conic + id);
            s_a[t] = a;
            s_f[t] = __ldg(r + 1);
            s_c[t] = c;
            s_id[t] = id;
            gaussian_mask_bits<T>(t, a, c, kNegLogThreshold, tx, ty, s_mask);
        }
        __syncthreads();
#pragma unroll 1
        for (int w = 0; w < WORDS; ++w) {
            unsigned mbits = s_mask[w][t];
            if (mbits) s_mask[w][t] = 0u;
            while (mbits && !done) {
                const int j = w * 32 + __ffs(mbits) - 1;
                mbits &= mbits - 1u;
                const float4 a = s_a[j];
                const float4 c = s_c[j];
                const float dx = a.x - pcx, dy = a.y - pcy;
                const float e = -0.5f * (c.x * dx * dx + c.z * dy * dy) - c.y * dx * dy;
                if (e > 0.0f) continue;
                const float G = expf(e);
                if (G < kTrainGaussThreshold) continue;
                const float al = a.z * G;
                const float bw = Tr * al;
                if (bw > 0.0f) {
                    atomicAdd(&s_gf[0][j], bw * g.x); atomicAdd(&s_gf[1][j], bw * g.y);
                    atomicAdd(&s_gf[2][j], bw * g.z); atomicAdd(&s_gf[3][j], bw * g.w);
                }
                const float4 f = s_f[j];
                Crun.x += bw * f.x; Crun.y += bw * f.y; Crun.z += bw * f.z; Crun.w += bw * f.w;
                const float oma = 1.0f - al;
                const float rcp = 1.0f / fmaxf(oma, kOneMinusAlphaEps);
                const float from_features = (Tr * f.x + (Crun.x - Cfin.x) * rcp) * g.x +
                                            (Tr * f.y + (Crun.y - Cfin.y) * rcp) * g.y +
                                            (Tr * f.z + (Crun.z - Cfin.z) * rcp) * g.z +
                                            (Tr * f.w + (Crun.w - Cfin.w) * rcp) * g.w;
                const float dalpha = from_features + K * rcp;
                const float dop = dalpha * G;
                if (dop != 0.0f) atomicAdd(&s_go[j], dop);
                Tr *= oma;
                if (Tr < kTransmittanceEps) done = true;
            }
        }
    }
    __syncthreads();
    flush_gradients();
}

// SH chain rule for every point, zero rows for culled ones, written as 72 contiguous bytes per point
// through a shared-memory slab so the stores are coalesced 16-byte vectors.
// src/bilinear/kernels.cu:86-104 + include/sh_utils.cuh:44-62; the zero rows replace the
// torch::zeros of src/rasterization_api.cu:139.
// SLOTS (warp blend): the view-space gradient of a point is the sum of its (up to four) written slots in slot order,
// see blend_bilinear_warp_backward_kernel; the opacity gradient is formed here too and written for every point.
struct GradientSlots {
    const float4* grad;      // [4 n][2]: {feature gradient}, {opacity gradient, -, -, -}
    const unsigned* mask;    // [n] bit s: slot s was written
};
template <bool SLOTS>
__global__ void __launch_bounds__(kPreThreads) preprocess_backward_kernel(
    const float* __restrict__ positions, const float* __restrict__ cam, const uint2* __restrict__ bounds,
    const float4* __restrict__ grad_feat_view, GradientSlots slots, float* __restrict__ grad_opacities,
    __half* __restrict__ grad_features, int64_t n, bool bulk_ok) {
    __shared__ __align__(16) __half s_out[kPreThreads * 36];
    const int64_t block_first = (int64_t)blockIdx.x * kPreThreads;
    const int in_block = (int)min((int64_t)kPreThreads, n - block_first);
    const int64_t i = block_first + threadIdx.x;
    __half* o = s_out + threadIdx.x * 36;
    bool touched = false;
    if (i < n) touched = tiles_of(__ldg(bounds + i)) != 0u;
    if (touched) {
        float b[9];
        sh_basis(__ldg(positions + 3 * i), __ldg(positions + 3 * i + 1), __ldg(positions + 3 * i + 2), cam, b);
        b[1] = -b[1]; b[3] = -b[3]; b[5] = -b[5]; b[7] = -b[7];
        float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (SLOTS) {
            float go = 0.0f;
            const unsigned m = __ldg(slots.mask + i);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if ((m >> q) & 1u) {
                    const float4 v = __ldg(slots.grad + (i * 4 + q) * 2);
                    gv.x += v.x; gv.y += v.y; gv.z += v.z; gv.w += v.w;
                    go += __ldg(slots.grad + (i * 4 + q) * 2 + 1).x;
                }
            }
            grad_opacities[i] = go;
        } else {
            gv = __ldg(grad_feat_view + i);
        }
#pragma unroll
        for (int k = 0; k < 9; ++k) {
            const __half2 xy = __float22half2_rn(make_float2(b[k] * gv.x, b[k] * gv.y));
            const __half2 zw = __float22half2_rn(make_float2(b[k] * gv.z, b[k] * gv.w));
            *reinterpret_cast<__half2*>(o + 4 * k) = xy;
            *reinterpret_cast<__half2*>(o + 4 * k + 2) = zw;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 18; ++k) *reinterpret_cast<unsigned*>(o + 2 * k) = 0u;
        if (SLOTS && i < n) grad_opacities[i] = 0.0f;
    }
    unsigned char* dst = reinterpret_cast<unsigned char*>(grad_features) + block_first * 72;
    const int bytes = in_block * 72;
    // one bulk asynchronous store of the block's contiguous 72-byte rows when base and size are multiples
    // of 16 bytes; 16-byte stores through registers otherwise
    const bool bulk = bulk_ok && (bytes & 15) == 0;
    if (bulk) fence_shared_for_bulk();
    __syncthreads();
    if (bulk) {
        if (threadIdx.x == 0) bulk_store_from_shared(dst, s_out, (unsigned)bytes);
        return;
    }
    const int n16 = bytes / 16;
    uint4* dst16 = reinterpret_cast<uint4*>(dst);
    const uint4* src16 = reinterpret_cast<const uint4*>(s_out);
    for (int k = threadIdx.x; k < n16; k += kPreThreads) dst16[k] = src16[k];
    for (int k = n16 * 16 + 2 * threadIdx.x; k < bytes; k += 2 * kPreThreads)
        *reinterpret_cast<unsigned short*>(dst + k) = *reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(s_out) + k);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
struct PointBlob {
    PointRec* rec;
    uint2* bounds;
    uint32_t* quad;                       // warp blend: packed footprint origin per point (see pack_quad)
    float4* conic;
    unsigned* block_visible;              // survivors per chunk of kPreThreads points
    unsigned* group_visible;              // per group of 4 chunks; scanned in place
    unsigned long long* group_instances;
    unsigned long long* counters;   // visible, instances, smallest / largest depth bit pattern
    unsigned* depth_min;
    unsigned* depth_max;
    uint32_t* keys[2];
    uint32_t* ids[2];
    unsigned* inst_block_sums;
    void* sort_ws;
    size_t total;
};

// Sized by the number of input points alone (every per-visible array gets room for all of them), so
// that the layout is known before the visible count has been read back.
PointBlob carve_point_blob(void* p, int64_t n, int mode) {
    PointBlob b;
    Carver c(p);
    const int64_t nb = ceil_div<int64_t>(n > 0 ? n : 1, kPreThreads);
    b.rec = c.take<PointRec>(n);
    b.bounds = c.take<uint2>(n);
    b.quad = c.take<uint32_t>(mode == INPC_MODE_BILINEAR ? n : 0);
    b.conic = mode == INPC_MODE_GAUSSIAN ? c.take<float4>(n) : nullptr;
    b.block_visible = c.take<unsigned>(nb);
    b.group_visible = c.take<unsigned>(ceil_div<int64_t>(nb, 4));
    b.group_instances = c.take<unsigned long long>(ceil_div<int64_t>(nb, 4));
    b.counters = c.take<unsigned long long>(4);
    b.depth_min = c.take<unsigned>(1);
    b.depth_max = c.take<unsigned>(1);
    for (int k = 0; k < 2; ++k) b.keys[k] = c.take<uint32_t>(n);
    for (int k = 0; k < 2; ++k) b.ids[k] = c.take<uint32_t>(n);
    b.inst_block_sums = c.take<unsigned>(ceil_div<int64_t>(n > 0 ? n : 1, kInstThreads));
    c.off = align_up(c.off);
    b.sort_ws = c.base + c.off;
    c.off += sort_workspace_bytes(n);
    b.total = c.used();
    return b;
}

struct InstanceBlob {
    uint32_t* keys[2];
    uint32_t* ids[2];
    uint2* ranges;
    Segment* segs;
    uint32_t* tile_first;
    uint32_t* n_segments;
    float* seg_T;
    float4* seg_C;
    float* seg_Z;
    float* seg_E;         // warp blend, inference: transmittance at the end of every segment
    int64_t max_segments;
    uint32_t* tile_rank;  // warp blend: per block of 1024 tiles, the segments and the non-empty tiles before it
    WarpItem* items0;     // warp blend: segment 0 of the non-empty tiles
    WarpItem* items1;     // warp blend: every segment behind a tile's first
    uint32_t* n_kept;     // warp blend: per item, length of the compacted list the forward pass blended
    void* sort_ws;
    size_t total;
};

// Upper bound on the number of (tile, segment) work items, known from the instance count alone.
int blend_batch(int tile);
int64_t max_segments(int64_t n_instances, int n_tiles, int tile) {
    return (int64_t)n_tiles + ceil_div<int64_t>(n_instances, (int64_t)blend_batch(tile) * kMinBatchesPerSegment);
}

// Which of the two blend organisations a call uses: one warp per tile part with the dead-instance filter
// (bilinear splats, 8x8 tiles, four view-space channels) or one block per (tile, segment).
constexpr int kWarpBlendParts = 2;   // work items per (tile, segment): the two 8x4 halves
bool uses_warp_blend(int mode, int tile, bool rows) { return mode == INPC_MODE_BILINEAR && tile == 8 && !rows; }

InstanceBlob carve_instance_blob(void* p, int64_t n_instances, int n_tiles, int tile, int mode, bool with_depth, int c4 = 1, bool rows = false) {
    InstanceBlob b;
    Carver c(p);
    const bool warp_blend = uses_warp_blend(mode, tile, rows);
    b.ranges = c.take<uint2>(n_tiles);
    for (int k = 0; k < 2; ++k) b.keys[k] = c.take<uint32_t>(n_instances);
    for (int k = 0; k < 2; ++k) b.ids[k] = c.take<uint32_t>(n_instances);
    // upper bound on the number of (tile, segment) pairs, known from the instance count alone
    b.max_segments = warp_blend ? (int64_t)n_tiles + ceil_div<int64_t>(n_instances, (int64_t)kLaterSegment) : max_segments(n_instances, n_tiles, tile);
    const size_t px = (size_t)b.max_segments * tile * tile;
    b.segs = c.take<Segment>(warp_blend ? 0 : b.max_segments);
    b.tile_first = c.take<uint32_t>(n_tiles);
    // [0] segments (block blend) or non-empty tiles (warp blend), [1] later segments (warp blend), [2..5] work tickets of
    // the warp blend passes FIRST, PRODUCT, REST and of its backward pass
    b.n_segments = c.take<uint32_t>(8);
    b.seg_T = c.take<float>(px);
    b.seg_C = c.take<float4>(px * (size_t)c4);
    b.seg_Z = c.take<float>(with_depth ? px : 0);
    b.seg_E = c.take<float>(with_depth && warp_blend ? px : 0);
    b.tile_rank = c.take<uint32_t>(warp_blend ? (size_t)n_tiles + 8 : 0);   // warp blend: (segments, tiles) per block of 1024 tiles
    b.items0 = c.take<WarpItem>(warp_blend ? (size_t)n_tiles : 0);
    b.items1 = c.take<WarpItem>(warp_blend ? (size_t)b.max_segments : 0);
    b.n_kept = c.take<uint32_t>(warp_blend ? (size_t)b.max_segments * kWarpBlendParts : 0);
    c.off = align_up(c.off);
    b.sort_ws = c.base + c.off;
    c.off += sort_workspace_bytes(n_instances);
    b.total = c.used();
    return b;
}

// The state handed back to the caller only stores blob bases and counts; which ping-pong buffer holds
// a sorted result follows from the number of radix passes, which follows from the counts.
int depth_result_buffer(int64_t n_visible, int depth_key_bits) { return n_visible > 1 ? (sort_pass_count(depth_key_bits) & 1) : 0; }
int tile_result_buffer(int64_t n_instances, int n_tiles) {
    const int end_bit = bit_length((uint32_t)(n_tiles - 1));
    return n_instances > 1 ? (sort_pass_count(end_bit) & 1) : 0;
}

// One event per host thread and device: an event belongs to the device that was current when it was made.
// Instance capacity the blobs of `st` were carved for, and which ping-pong buffer holds the tile-sorted lists.
int64_t instance_capacity(const inpc_raster_state* st) { return st->deferred_counts ? 4 * st->n_points : st->n_instances; }
int tile_buffer_of(const inpc_raster_state* st, int n_tiles) {
    if (st->deferred_counts) return sort_pass_count(bit_length((uint32_t)(n_tiles - 1))) & 1;
    return tile_result_buffer(st->n_instances, n_tiles);
}
int depth_buffer_of(const inpc_raster_state* st) {
    if (st->deferred_counts) return sort_pass_count(st->depth_key_bits) & 1;
    return depth_result_buffer(st->n_visible, st->depth_key_bits);
}

cudaEvent_t counters_event() {
    static thread_local cudaEvent_t events[kMaxDevices] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!events[dev] && cudaEventCreateWithFlags(&events[dev], cudaEventDisableTiming) != cudaSuccess) events[dev] = nullptr;
    return events[dev];
}

unsigned long long* pinned_counters() {
    static thread_local unsigned long long* p = nullptr;
    if (!p && cudaHostAlloc(reinterpret_cast<void**>(&p), 4 * sizeof(unsigned long long), cudaHostAllocDefault) != cudaSuccess) p = nullptr;
    return p;
}

int check_view(const inpc_view* v, int tile_size, int mode, int64_t n) {
    if (!v || !v->w2c || !v->cam_position) { set_error("view, view.w2c and view.cam_position must be non-null"); return INPC_E_INVALID; }
    if (mode != INPC_MODE_BILINEAR && mode != INPC_MODE_GAUSSIAN) { set_error("unsupported rasterizer mode %d", mode); return INPC_E_INVALID; }
    if (tile_size != 8 && tile_size != 16) { set_error("tile_size must be 8 or 16, got %d", tile_size); return INPC_E_INVALID; }
    if (v->width <= 0 || v->height <= 0 || v->width > 65535 * tile_size || v->height > 65535 * tile_size) {
        set_error("image size %dx%d out of range", v->width, v->height);
        return INPC_E_INVALID;
    }
    if (mode == INPC_MODE_BILINEAR && tile_size == 8 && (v->width > kMaxCodedSide || ceil_div(v->height, 8) > kMaxCodedTileRows)) {
        set_error("image size %dx%d exceeds the %d x %d pixels of the 8x8-tile bilinear path (use tile_size 16)", v->width, v->height, kMaxCodedSide,
                  kMaxCodedTileRows * 8);
        return INPC_E_INVALID;
    }
    // tile indices live in the low kTileKeyBits bits of the instance keys
    const int64_t tiles = (int64_t)ceil_div(v->width, tile_size) * ceil_div(v->height, tile_size);
    if (tiles > ((int64_t)1 << kTileKeyBits)) {
        set_error("image size %dx%d gives %lld tiles of %d pixels, more than the supported 2^%u", v->width, v->height, (long long)tiles, tile_size, kTileKeyBits);
        return INPC_E_INVALID;
    }
    if (n < 0 || n >= ((int64_t)1 << 30)) { set_error("n=%lld out of range [0, 2^30)", (long long)n); return INPC_E_INVALID; }
    return INPC_OK;
}

// Checked build: publish the index limit before a call's kernels / collect the failure count after them.
int begin_index_checks(int64_t n_points, cudaStream_t stream) {
#ifdef INPC_CHECK_INDICES
    const unsigned long long limit = (unsigned long long)n_points;
    const unsigned zero = 0;
    INPC_CUDA_TRY(cudaMemcpyToSymbolAsync(g_check_n_points, &limit, sizeof(limit), 0, cudaMemcpyHostToDevice, stream));
    INPC_CUDA_TRY(cudaMemcpyToSymbolAsync(g_check_failures, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, stream));
#else
    (void)n_points; (void)stream;
#endif
    return INPC_OK;
}

int end_index_checks(cudaStream_t stream) {
#ifdef INPC_CHECK_INDICES
    unsigned failures = 0;
    INPC_CUDA_TRY(cudaMemcpyFromSymbolAsync(&failures, g_check_failures, sizeof(failures), 0, cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    if (failures) {
        set_error("checked build: %u point indices read from the sorted lists were out of range (accesses skipped)", failures);
        return INPC_E_DEVICE;
    }
#else
    (void)stream;
#endif
    return INPC_OK;
}

template <int MODE, int VARIANT>
int run_front(const RasterParams& rp, int64_t n, const float* positions, const void* features, const float* opacities,
              inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* user, inpc_raster_state* st,
              bool with_depth, PointBlob* pb_out, InstanceBlob* ib_out, cudaStream_t stream, const char* entry, int c4 = 1,
              const PointSets* sets = nullptr) {
    // `sets`: the input of a batched multi-set call (then n is the virtual total and the three pointers are unused)
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    PointSets ps;
    if (sets) {
        ps = *sets;
    } else {
        ps.count = 1;
        ps.start[0] = 0; ps.start[1] = n;
        ps.size[0] = n;
        ps.positions[0] = positions; ps.features[0] = features; ps.opacities[0] = opacities;
    }
    {
        // a failure an earlier call of this thread reported from the device surfaces here at the latest
        const int rc_prev = check_previous_calls();
        if (rc_prev != INPC_OK) return rc_prev;
    }
    unsigned* status = acquire_status(entry);
    if (!status) return INPC_E_CUDA;
    constexpr bool kRows = VARIANT == VAR_ROWS;
    const bool warp_blend = uses_warp_blend(MODE, rp.tile, kRows);
    const int64_t nb = ceil_div<int64_t>(n > 0 ? n : 1, kPreThreads);
    const PointBlob sizing = carve_point_blob(nullptr, n, MODE);
    void* pblob = alloc_point(user, sizing.total);
    if (!pblob) { set_error("point allocator returned NULL for %zu bytes", sizing.total); return INPC_E_ALLOC; }
    const PointBlob pb = carve_point_blob(pblob, n, MODE);
    {
        const int rc_check = begin_index_checks(n, stream);
        if (rc_check != INPC_OK) return rc_check;
    }

    // Bilinear splats touch at most 2x2 tiles, so the warp-blend path sizes everything behind the visibility pass
    // for 4 n instances and lets the kernels read the two counts from device memory: no host synchronisation at
    // all (the reference reads both counts back with blocking copies, src/bilinear/forward.cu:86-89).  The other
    // paths (gaussian splats have no such bound) read the counts back once.
    const bool deferred = warp_blend && n > 0 && n < ((int64_t)1 << 28);
    int64_t n_visible = 0, n_instances = 0;
    uint32_t key_base = 0;
    int key_bits = 0;
    const unsigned long long* n_visible_dev = deferred ? pb.counters : nullptr;
    const unsigned long long* n_instances_dev = deferred ? pb.counters + 1 : nullptr;
    if (n > 0) {
        unsigned long long* host = nullptr;
        cudaEvent_t ready = nullptr;
        int pack_count = -1;
        uint32_t lo_bits = 0u, hi_bits = 0u;
        if (deferred) {
            // depth keys are offsets from the near plane's bit pattern, bounded by the far plane's: nothing is measured
            const float lo = rp.v.near_plane > 0.0f ? rp.v.near_plane : 0.0f, hi = rp.v.far_plane > lo ? rp.v.far_plane : lo;
            memcpy(&lo_bits, &lo, 4);
            memcpy(&hi_bits, &hi, 4);
            if (!(rp.v.near_plane > 0.0f)) { lo_bits = 0u; hi_bits = 0xFFFFFFFFu; }
            key_bits = rp.v.near_plane > 0.0f ? bit_length(hi_bits - lo_bits) : 32;
            if (key_bits == 0) key_bits = 1;
            key_base = lo_bits;
            pack_count = key_bits <= (int)kCountShift ? 1 : 0;
            n_visible = n;                // capacities from here on
            n_instances = 4 * n;
        } else {
            host = pinned_counters();
            ready = counters_event();
            if (!host || !ready) return cuda_fail(cudaGetLastError(), "cudaHostAlloc / cudaEventCreate (counters)");
        }
        {
            StageScope scope(STAGE_PREPROCESS, stream);
            INPC_CUDA_TRY(cudaMemsetAsync(pb.depth_min, 0xFF, sizeof(unsigned), stream));
            INPC_CUDA_TRY(cudaMemsetAsync(pb.depth_max, 0, sizeof(unsigned), stream));
            const int64_t groups = ceil_div<int64_t>(nb, 4);
            visibility_count_kernel<MODE, VARIANT><<<(unsigned)groups, kPreThreads, 0, stream>>>(ps, rp, pb.block_visible, pb.group_visible,
                                                                                             pb.group_instances, deferred ? nullptr : pb.depth_min,
                                                                                             deferred ? nullptr : pb.depth_max);
            INPC_LAUNCH_CHECK("visibility_count_kernel");
            scan_block_counts_kernel<<<1, kScanThreads, 0, stream>>>(pb.group_visible, pb.group_instances, groups, pb.depth_min, pb.depth_max, pb.counters,
                                                                     deferred ? 1 : 0, lo_bits, hi_bits);
            INPC_LAUNCH_CHECK("scan_block_counts_kernel");
            if (!deferred) {
                INPC_CUDA_TRY(cudaMemcpyAsync(host, pb.counters, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream));
                INPC_CUDA_TRY(cudaEventRecord(ready, stream));
            }
            // the projection pass needs nothing from the host: it runs while the host waits for the counters
            preprocess_kernel<MODE, VARIANT><<<(unsigned)nb, kPreThreads, 0, stream>>>(
                ps, rp, pb.block_visible, pb.group_visible, pb.depth_min, pb.depth_max,
                pb.rec, pb.bounds, warp_blend ? pb.quad : nullptr,
                pb.conic, pb.keys[0], pb.ids[0], pack_count, status);
            INPC_LAUNCH_CHECK("preprocess_kernel");
        }
        if (!deferred) {
            INPC_CUDA_TRY(cudaEventSynchronize(ready));
            n_visible = (int64_t)host[0];
            n_instances = (int64_t)host[1];
            // counts that cannot be: more survivors than points, or (bilinear: at most 2x2 tiles per splat)
            // more instances than four per survivor, or instances without survivors
            if (n_visible > n || (n_visible == 0 && n_instances != 0) || (MODE == INPC_MODE_BILINEAR && n_instances > 4 * n_visible)) {
                set_error("inconsistent counts from the visibility pass: %lld visible of %lld points, %lld instances", (long long)n_visible,
                          (long long)n, (long long)n_instances);
                return INPC_E_DEVICE;
            }
            if (n_visible > 0) {
                key_base = (uint32_t)host[2];
                key_bits = bit_length((uint32_t)host[3] - key_base);
            }
        }
    }
    if (n_instances >= ((int64_t)1 << 30)) {
        set_error("%lld (point, tile) instances exceed the 2^30 capacity", (long long)n_instances);
        return INPC_E_CAPACITY;
    }

    const InstanceBlob isz = carve_instance_blob(nullptr, n_instances, n_tiles, rp.tile, MODE, with_depth, c4, kRows);
    void* iblob = alloc_instance(user, isz.total);
    if (!iblob) { set_error("instance allocator returned NULL for %zu bytes", isz.total); return INPC_E_ALLOC; }
    InstanceBlob ib = carve_instance_blob(iblob, n_instances, n_tiles, rp.tile, MODE, with_depth, c4, kRows);
    INPC_CUDA_TRY(cudaMemsetAsync(ib.ranges, 0, sizeof(uint2) * (size_t)n_tiles, stream));

    int in_alt = 0;
    int rc;
    {
        StageScope scope(STAGE_SORT_DEPTH, stream);
        rc = deferred ? sort_pairs_device_count(pb.keys[0], pb.keys[1], pb.ids[0], pb.ids[1], n_visible, n_visible_dev, key_bits, pb.sort_ws, status, &in_alt, stream)
                      : sort_pairs(pb.keys[0], pb.keys[1], pb.ids[0], pb.ids[1], n_visible, key_bits, pb.sort_ws, status, &in_alt, stream);
    }
    if (rc != INPC_OK) return rc;
    const uint32_t* sorted_ids = pb.ids[in_alt];
    if (n_visible > 0 && n_instances > 0) {
        const int64_t ibk = ceil_div<int64_t>(n_visible, kInstThreads);
        {
            StageScope scope(STAGE_INSTANCES, stream);
            // the count of touched tiles rides in the top key bits when the depth offsets left them free
            if (MODE == INPC_MODE_BILINEAR && key_bits <= (int)kCountShift)
                instance_count_kernel<true><<<(unsigned)ibk, kInstThreads / 4, 0, stream>>>(pb.keys[in_alt], sorted_ids, pb.bounds, n_visible, n_visible_dev, pb.inst_block_sums);
            else
                instance_count_kernel<false><<<(unsigned)ibk, kInstThreads / 4, 0, stream>>>(pb.keys[in_alt], sorted_ids, pb.bounds, n_visible, n_visible_dev, pb.inst_block_sums);
            INPC_LAUNCH_CHECK("instance_count_kernel");
            scan_u32_kernel<<<1, kScanThreads, 0, stream>>>(pb.inst_block_sums, ibk);
            INPC_LAUNCH_CHECK("scan_u32_kernel");
            if (warp_blend)
                emit_instances_kernel<true><<<(unsigned)ibk, kInstThreads, 0, stream>>>(sorted_ids, pb.bounds, pb.quad, n_visible, n_visible_dev, pb.inst_block_sums, rp.gw, ib.keys[0], ib.ids[0]);
            else
                emit_instances_kernel<false><<<(unsigned)ibk, kInstThreads, 0, stream>>>(sorted_ids, pb.bounds, nullptr, n_visible, n_visible_dev, pb.inst_block_sums, rp.gw, ib.keys[0], ib.ids[0]);
            INPC_LAUNCH_CHECK("emit_instances_kernel");
        }
        StageScope scope(STAGE_SORT_TILE, stream);
        int t_alt = 0;
        const int tile_bits = bit_length((uint32_t)(n_tiles - 1));
        rc = deferred ? sort_pairs_device_count(ib.keys[0], ib.keys[1], ib.ids[0], ib.ids[1], n_instances, n_instances_dev, tile_bits, ib.sort_ws, status, &t_alt, stream)
                      : sort_pairs(ib.keys[0], ib.keys[1], ib.ids[0], ib.ids[1], n_instances, tile_bits, ib.sort_ws, status, &t_alt, stream);
        if (rc != INPC_OK) return rc;
        tile_ranges_kernel<<<(unsigned)ceil_div<int64_t>(n_instances, 256 * 8), 256, 0, stream>>>(ib.keys[t_alt], n_instances, n_instances_dev, ib.ranges);
        INPC_LAUNCH_CHECK("tile_ranges_kernel");
    }
    if (warp_blend) {
        StageScope scope(STAGE_SORT_TILE, stream);
        INPC_CUDA_TRY(cudaMemsetAsync(ib.n_segments, 0, 8 * sizeof(uint32_t), stream));
        const int item_blocks = ceil_div(n_tiles, kItemTilesPerBlock);
        uint2* item_sums = reinterpret_cast<uint2*>(ib.tile_rank);
        warp_items_count_kernel<<<item_blocks, kItemThreads, 0, stream>>>(ib.ranges, n_tiles, item_sums);
        INPC_LAUNCH_CHECK("warp_items_count_kernel");
        warp_items_scan_kernel<<<1, kScanThreads, 0, stream>>>(item_sums, item_blocks, ib.n_segments);
        INPC_LAUNCH_CHECK("warp_items_scan_kernel");
        warp_items_fill_kernel<<<item_blocks, kItemThreads, 0, stream>>>(ib.ranges, n_tiles, item_sums, ib.items0, ib.items1);
        INPC_LAUNCH_CHECK("warp_items_fill_kernel");
    } else {
        StageScope scope(STAGE_SORT_TILE, stream);
        count_segments_kernel<<<1, kScanThreads, 0, stream>>>(ib.ranges, n_tiles, blend_batch(rp.tile), ib.tile_first, ib.n_segments);
        INPC_LAUNCH_CHECK("count_segments_kernel");
        emit_segments_kernel<<<ceil_div(n_tiles, 256), 256, 0, stream>>>(ib.ranges, n_tiles, blend_batch(rp.tile), ib.tile_first, ib.segs);
        INPC_LAUNCH_CHECK("emit_segments_kernel");
    }
    st->point_blob = pblob;
    st->instance_blob = iblob;
    st->n_points = n;
    st->n_visible = deferred ? -1 : n_visible;       // -1: still on the device, see inpc_raster_resolve
    st->n_instances = deferred ? -1 : n_instances;
    st->tile_size = rp.tile;
    st->mode = MODE;
    st->depth_key_base = key_base;
    st->depth_key_bits = key_bits;
    st->channels = VARIANT == VAR_ROWS ? 4 * c4 : 4;
    st->deferred_counts = deferred ? 1 : 0;
    *pb_out = pb;
    *ib_out = ib;
    return INPC_OK;
}

RasterParams make_params(const inpc_view* view, int tile_size, float sigma_world, float sigma_cutoff, const float* scales) {
    RasterParams rp;
    rp.v = to_params(view);
    rp.tile = tile_size;
    rp.inv_tile = 1.0f / (float)tile_size;
    rp.gw = ceil_div(view->width, tile_size);
    rp.gh = ceil_div(view->height, tile_size);
    rp.n_sets = 1;
    rp.sigma_world = sigma_world;
    rp.sigma_cutoff = sigma_cutoff;
    rp.scales = scales;
    return rp;
}

// Instances staged per pixel thread and batch.  Measured on B200 (2^23 points, clustered and uniform
// scenes): one per thread is fastest for both tile sizes; deeper batches lose more to mask traffic
// and same-word atomicOr contention than they gain from fewer barriers.
template <int T> struct BlendConfig;
template <> struct BlendConfig<8> { static constexpr int kIpt = 1; };
template <> struct BlendConfig<16> { static constexpr int kIpt = 1; };

int blend_batch(int tile) { return tile == 8 ? 64 * BlendConfig<8>::kIpt : 256 * BlendConfig<16>::kIpt; }

// Persistent grid of the warp blend: enough blocks to fill the GPU (the item counts live on the device).
int warp_blend_grid(unsigned* grid) {
    *grid = (unsigned)max(1, sm_count() * 4);
    return INPC_OK;
}

struct ForwardPassArgs {
    const uint32_t *keys, *ids;
    const PointRec* rec;
    float* seg_T;
    float4* seg_C;
    float *seg_Z, *seg_E, *image, *depth, *alpha, *blending_weights;
    uint32_t *kept0, *kept1, *n_kept;
    int W, H, gw, gh;
};

// One pass of the warp blend's forward: its shared memory (the per-warp rings) is above the 48 KB a kernel gets unasked.
template <int PASS, int KIND>
int launch_warp_forward_pass(unsigned grid, const WarpItem* items, const uint32_t* counts, unsigned* ticket, const ForwardPassArgs& a,
                             cudaStream_t stream) {
    static bool attr_set[kMaxDevices] = {false};
    constexpr size_t smem = warp_forward_smem_bytes<PASS, KIND>();
    const int rc = opt_in_dynamic_smem(blend_bilinear_warp_forward_kernel<PASS, KIND>, smem, attr_set);
    if (rc != INPC_OK) return rc;
    blend_bilinear_warp_forward_kernel<PASS, KIND><<<grid, kWarpBlendWarps * 32, smem, stream>>>(
        items, counts, ticket, a.keys, a.ids, a.rec, a.seg_T, a.seg_C, a.seg_Z, a.seg_E, a.image, a.depth, a.alpha, a.blending_weights,
        a.kept0, a.kept1, a.n_kept, a.W, a.H, a.gw, a.gh);
    INPC_LAUNCH_CHECK("blend_bilinear_warp_forward_kernel");
    return INPC_OK;
}

template <int KIND>
int launch_bilinear_warp_forward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, int t_alt, float* image,
                                 float* depth, float* alpha, float* blending_weights, cudaStream_t stream) {
    unsigned grid = 1;
    const int rc = warp_blend_grid(&grid);
    if (rc != INPC_OK) return rc;
    const int W = rp.v.width, H = rp.v.height;
    // tiles without instances are not work items: their pixels are cleared here
    const size_t n_px = (size_t)W * H * rp.n_sets;
    INPC_CUDA_TRY(cudaMemsetAsync(image, 0, sizeof(float) * 4 * n_px, stream));
    INPC_CUDA_TRY(cudaMemsetAsync(alpha, 0, sizeof(float) * n_px, stream));
    if (KIND == BLEND_INFER) INPC_CUDA_TRY(cudaMemsetAsync(depth, 0, sizeof(float) * n_px, stream));
    // the ping-pong buffers the tile sort left unused receive the compacted lists (part 0: ids, part 1: keys)
    const uint32_t* keys = ib.keys[t_alt];
    const uint32_t* ids = ib.ids[t_alt];
    uint32_t* kept0 = ib.ids[1 - t_alt];
    uint32_t* kept1 = ib.keys[1 - t_alt];
    const unsigned threads = kWarpBlendWarps * 32;
    const ForwardPassArgs a{keys, ids, pb.rec, ib.seg_T, ib.seg_C, ib.seg_Z, ib.seg_E, image, depth, alpha, blending_weights,
                            kept0, kept1, ib.n_kept, W, H, rp.gw, rp.gh};
    int rc_pass = launch_warp_forward_pass<PASS_FIRST, KIND>(grid, ib.items0, ib.n_segments, ib.n_segments + 2, a, stream);
    if (rc_pass != INPC_OK) return rc_pass;
    rc_pass = launch_warp_forward_pass<PASS_PRODUCT, KIND>(grid, ib.items1, ib.n_segments, ib.n_segments + 3, a, stream);
    if (rc_pass != INPC_OK) return rc_pass;
    warp_blend_prefix_kernel<<<grid, threads, 0, stream>>>(ib.items0, ib.n_segments, ib.seg_T);
    INPC_LAUNCH_CHECK("warp_blend_prefix_kernel");
    rc_pass = launch_warp_forward_pass<PASS_REST, KIND>(grid, ib.items1, ib.n_segments, ib.n_segments + 4, a, stream);
    if (rc_pass != INPC_OK) return rc_pass;
    warp_blend_combine_kernel<KIND><<<grid, threads, 0, stream>>>(ib.items0, ib.n_segments, ib.seg_C, ib.seg_Z, ib.seg_E,
                                                                      image, depth, alpha, W, H, rp.gw, rp.gh);
    INPC_LAUNCH_CHECK("warp_blend_combine_kernel");
    return INPC_OK;
}

int launch_bilinear_warp_backward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, int t_alt, const float* grad_image,
                                  const float* grad_alpha, const float* image, const float* alpha, float4* slot_grad,
                                  unsigned* slot_mask, cudaStream_t stream) {
    unsigned grid = 1;
    const int rc = warp_blend_grid(&grid);
    if (rc != INPC_OK) return rc;
    INPC_CUDA_TRY(cudaMemsetAsync(ib.n_segments + 5, 0, sizeof(uint32_t), stream));   // the work ticket
    static bool attr_set[kMaxDevices] = {false};
    const int rc_attr = opt_in_dynamic_smem(blend_bilinear_warp_backward_kernel, kWarpBackwardSmemBytes, attr_set);
    if (rc_attr != INPC_OK) return rc_attr;
    blend_bilinear_warp_backward_kernel<<<grid, kWarpBlendWarps * 32, kWarpBackwardSmemBytes, stream>>>(
        ib.items0, ib.items1, ib.n_segments, ib.n_segments + 5, ib.ids[1 - t_alt], ib.keys[1 - t_alt], ib.n_kept, pb.rec,
        ib.seg_T, ib.seg_C, grad_image, grad_alpha, image, alpha, slot_grad, slot_mask, rp.v.width, rp.v.height, rp.gw);
    INPC_LAUNCH_CHECK("blend_bilinear_warp_backward_kernel");
    return INPC_OK;
}

template <int T, int KIND>
int launch_bilinear_forward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, const uint32_t* ids, float* image,
                            float* depth, float* alpha, float* blending_weights, cudaStream_t stream) {
    constexpr int IPT = BlendConfig<T>::kIpt;
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    const int W = rp.v.width, H = rp.v.height;
    const unsigned grid = (unsigned)ib.max_segments;
    blend_bilinear_transmittance_kernel<T, IPT><<<grid, T * T, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, ib.seg_T, W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_bilinear_transmittance_kernel");
    blend_prefix_kernel<T><<<n_tiles, T * T, 0, stream>>>(ib.segs, ib.tile_first, ib.seg_T);
    INPC_LAUNCH_CHECK("blend_prefix_kernel");
    blend_bilinear_forward_kernel<T, IPT, KIND><<<grid, T * T, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, ib.seg_T, ib.seg_C, ib.seg_Z,
                                                                           image, depth, alpha, blending_weights, W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_bilinear_forward_kernel");
    blend_combine_kernel<T, KIND><<<n_tiles, T * T, 0, stream>>>(ib.segs, ib.tile_first, ib.seg_C, ib.seg_Z, ib.seg_T, image, depth, alpha,
                                                                W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_combine_kernel");
    return INPC_OK;
}

template <int T>
int launch_bilinear_backward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, const uint32_t* ids,
                             const float* grad_image, const float* grad_alpha, const float* image, const float* alpha, float4* gfv,
                             float* grad_opacities, cudaStream_t stream) {
    constexpr int IPT = BlendConfig<T>::kIpt;
    constexpr size_t smem = backward_smem_bytes<T, IPT>();
    static bool attr_set[kMaxDevices] = {false};
    {
        const int rc_attr = opt_in_dynamic_smem(blend_bilinear_backward_kernel<T, IPT>, smem, attr_set);
        if (rc_attr != INPC_OK) return rc_attr;
    }
    blend_bilinear_backward_kernel<T, IPT><<<(unsigned)ib.max_segments, T * T, smem, stream>>>(
        ib.segs, ib.n_segments, ids, pb.rec, ib.seg_T, ib.seg_C, grad_image, grad_alpha, image, alpha, gfv, grad_opacities,
        rp.v.width, rp.v.height, rp.gw);
    INPC_LAUNCH_CHECK("blend_bilinear_backward_kernel");
    return INPC_OK;
}

template <int T, int KIND>
int launch_gaussian_forward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, const uint32_t* ids, float* image,
                            float* depth, float* alpha, float* blending_weights, float threshold, cudaStream_t stream) {
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    const int W = rp.v.width, H = rp.v.height;
    const unsigned grid = (unsigned)ib.max_segments;
    const float neg_log_threshold = -logf(threshold);
    blend_gaussian_transmittance_kernel<T, KIND == BLEND_INFER><<<grid, T * T, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, pb.conic, ib.seg_T, W, H,
                                                                                          rp.gw, threshold, neg_log_threshold);
    INPC_LAUNCH_CHECK("blend_gaussian_transmittance_kernel");
    blend_prefix_kernel<T><<<n_tiles, T * T, 0, stream>>>(ib.segs, ib.tile_first, ib.seg_T);
    INPC_LAUNCH_CHECK("blend_prefix_kernel");
    blend_gaussian_forward_kernel<T, KIND><<<grid, T * T, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, pb.conic, ib.seg_T, ib.seg_C, ib.seg_Z, image,
                                                                      depth, alpha, blending_weights, W, H, rp.gw, threshold, neg_log_threshold);
    INPC_LAUNCH_CHECK("blend_gaussian_forward_kernel");
    blend_combine_kernel<T, KIND><<<n_tiles, T * T, 0, stream>>>(ib.segs, ib.tile_first, ib.seg_C, ib.seg_Z, ib.seg_T, image, depth, alpha, W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_combine_kernel");
    return INPC_OK;
}

template <int KIND>
int launch_blend_forward(int mode, const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, const inpc_raster_state* st,
                         float* image, float* depth, float* alpha, float* blending_weights, float threshold,
                         cudaStream_t stream) {
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    const int t_alt = tile_buffer_of(st, n_tiles);
    const uint32_t* ids = ib.ids[t_alt];
    StageScope scope(STAGE_BLEND_FWD, stream);
    if (mode == INPC_MODE_BILINEAR) {
        if (rp.tile == 8) return launch_bilinear_warp_forward<KIND>(rp, pb, ib, t_alt, image, depth, alpha, blending_weights, stream);
        return launch_bilinear_forward<16, KIND>(rp, pb, ib, ids, image, depth, alpha, blending_weights, stream);
    }
    if (rp.tile == 8) return launch_gaussian_forward<8, KIND>(rp, pb, ib, ids, image, depth, alpha, blending_weights, threshold, stream);
    return launch_gaussian_forward<16, KIND>(rp, pb, ib, ids, image, depth, alpha, blending_weights, threshold, stream);
}

template <int T, int C4, int KIND>
int launch_rows_forward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, const uint32_t* ids, const float* features,
                        float* image, float* depth, float* alpha, float* blending_weights, cudaStream_t stream) {
    constexpr size_t smem = rows_forward_smem_bytes<T, C4>();
    static bool attr_set[kMaxDevices] = {false};
    {
        const int rc_attr = opt_in_dynamic_smem(blend_rows_forward_kernel<T, C4, KIND>, smem, attr_set);
        if (rc_attr != INPC_OK) return rc_attr;
    }
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    const int W = rp.v.width, H = rp.v.height;
    const unsigned grid = (unsigned)ib.max_segments;
    blend_bilinear_transmittance_kernel<T, 1><<<grid, T * T, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, ib.seg_T, W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_bilinear_transmittance_kernel");
    blend_prefix_kernel<T><<<n_tiles, T * T, 0, stream>>>(ib.segs, ib.tile_first, ib.seg_T);
    INPC_LAUNCH_CHECK("blend_prefix_kernel");
    blend_rows_forward_kernel<T, C4, KIND><<<grid, T * T, smem, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, reinterpret_cast<const float4*>(features),
                                                                         ib.seg_T, ib.seg_C, ib.seg_Z, image, depth, alpha, blending_weights, W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_rows_forward_kernel");
    blend_rows_combine_kernel<T, C4, KIND><<<n_tiles, T * T, 0, stream>>>(ib.segs, ib.tile_first, ib.seg_C, ib.seg_Z, ib.seg_T, image, depth, alpha,
                                                                         W, H, rp.gw);
    INPC_LAUNCH_CHECK("blend_rows_combine_kernel");
    return INPC_OK;
}

template <int T, int C4>
int launch_rows_backward(const RasterParams& rp, const PointBlob& pb, const InstanceBlob& ib, const uint32_t* ids, const float* features,
                         const float* grad_image, const float* grad_alpha, const float* image, const float* alpha,
                         float* grad_features, float* grad_opacities, cudaStream_t stream) {
    constexpr size_t smem = rows_backward_smem_bytes<T, C4>();
    static bool attr_set[kMaxDevices] = {false};
    {
        const int rc_attr = opt_in_dynamic_smem(blend_rows_backward_kernel<T, C4>, smem, attr_set);
        if (rc_attr != INPC_OK) return rc_attr;
    }
    blend_rows_backward_kernel<T, C4><<<(unsigned)ib.max_segments, T * T, smem, stream>>>(
        ib.segs, ib.n_segments, ids, pb.rec, reinterpret_cast<const float4*>(features), ib.seg_T, ib.seg_C, grad_image, grad_alpha, image, alpha,
        reinterpret_cast<float4*>(grad_features), grad_opacities, rp.v.width, rp.v.height, rp.gw);
    INPC_LAUNCH_CHECK("blend_rows_backward_kernel");
    return INPC_OK;
}

// Tile edge and channel count are template parameters of the kernels: one switch for all of them.
template <typename F>
int dispatch_rows(int tile, int channels, F&& f) {
    if (tile == 8) {
        if (channels == 4) return f(std::integral_constant<int, 8>(), std::integral_constant<int, 1>());
        if (channels == 8) return f(std::integral_constant<int, 8>(), std::integral_constant<int, 2>());
        if (channels == 16) return f(std::integral_constant<int, 8>(), std::integral_constant<int, 4>());
        if (channels == 32) return f(std::integral_constant<int, 8>(), std::integral_constant<int, 8>());
    } else if (tile == 16) {
        if (channels == 4) return f(std::integral_constant<int, 16>(), std::integral_constant<int, 1>());
        if (channels == 8) return f(std::integral_constant<int, 16>(), std::integral_constant<int, 2>());
        if (channels == 16) return f(std::integral_constant<int, 16>(), std::integral_constant<int, 4>());
        if (channels == 32) return f(std::integral_constant<int, 16>(), std::integral_constant<int, 8>());
    }
    set_error("feature rows: channels must be 4, 8, 16 or 32 (got %d) and tile_size 8 or 16 (got %d)", channels, tile);
    return INPC_E_INVALID;
}

template <int KIND>
int rows_forward(int tile_size, const inpc_view* view, int64_t n, const float* positions, const float* features, int channels,
                 const float* opacities, float* image, float* depth, float* alpha, float* blending_weights,
                 inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user, inpc_raster_state* state, cudaStream_t stream) {
    const RasterParams rp = make_params(view, tile_size, 0.0f, 3.0f, nullptr);
    PointBlob pb;
    InstanceBlob ib;
    int rc = run_front<INPC_MODE_BILINEAR, VAR_ROWS>(rp, n, positions, nullptr, opacities, alloc_point, alloc_instance, alloc_user, state,
                                                     KIND == BLEND_INFER, &pb, &ib, stream, KIND == BLEND_INFER ? "inpc_render_rows" : "inpc_rasterize_rows_forward", channels / 4);
    if (rc != INPC_OK) return rc;
    const uint32_t* ids = ib.ids[tile_buffer_of(state, rp.gw * rp.gh)];
    {
        StageScope scope(STAGE_BLEND_FWD, stream);
        rc = dispatch_rows(tile_size, channels, [&](auto t, auto c4) {
            return launch_rows_forward<decltype(t)::value, decltype(c4)::value, KIND>(rp, pb, ib, ids, features, image, depth, alpha, blending_weights, stream);
        });
    }
    return rc != INPC_OK ? rc : end_index_checks(stream);
}

}  // namespace

}  // namespace inpc

using namespace inpc;

extern "C" int inpc_rasterize_forward(int mode, int tile_size, const inpc_view* view, int64_t n, const float* positions,
                                      const void* features, const float* opacities, float* image, float* alpha,
                                      float* blending_weights, inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance,
                                      void* alloc_user, inpc_raster_state* state, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_view(view, tile_size, mode, n);
    if (rc != INPC_OK) return rc;
    if (!state || !alloc_point || !alloc_instance || !image || !alpha || (n > 0 && (!positions || !features || !opacities || !blending_weights))) {
        set_error("inpc_rasterize_forward: null argument");
        return INPC_E_INVALID;
    }
    const RasterParams rp = make_params(view, tile_size, 0.0f, 3.0f, nullptr);
    if (n > 0) INPC_CUDA_TRY(cudaMemsetAsync(blending_weights, 0, sizeof(float) * (size_t)n, stream));
    PointBlob pb;
    InstanceBlob ib;
    if (mode == INPC_MODE_BILINEAR)
        rc = run_front<INPC_MODE_BILINEAR, VAR_TRAIN>(rp, n, positions, features, opacities, alloc_point, alloc_instance, alloc_user, state, false, &pb, &ib, stream, "inpc_rasterize_forward");
    else
        rc = run_front<INPC_MODE_GAUSSIAN, VAR_TRAIN>(rp, n, positions, features, opacities, alloc_point, alloc_instance, alloc_user, state, false, &pb, &ib, stream, "inpc_rasterize_forward");
    if (rc != INPC_OK) return rc;
    rc = launch_blend_forward<BLEND_TRAIN>(mode, rp, pb, ib, state, image, nullptr, alpha, blending_weights, kTrainGaussThreshold, stream);
    return rc != INPC_OK ? rc : end_index_checks(stream);
}

extern "C" int inpc_rasterize_backward(const inpc_raster_state* state, const inpc_view* view, const float* grad_image,
                                       const float* grad_alpha, const float* image, const float* alpha,
                                       const float* positions, const float* opacities, float* grad_features_view,
                                       void* grad_features, float* grad_opacities, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!state) { set_error("inpc_rasterize_backward: null state"); return INPC_E_INVALID; }
    int rc = check_view(view, state->tile_size, state->mode, state->n_points);
    if (rc != INPC_OK) return rc;
    const int64_t n = state->n_points;
    if (!grad_image || !grad_alpha || !image || !alpha || (n > 0 && (!positions || !grad_features_view || !grad_features || !grad_opacities || !state->point_blob || !state->instance_blob))) {
        set_error("inpc_rasterize_backward: null argument");
        return INPC_E_INVALID;
    }
    (void)opacities;   // the opacity travels in the point record
    if (n == 0) return INPC_OK;
    rc = begin_index_checks(n, stream);
    if (rc != INPC_OK) return rc;
    const RasterParams rp = make_params(view, state->tile_size, 0.0f, 3.0f, nullptr);
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    const PointBlob pb = carve_point_blob(state->point_blob, n, state->mode);
    const InstanceBlob ib = carve_instance_blob(state->instance_blob, instance_capacity(state), n_tiles, state->tile_size, state->mode, false);
    const uint32_t* ids = ib.ids[tile_buffer_of(state, n_tiles)];
    float4* gfv = reinterpret_cast<float4*>(grad_features_view);
    const int W = rp.v.width, H = rp.v.height;
    // the caller's scratch holds 33 floats per point: four 32-byte slot records and one mask word for the warp blend
    // or, for the other paths, the (n,4) accumulation buffer of their atomics
    const bool slots = uses_warp_blend(state->mode, state->tile_size, false);
    if (slots && (reinterpret_cast<uintptr_t>(grad_features_view) & 31u)) {
        set_error("inpc_rasterize_backward: grad_features_view must be 32-byte aligned");
        return INPC_E_INVALID;
    }
    float4* slot_grad = gfv;
    unsigned* slot_mask = reinterpret_cast<unsigned*>(grad_features_view + 32 * (size_t)n);
    if (slots) {
        INPC_CUDA_TRY(cudaMemsetAsync(slot_mask, 0, sizeof(unsigned) * (size_t)n, stream));
    } else {
        INPC_CUDA_TRY(cudaMemsetAsync(grad_features_view, 0, sizeof(float4) * (size_t)n, stream));
        INPC_CUDA_TRY(cudaMemsetAsync(grad_opacities, 0, sizeof(float) * (size_t)n, stream));
    }
    {
        StageScope scope(STAGE_BLEND_BWD, stream);
        if (state->mode == INPC_MODE_BILINEAR) {
            rc = rp.tile == 8 ? launch_bilinear_warp_backward(rp, pb, ib, tile_buffer_of(state, n_tiles), grad_image, grad_alpha, image, alpha, slot_grad, slot_mask, stream)
                              : launch_bilinear_backward<16>(rp, pb, ib, ids, grad_image, grad_alpha, image, alpha, gfv, grad_opacities, stream);
            if (rc != INPC_OK) return rc;
        } else {
            const unsigned grid = (unsigned)ib.max_segments;
            if (rp.tile == 8)
                blend_gaussian_backward_kernel<8><<<grid, 64, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, pb.conic, ib.seg_T, ib.seg_C, grad_image, grad_alpha, image, alpha, gfv, grad_opacities, W, H, rp.gw);
            else
                blend_gaussian_backward_kernel<16><<<grid, 256, 0, stream>>>(ib.segs, ib.n_segments, ids, pb.rec, pb.conic, ib.seg_T, ib.seg_C, grad_image, grad_alpha, image, alpha, gfv, grad_opacities, W, H, rp.gw);
            INPC_LAUNCH_CHECK("blend_gaussian_backward_kernel");
        }
    }
    StageScope scope(STAGE_PREPROCESS_BWD, stream);
    const GradientSlots gs{slot_grad, slot_mask};
    const bool bulk_ok = (reinterpret_cast<uintptr_t>(grad_features) & 15u) == 0;
    if (slots)
        preprocess_backward_kernel<true><<<(unsigned)ceil_div<int64_t>(n, kPreThreads), kPreThreads, 0, stream>>>(
            positions, view->cam_position, pb.bounds, gfv, gs, grad_opacities, static_cast<__half*>(grad_features), n, bulk_ok);
    else
        preprocess_backward_kernel<false><<<(unsigned)ceil_div<int64_t>(n, kPreThreads), kPreThreads, 0, stream>>>(
            positions, view->cam_position, pb.bounds, gfv, gs, grad_opacities, static_cast<__half*>(grad_features), n, bulk_ok);
    INPC_LAUNCH_CHECK("preprocess_backward_kernel");
    return end_index_checks(stream);
}

extern "C" int inpc_render(int mode, int tile_size, const inpc_view* view, int64_t n, const float* positions,
                           const void* features_raw, float sigma_world, float sigma_cutoff, float* image, float* depth,
                           float* alpha, inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user,
                           void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_view(view, tile_size, mode, n);
    if (rc != INPC_OK) return rc;
    if (!alloc_point || !alloc_instance || !image || !depth || !alpha || (n > 0 && (!positions || !features_raw))) {
        set_error("inpc_render: null argument");
        return INPC_E_INVALID;
    }
    const RasterParams rp = make_params(view, tile_size, sigma_world, sigma_cutoff, nullptr);
    inpc_raster_state st;
    PointBlob pb;
    InstanceBlob ib;
    if (mode == INPC_MODE_BILINEAR)
        rc = run_front<INPC_MODE_BILINEAR, VAR_RAW37>(rp, n, positions, features_raw, nullptr, alloc_point, alloc_instance, alloc_user, &st, true, &pb, &ib, stream, "inpc_render");
    else
        rc = run_front<INPC_MODE_GAUSSIAN, VAR_RAW37>(rp, n, positions, features_raw, nullptr, alloc_point, alloc_instance, alloc_user, &st, true, &pb, &ib, stream, "inpc_render");
    if (rc != INPC_OK) return rc;
    // runtime cut-off exp(-cutoff^2/2): src/gaussian/inference.cu:171
    const float threshold = expf(-0.5f * sigma_cutoff * sigma_cutoff);
    rc = launch_blend_forward<BLEND_INFER>(mode, rp, pb, ib, &st, image, depth, alpha, nullptr, threshold, stream);
    return rc != INPC_OK ? rc : end_index_checks(stream);
}

extern "C" int inpc_render_preextracted(int mode, int tile_size, const inpc_view* view, int64_t n, const float* positions,
                                        const void* features, const float* opacities, const float* scales,
                                        float sigma_world, float sigma_cutoff, float* image, float* depth, float* alpha,
                                        inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user,
                                        void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_view(view, tile_size, mode, n);
    if (rc != INPC_OK) return rc;
    if (!alloc_point || !alloc_instance || !image || !depth || !alpha || (n > 0 && (!positions || !features || !opacities))) {
        set_error("inpc_render_preextracted: null argument");
        return INPC_E_INVALID;
    }
    const RasterParams rp = make_params(view, tile_size, sigma_world, sigma_cutoff, scales);
    inpc_raster_state st;
    PointBlob pb;
    InstanceBlob ib;
    if (mode == INPC_MODE_BILINEAR)
        rc = run_front<INPC_MODE_BILINEAR, VAR_PREEXTRACTED>(rp, n, positions, features, opacities, alloc_point, alloc_instance, alloc_user, &st, true, &pb, &ib, stream, "inpc_render_preextracted");
    else
        rc = run_front<INPC_MODE_GAUSSIAN, VAR_PREEXTRACTED>(rp, n, positions, features, opacities, alloc_point, alloc_instance, alloc_user, &st, true, &pb, &ib, stream, "inpc_render_preextracted");
    if (rc != INPC_OK) return rc;
    const float threshold = expf(-0.5f * sigma_cutoff * sigma_cutoff);
    rc = launch_blend_forward<BLEND_INFER>(mode, rp, pb, ib, &st, image, depth, alpha, nullptr, threshold, stream);
    return rc != INPC_OK ? rc : end_index_checks(stream);
}

extern "C" int inpc_render_multi(int tile_size, const inpc_view* view, int n_sets, const int64_t* n_points, const float* const* positions,
                                 const void* const* features_raw, float* images, float* depths, float* alphas,
                                 inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_sets < 1 || n_sets > kMaxSets) { set_error("inpc_render_multi: n_sets=%d outside [1, %d]", n_sets, kMaxSets); return INPC_E_INVALID; }
    if (!n_points || !positions || !features_raw || !alloc_point || !alloc_instance || !images || !depths || !alphas) {
        set_error("inpc_render_multi: null argument");
        return INPC_E_INVALID;
    }
    if (tile_size != 8) { set_error("inpc_render_multi: bilinear splats on 8x8 tiles only (tile_size %d)", tile_size); return INPC_E_INVALID; }
    PointSets ps;
    ps.count = n_sets;
    int64_t cursor = 0;
    for (int j = 0; j < n_sets; ++j) {
        if (n_points[j] < 0 || (n_points[j] > 0 && (!positions[j] || !features_raw[j]))) { set_error("inpc_render_multi: bad set %d", j); return INPC_E_INVALID; }
        ps.start[j] = cursor;
        ps.size[j] = n_points[j];
        ps.positions[j] = positions[j];
        ps.features[j] = features_raw[j];
        ps.opacities[j] = nullptr;
        cursor = (cursor + n_points[j] + kSetAlign - 1) / kSetAlign * kSetAlign;   // every set starts a block of the input passes
    }
    ps.start[n_sets] = cursor;
    const int64_t n_virtual = cursor;
    int rc = check_view(view, tile_size, INPC_MODE_BILINEAR, n_virtual);
    if (rc != INPC_OK) return rc;
    RasterParams rp = make_params(view, tile_size, 0.0f, 3.0f, nullptr);
    rp.n_sets = n_sets;
    // the stacked grid has to fit what a single image may use: tile indices in 24 bits, tile rows in 11
    if ((int64_t)rp.gw * rp.gh * n_sets > ((int64_t)1 << kTileKeyBits) || (int64_t)rp.gh * n_sets > kMaxCodedTileRows) {
        set_error("inpc_render_multi: %d images of %dx%d exceed the stacked tile grid", n_sets, view->width, view->height);
        return INPC_E_INVALID;
    }
    inpc_raster_state st;
    PointBlob pb;
    InstanceBlob ib;
    rc = run_front<INPC_MODE_BILINEAR, VAR_RAW37>(rp, n_virtual, nullptr, nullptr, nullptr, alloc_point, alloc_instance, alloc_user, &st, true, &pb, &ib,
                                                  stream, "inpc_render_multi", 1, &ps);
    if (rc != INPC_OK) return rc;
    rc = launch_blend_forward<BLEND_INFER>(INPC_MODE_BILINEAR, rp, pb, ib, &st, images, depths, alphas, nullptr, 0.0f, stream);
    return rc != INPC_OK ? rc : end_index_checks(stream);
}

namespace {
int check_rows(const inpc_view* view, int tile_size, int64_t n, int channels) {
    const int rc = check_view(view, tile_size, INPC_MODE_BILINEAR, n);
    if (rc != INPC_OK) return rc;
    if (channels != 4 && channels != 8 && channels != 16 && channels != 32) { set_error("feature rows: channels must be 4, 8, 16 or 32, got %d", channels); return INPC_E_INVALID; }
    return INPC_OK;
}
}  // namespace

extern "C" int inpc_rasterize_rows_forward(int tile_size, const inpc_view* view, int64_t n, const float* positions,
                                           const float* features, int channels, const float* opacities, float* image,
                                           float* alpha, float* blending_weights, inpc_alloc_fn alloc_point,
                                           inpc_alloc_fn alloc_instance, void* alloc_user, inpc_raster_state* state, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_rows(view, tile_size, n, channels);
    if (rc != INPC_OK) return rc;
    if (!state || !alloc_point || !alloc_instance || !image || !alpha || (n > 0 && (!positions || !features || !opacities || !blending_weights))) {
        set_error("inpc_rasterize_rows_forward: null argument");
        return INPC_E_INVALID;
    }
    if (reinterpret_cast<uintptr_t>(features) & 15u) { set_error("inpc_rasterize_rows_forward: features must be 16-byte aligned"); return INPC_E_INVALID; }
    if (n > 0) INPC_CUDA_TRY(cudaMemsetAsync(blending_weights, 0, sizeof(float) * (size_t)n, stream));
    return rows_forward<BLEND_TRAIN>(tile_size, view, n, positions, features, channels, opacities, image, nullptr, alpha, blending_weights,
                                     alloc_point, alloc_instance, alloc_user, state, stream);
}

extern "C" int inpc_render_rows(int tile_size, const inpc_view* view, int64_t n, const float* positions, const float* features,
                                int channels, const float* opacities, float* image, float* depth, float* alpha,
                                inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_rows(view, tile_size, n, channels);
    if (rc != INPC_OK) return rc;
    if (!alloc_point || !alloc_instance || !image || !depth || !alpha || (n > 0 && (!positions || !features || !opacities))) {
        set_error("inpc_render_rows: null argument");
        return INPC_E_INVALID;
    }
    if (reinterpret_cast<uintptr_t>(features) & 15u) { set_error("inpc_render_rows: features must be 16-byte aligned"); return INPC_E_INVALID; }
    inpc_raster_state st;
    return rows_forward<BLEND_INFER>(tile_size, view, n, positions, features, channels, opacities, image, depth, alpha, nullptr,
                                     alloc_point, alloc_instance, alloc_user, &st, stream);
}

extern "C" int inpc_rasterize_rows_backward(const inpc_raster_state* state, const inpc_view* view, const float* grad_image,
                                            const float* grad_alpha, const float* image, const float* alpha, const float* features,
                                            float* grad_features, float* grad_opacities, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!state) { set_error("inpc_rasterize_rows_backward: null state"); return INPC_E_INVALID; }
    int rc = check_rows(view, state->tile_size, state->n_points, state->channels);
    if (rc != INPC_OK) return rc;
    if (state->mode != INPC_MODE_BILINEAR) { set_error("inpc_rasterize_rows_backward: state is not from inpc_rasterize_rows_forward"); return INPC_E_INVALID; }
    const int64_t n = state->n_points;
    const int channels = state->channels;
    if (!grad_image || !grad_alpha || !image || !alpha || (n > 0 && (!features || !grad_features || !grad_opacities || !state->point_blob || !state->instance_blob))) {
        set_error("inpc_rasterize_rows_backward: null argument");
        return INPC_E_INVALID;
    }
    if ((reinterpret_cast<uintptr_t>(features) | reinterpret_cast<uintptr_t>(grad_features)) & 15u) {
        set_error("inpc_rasterize_rows_backward: features and grad_features must be 16-byte aligned");
        return INPC_E_INVALID;
    }
    if (n == 0) return INPC_OK;
    const RasterParams rp = make_params(view, state->tile_size, 0.0f, 3.0f, nullptr);
    const int n_tiles = rp.gw * rp.gh * rp.n_sets;
    const PointBlob pb = carve_point_blob(state->point_blob, n, state->mode);
    const InstanceBlob ib = carve_instance_blob(state->instance_blob, instance_capacity(state), n_tiles, state->tile_size, state->mode, false, channels / 4, true);
    const uint32_t* ids = ib.ids[tile_buffer_of(state, n_tiles)];
    INPC_CUDA_TRY(cudaMemsetAsync(grad_features, 0, sizeof(float) * (size_t)n * channels, stream));
    INPC_CUDA_TRY(cudaMemsetAsync(grad_opacities, 0, sizeof(float) * (size_t)n, stream));
    rc = begin_index_checks(n, stream);
    if (rc != INPC_OK) return rc;
    {
        StageScope scope(STAGE_BLEND_BWD, stream);
        rc = dispatch_rows(state->tile_size, channels, [&](auto t, auto c4) {
            return launch_rows_backward<decltype(t)::value, decltype(c4)::value>(rp, pb, ib, ids, features, grad_image, grad_alpha, image, alpha,
                                                                                grad_features, grad_opacities, stream);
        });
    }
    return rc != INPC_OK ? rc : end_index_checks(stream);
}

extern "C" int inpc_raster_resolve(inpc_raster_state* state, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!state) { set_error("inpc_raster_resolve: null state"); return INPC_E_INVALID; }
    if (!state->deferred_counts || state->n_points == 0) return INPC_OK;
    if (!state->point_blob) { set_error("inpc_raster_resolve: state without a point blob"); return INPC_E_INVALID; }
    const PointBlob pb = carve_point_blob(state->point_blob, state->n_points, state->mode);
    unsigned long long host[4];
    INPC_CUDA_TRY(cudaMemcpyAsync(host, pb.counters, sizeof(host), cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    state->n_visible = (int64_t)host[0];
    state->n_instances = (int64_t)host[1];
    state->depth_key_base = state->n_visible > 0 ? (uint32_t)host[2] : 0u;
    if (state->n_visible > state->n_points || state->n_instances > 4 * state->n_visible) {
        set_error("inconsistent counts from the visibility pass: %lld visible of %lld points, %lld instances", (long long)state->n_visible,
                  (long long)state->n_points, (long long)state->n_instances);
        return INPC_E_DEVICE;
    }
    return INPC_OK;
}

namespace inpc_debug {
__global__ void add_base_kernel(const uint32_t* __restrict__ src, int64_t n, uint32_t base, uint32_t mask, uint32_t* __restrict__ dst) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = (src[i] & mask) + base;
}

__global__ void unpack_points_kernel(const PointRec* __restrict__ rec, const uint2* __restrict__ bounds, int64_t n, int which,
                                     void* __restrict__ dst) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint2 b = bounds[i];
    const bool vis = tiles_of(b) != 0u;
    const float4* r = reinterpret_cast<const float4*>(rec + i);
    if (which == 4) static_cast<unsigned*>(dst)[i] = tiles_of(b);
    else if (which == 5) { const float4 a = vis ? r[0] : make_float4(0, 0, 0, 0); static_cast<float2*>(dst)[i] = make_float2(a.x, a.y); }
    else if (which == 6) static_cast<float*>(dst)[i] = vis ? r[0].w : 0.0f;
    else if (which == 7) static_cast<float4*>(dst)[i] = vis ? r[1] : make_float4(0, 0, 0, 0);
    else if (which == 8) {
        unsigned short* o = static_cast<unsigned short*>(dst) + 4 * i;
        o[0] = (unsigned short)(b.x & 0xffffu); o[1] = (unsigned short)(b.x >> 16);
        o[2] = (unsigned short)(b.y & 0xffffu); o[3] = (unsigned short)(b.y >> 16);
    }
}
}  // namespace inpc_debug

extern "C" int inpc_raster_debug_copy(const inpc_raster_state* state, const inpc_view* view, int which, void* dst,
                                      void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!state || !view || !dst) { set_error("inpc_raster_debug_copy: null argument"); return INPC_E_INVALID; }
    const int gw = ceil_div(view->width, state->tile_size), gh = ceil_div(view->height, state->tile_size);
    const int n_tiles = gw * gh;
    const PointBlob pb = carve_point_blob(state->point_blob, state->n_points, state->mode);
    if (state->n_visible < 0 || state->n_instances < 0) { set_error("inpc_raster_debug_copy: the counts of this state are still on the device; call inpc_raster_resolve first"); return INPC_E_INVALID; }
    const InstanceBlob ib = carve_instance_blob(state->instance_blob, instance_capacity(state), n_tiles, state->tile_size, state->mode, false);
    const int d = depth_buffer_of(state);
    const int ti = tile_buffer_of(state, n_tiles);
    switch (which) {
        case 0: INPC_CUDA_TRY(cudaMemcpyAsync(dst, pb.ids[d], 4 * (size_t)state->n_visible, cudaMemcpyDeviceToDevice, stream)); break;
        case 1:   // the sort works on offsets from the smallest depth key: add the base back
            if (state->n_visible > 0) {
                inpc_debug::add_base_kernel<<<(unsigned)ceil_div<int64_t>(state->n_visible, 256), 256, 0, stream>>>(
                    pb.keys[d], state->n_visible, state->depth_key_base,
                    state->depth_key_bits <= 30 ? 0x3FFFFFFFu : 0xFFFFFFFFu, static_cast<uint32_t*>(dst));
                INPC_LAUNCH_CHECK("add_base_kernel");
            }
            break;
        case 2: INPC_CUDA_TRY(cudaMemcpyAsync(dst, ib.ids[ti], 4 * (size_t)state->n_instances, cudaMemcpyDeviceToDevice, stream)); break;
        case 3: INPC_CUDA_TRY(cudaMemcpyAsync(dst, ib.ranges, 8 * (size_t)n_tiles, cudaMemcpyDeviceToDevice, stream)); break;
        case 4: case 5: case 6: case 7: case 8:
            if (state->n_points > 0) {
                inpc_debug::unpack_points_kernel<<<(unsigned)ceil_div<int64_t>(state->n_points, 256), 256, 0, stream>>>(pb.rec, pb.bounds, state->n_points, which, dst);
                INPC_LAUNCH_CHECK("unpack_points_kernel");
            }
            break;
        default: set_error("inpc_raster_debug_copy: unknown array %d", which); return INPC_E_INVALID;
    }
    return INPC_OK;
}

