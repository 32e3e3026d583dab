// Structural updates of the octree probability field: prune (drop leaves below an occupancy
// threshold) and subdivide (replace high-score leaves by their eight children).  Both are stable
// stream compactions, written as a count pass, a one-block scan of block sums and a fill pass, so
// the output order is fixed: the survivors in their old order, then (subdivide) the children of
// the selected leaves in leaf order, child k = (x bit, y bit, z bit) = (k&1, k&2, k&4).
// Reference: Modules/ProbabilityField.py:159-165 (prune) and :217-257 (subdivide), which do the same
// with boolean-mask indexing, repeat_interleave and strided slice updates in torch.
#include "common.cuh"

namespace inpc {

namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 4;
constexpr int kChunk = kThreads * kPerThread;   // leaves per block
constexpr int kScanThreads = 1024;

enum { SELECT_PRUNE = 0, SELECT_SUBDIVIDE = 1 };

template <int KIND>
__device__ __forceinline__ bool selected(const float* __restrict__ values, const int32_t* __restrict__ levels, int64_t i, float threshold,
                                         int max_level) {
    const float v = __ldg(values + i);
    if (KIND == SELECT_PRUNE) return v > threshold;                      // kept leaves: weight > threshold
    return v > threshold && __ldg(levels + i) < max_level;               // split leaves: score > threshold, level < limit
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) leaf_select_count_kernel(const float* __restrict__ values, const int32_t* __restrict__ levels,
                                                                     int64_t n, float threshold, int max_level,
                                                                     unsigned* __restrict__ block_sums) {
    __shared__ unsigned s_scan[kThreads / 32 + 1];
    const int64_t first = (int64_t)blockIdx.x * kChunk + (int64_t)threadIdx.x * kPerThread;
    unsigned c = 0;
#pragma unroll
    for (int k = 0; k < kPerThread; ++k)
        if (first + k < n && selected<KIND>(values, levels, first + k, threshold, max_level)) ++c;
    unsigned total;
    block_exclusive_scan(c, s_scan, &total);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// Exclusive scan of the block sums in place by one block; the grand total goes to *total_out.
__global__ void __launch_bounds__(kScanThreads) leaf_scan_sums_kernel(unsigned* __restrict__ sums, int64_t n_blocks,
                                                                      unsigned long long* __restrict__ total_out) {
    __shared__ unsigned s_scan[kScanThreads / 32 + 1];
    const int64_t per = ceil_div<int64_t>(n_blocks, kScanThreads);
    const int64_t lo = (int64_t)threadIdx.x * per, hi = min(n_blocks, lo + per);
    unsigned local = 0;
    for (int64_t b = lo; b < hi; ++b) local += sums[b];
    unsigned total;
    unsigned run = block_exclusive_scan(local, s_scan, &total);
    for (int64_t b = lo; b < hi; ++b) {
        const unsigned v = sums[b];
        sums[b] = run;
        run += v;
    }
    if (threadIdx.x == 0) *total_out = total;
}

struct LeafArrays {
    const float* centers;
    const int32_t* levels;
    const float* weights;
    const float* scores;
};
struct LeafOutputs {
    float* centers;
    int32_t* levels;
    float* weights;
    float* scores;
};

__device__ __forceinline__ void copy_leaf(const LeafArrays& in, int64_t i, const LeafOutputs& out, int64_t o) {
    out.centers[3 * o] = __ldg(in.centers + 3 * i);
    out.centers[3 * o + 1] = __ldg(in.centers + 3 * i + 1);
    out.centers[3 * o + 2] = __ldg(in.centers + 3 * i + 2);
    out.levels[o] = __ldg(in.levels + i);
    out.weights[o] = __ldg(in.weights + i);
    out.scores[o] = __ldg(in.scores + i);
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) leaf_fill_kernel(LeafArrays in, int64_t n, float threshold, int max_level, float initial_size,
                                                             const unsigned* __restrict__ block_offsets, int64_t n_selected,
                                                             LeafOutputs out) {
    __shared__ unsigned s_scan[kThreads / 32 + 1];
    const int64_t first = (int64_t)blockIdx.x * kChunk + (int64_t)threadIdx.x * kPerThread;
    bool sel[kPerThread];
    unsigned c = 0;
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
        sel[k] = first + k < n && selected<KIND>(KIND == SELECT_PRUNE ? in.weights : in.scores, in.levels, first + k, threshold, max_level);
        c += sel[k] ? 1u : 0u;
    }
    unsigned total;
    int64_t rank = (int64_t)block_offsets[blockIdx.x] + block_exclusive_scan(c, s_scan, &total);   // selected leaves before this one
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
        const int64_t i = first + k;
        if (i >= n) break;
        if (KIND == SELECT_PRUNE) {
            if (sel[k]) copy_leaf(in, i, out, rank);
        } else if (!sel[k]) {
            copy_leaf(in, i, out, i - rank);
        } else {
            // children: level + 1, the parent's weight, score 0, centre moved by half a child edge per
            // axis: initial_size / 2^(new level + 1)   (ProbabilityField.py:231-251)
            const int level = __ldg(in.levels + i) + 1;
            const float offset = initial_size / (float)(1u << (level + 1));
            const float cx = __ldg(in.centers + 3 * i), cy = __ldg(in.centers + 3 * i + 1), cz = __ldg(in.centers + 3 * i + 2);
            const float w = __ldg(in.weights + i);
            const int64_t base = (n - n_selected) + 8 * rank;
#pragma unroll
            for (int child = 0; child < 8; ++child) {
                const int64_t o = base + child;
                out.centers[3 * o] = (child & 1) ? cx + offset : cx - offset;
                out.centers[3 * o + 1] = (child & 2) ? cy + offset : cy - offset;
                out.centers[3 * o + 2] = (child & 4) ? cz + offset : cz - offset;
                out.levels[o] = level;
                out.weights[o] = w;
                out.scores[o] = 0.0f;
            }
        }
        rank += sel[k] ? 1 : 0;
    }
}

bool bad_leaf_count(int64_t n) { return n < 0 || n >= ((int64_t)1 << 31); }

}  // namespace

}  // namespace inpc

using namespace inpc;

extern "C" size_t inpc_leaf_select_workspace_bytes(int64_t n_leaves) {
    const int64_t blocks = ceil_div<int64_t>(n_leaves > 0 ? n_leaves : 1, kChunk);
    return align_up(sizeof(unsigned) * (size_t)blocks) + 256;
}

namespace {
unsigned long long* total_slot(void* workspace, int64_t n) {
    const int64_t blocks = ceil_div<int64_t>(n > 0 ? n : 1, kChunk);
    return reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(workspace) + align_up(sizeof(unsigned) * (size_t)blocks));
}
}  // namespace

extern "C" int inpc_leaf_select_count(int kind, const float* values, const int32_t* levels, int64_t n, float threshold, int max_level,
                                      void* workspace, int64_t* n_selected, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!n_selected) { set_error("inpc_leaf_select_count: n_selected is null"); return INPC_E_INVALID; }
    *n_selected = 0;
    if (n == 0) return INPC_OK;
    if (bad_leaf_count(n) || !values || !workspace || (kind != SELECT_PRUNE && kind != SELECT_SUBDIVIDE) ||
        (kind == SELECT_SUBDIVIDE && (!levels || max_level < 0 || max_level > 29))) {
        set_error("inpc_leaf_select_count: bad argument");
        return INPC_E_INVALID;
    }
    unsigned* sums = static_cast<unsigned*>(workspace);
    const int64_t blocks = ceil_div<int64_t>(n, kChunk);
    if (kind == SELECT_PRUNE)
        leaf_select_count_kernel<SELECT_PRUNE><<<(unsigned)blocks, kThreads, 0, stream>>>(values, levels, n, threshold, max_level, sums);
    else
        leaf_select_count_kernel<SELECT_SUBDIVIDE><<<(unsigned)blocks, kThreads, 0, stream>>>(values, levels, n, threshold, max_level, sums);
    INPC_LAUNCH_CHECK("leaf_select_count_kernel");
    unsigned long long* total = total_slot(workspace, n);
    leaf_scan_sums_kernel<<<1, kScanThreads, 0, stream>>>(sums, blocks, total);
    INPC_LAUNCH_CHECK("leaf_scan_sums_kernel");
    unsigned long long host = 0;
    INPC_CUDA_TRY(cudaMemcpyAsync(&host, total, sizeof(host), cudaMemcpyDeviceToHost, stream));
    INPC_CUDA_TRY(cudaStreamSynchronize(stream));
    *n_selected = (int64_t)host;
    return INPC_OK;
}

extern "C" int inpc_leaf_prune_fill(const float* centers, const int32_t* levels, const float* weights, const float* scores, int64_t n,
                                    float threshold, const void* workspace, float* out_centers, int32_t* out_levels,
                                    float* out_weights, float* out_scores, void* stream_) {
    if (n == 0) return INPC_OK;
    if (bad_leaf_count(n) || !centers || !levels || !weights || !scores || !workspace || !out_centers || !out_levels || !out_weights || !out_scores) {
        set_error("inpc_leaf_prune_fill: bad argument");
        return INPC_E_INVALID;
    }
    const int64_t blocks = ceil_div<int64_t>(n, kChunk);
    leaf_fill_kernel<SELECT_PRUNE><<<(unsigned)blocks, kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
        LeafArrays{centers, levels, weights, scores}, n, threshold, 0, 0.0f, static_cast<const unsigned*>(workspace), 0,
        LeafOutputs{out_centers, out_levels, out_weights, out_scores});
    INPC_LAUNCH_CHECK("leaf_fill_kernel");
    return INPC_OK;
}

extern "C" int inpc_leaf_subdivide_fill(const float* centers, const int32_t* levels, const float* weights, const float* scores, int64_t n,
                                        float threshold, int max_level, float initial_size, int64_t n_selected, const void* workspace,
                                        float* out_centers, int32_t* out_levels, float* out_weights, float* out_scores, void* stream_) {
    if (n == 0) return INPC_OK;
    if (bad_leaf_count(n) || n_selected < 0 || n_selected > n || bad_leaf_count(n + 7 * n_selected) || max_level < 0 || max_level > 29 || !centers ||
        !levels || !weights || !scores || !workspace || !out_centers || !out_levels || !out_weights || !out_scores) {
        set_error("inpc_leaf_subdivide_fill: bad argument");
        return INPC_E_INVALID;
    }
    const int64_t blocks = ceil_div<int64_t>(n, kChunk);
    leaf_fill_kernel<SELECT_SUBDIVIDE><<<(unsigned)blocks, kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
        LeafArrays{centers, levels, weights, scores}, n, threshold, max_level, initial_size, static_cast<const unsigned*>(workspace), n_selected,
        LeafOutputs{out_centers, out_levels, out_weights, out_scores});
    INPC_LAUNCH_CHECK("leaf_fill_kernel");
    return INPC_OK;
}
