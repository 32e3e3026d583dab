// Fused element-wise helpers of the inpc_b200 library (hash-grid weight decay, spherical
// contraction, Cauchy loss).  Pure HBM streams: 16-byte vector accesses where the layout allows and
// grid-stride loops sized to the SM count.  Citations are paths below
// INPCCudaBackend/INPCCudaBackend/misc/ of the reference.
#include "common.cuh"

namespace inpc {

namespace {

constexpr int kThreads = 256;

int grid_for(int64_t work_items) {
    const int sms = sm_count();
    const int64_t want = ceil_div<int64_t>(work_items, kThreads);
    const int64_t cap = (int64_t)sms * 8;
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

// Per-level factor 0.2 / len(level) of the fixed ten-level hash grid, zero below index 6144:
// src/misc_kernels.cu:15-36.
__device__ __forceinline__ float decay_factor(unsigned idx) {
    constexpr float f0 = 0.1f * 2.0f / float(210917376 - 177362944);
    constexpr float f1 = 0.1f * 2.0f / float(177362944 - 143808512);
    constexpr float f2 = 0.1f * 2.0f / float(143808512 - 110254080);
    constexpr float f3 = 0.1f * 2.0f / float(110254080 - 76699648);
    constexpr float f4 = 0.1f * 2.0f / float(76699648 - 43145216);
    constexpr float f5 = 0.1f * 2.0f / float(43145216 - 9590784);
    constexpr float f6 = 0.1f * 2.0f / float(9590784 - 1202176);
    constexpr float f7 = 0.1f * 2.0f / float(1202176 - 153600);
    constexpr float f8 = 0.1f * 2.0f / float(153600 - 22528);
    constexpr float f9 = 0.1f * 2.0f / float(22528 - 6144);
    if (idx >= 177362944u) return f0;
    if (idx >= 143808512u) return f1;
    if (idx >= 110254080u) return f2;
    if (idx >= 76699648u) return f3;
    if (idx >= 43145216u) return f4;
    if (idx >= 9590784u) return f5;
    if (idx >= 1202176u) return f6;
    if (idx >= 153600u) return f7;
    if (idx >= 22528u) return f8;
    if (idx >= 6144u) return f9;
    return 0.0f;
}

// Every level boundary is a multiple of 4, so a float4 never straddles two levels.
template <bool ADD>
__global__ void __launch_bounds__(kThreads) weight_decay_kernel(const float* __restrict__ w, float* __restrict__ g, int64_t n,
                                                                bool vec_ok) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int64_t n4 = vec_ok ? n / 4 : 0;
    for (int64_t v = tid; v < n4; v += stride) {
        const float f = decay_factor((unsigned)(4 * v));
        const float4 wv = __ldg(reinterpret_cast<const float4*>(w) + v);
        float4 gv;
        if (ADD) {
            gv = reinterpret_cast<float4*>(g)[v];
            gv.x += f * wv.x; gv.y += f * wv.y; gv.z += f * wv.z; gv.w += f * wv.w;
        } else {
            gv = make_float4(f * wv.x, f * wv.y, f * wv.z, f * wv.w);
        }
        reinterpret_cast<float4*>(g)[v] = gv;
    }
    for (int64_t i = 4 * n4 + tid; i < n; i += stride) {
        const float f = decay_factor((unsigned)i);
        if (ADD) g[i] += f * w[i];
        else g[i] = f * w[i];
    }
}

// src/misc_kernels.cu:49-66
__global__ void __launch_bounds__(kThreads) contraction_kernel(const float* __restrict__ p, float* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float x = __ldg(p + 3 * i), y = __ldg(p + 3 * i + 1), z = __ldg(p + 3 * i + 2);
        const float length_sq = fmaxf(x * x + y * y + z * z, 1.0f);
        const float scale = (sqrtf(length_sq) * 2.0f - 1.0f) / length_sq * 0.25f;
        out[3 * i] = __saturatef(scale * x + 0.5f);
        out[3 * i + 1] = __saturatef(scale * y + 0.5f);
        out[3 * i + 2] = __saturatef(scale * z + 0.5f);
    }
}

// Cauchy loss, src/misc_kernels.cu:68-79, with the mean reduction fused: per-block partial sums in a
// fixed order, then one block adds the partials in index order.
__global__ void __launch_bounds__(kThreads) cauchy_partial_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                  int64_t n, float* __restrict__ partial) {
    __shared__ float s[kThreads / 32];
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const float nf = (float)(unsigned)n;
    float acc = 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float d = __ldg(a + i) - __ldg(b + i);
        acc += log1pf(d * d * 12.5f) / nf;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane_id() == 0) s[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < kThreads / 32; ++w) t += s[w];
        partial[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(1024) cauchy_final_kernel(const float* __restrict__ partial, int n_partial, float* __restrict__ loss) {
    __shared__ float s[32];
    float acc = 0.0f;
    for (int i = threadIdx.x; i < n_partial; i += 1024) acc += partial[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane_id() == 0) s[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 32; ++w) t += s[w];
        *loss = t;
    }
}

// src/misc_kernels.cu:81-94
__global__ void __launch_bounds__(kThreads) cauchy_backward_kernel(const float* __restrict__ grad, const float* __restrict__ a,
                                                                   const float* __restrict__ b, int64_t n, float* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const float g = __ldg(grad);
    const float nf = (float)(unsigned)n;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float d = __ldg(a + i) - __ldg(b + i);
        const float denominator = nf * (12.5f * d * d + 1.0f);
        out[i] = 25.0f * d / fmaxf(denominator, 1.0e-12f) * g;
    }
}

constexpr int kCauchyMaxBlocks = 148 * 8;

// ---- per-leaf statistics of one step and the occupancy update (Modules/ProbabilityField.py:146-157) ----
// Blending weights are non-negative, so their bit patterns order like the values and integer atomic
// max reduces them exactly and in any order.  One 8-byte word per leaf {x: bits of the maximum,
// y: 0x7FFFFFFF - bits of the minimum}: both halves only ever grow, both reduce with MAX (also
// across ranks, as int32), one 8-byte read fetches both, and all-zero means "no sample", which the
// update reads as max = min = 0 (scatter_reduce with include_self=False on a zero tensor).
constexpr unsigned kMinFlip = 0x7FFFFFFFu;

__global__ void __launch_bounds__(kThreads) leaf_stats_kernel(const long long* __restrict__ indices, const float* __restrict__ weights,
                                                              int64_t n, int64_t n_leaves, uint2* __restrict__ stats) {
    // four samples per thread and round, their loads issued together: the kernel is bound by the latency of the
    // random reads of `stats`, not by bandwidth
    constexpr int kPer = 4;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; i0 < n; i0 += stride * kPer) {
        long long leaf[kPer];
        unsigned bits[kPer];
        uint2 cur[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int64_t i = i0 + k * stride;
            leaf[k] = i < n ? __ldg(indices + i) : -1;
            bits[k] = i < n ? __float_as_uint(fmaxf(__ldg(weights + i), 0.0f)) : 0u;
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            if (leaf[k] < 0 || leaf[k] >= n_leaves) leaf[k] = -1;
            cur[k] = leaf[k] >= 0 ? __ldcg(stats + leaf[k]) : make_uint2(0xFFFFFFFFu, 0xFFFFFFFFu);
        }
        // Both halves only grow, so a value that does not beat what a plain (possibly stale) read
        // returns cannot beat the current one either: most samples of a leaf that has already seen a
        // few skip both atomics.
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            if (leaf[k] < 0) continue;
            const unsigned flipped = kMinFlip - bits[k];
            if (bits[k] > cur[k].x) atomicMax(&stats[leaf[k]].x, bits[k]);
            if (flipped > cur[k].y) atomicMax(&stats[leaf[k]].y, flipped);
        }
    }
}

__global__ void __launch_bounds__(kThreads) leaf_update_kernel(float* __restrict__ leaf_weights, float* __restrict__ scores,
                                                               const uint2* __restrict__ stats, int64_t n_leaves, float decay) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t l = (int64_t)blockIdx.x * kThreads + threadIdx.x; l < n_leaves; l += stride) {
        const uint2 st = __ldg(stats + l);
        const float mx = __uint_as_float(st.x);
        const float mn = st.y == 0u ? 0.0f : __uint_as_float(kMinFlip - st.y);
        leaf_weights[l] = fmaxf(leaf_weights[l] * decay, mx);
        scores[l] = fmaxf(scores[l] * decay, __saturatef(mx - mn));
    }
}

// ---- image composition after the blend (Renderer.py:80 training, :105-122 inference) -------------
// Every product and sum is rounded on its own (__fmul_rn / __fadd_rn / __fdiv_rn keep the compiler
// from contracting them), as the chain of separate torch element-wise kernels it replaces does.

// out[c] = image[c] + (1 - alpha) * background[c]
__global__ void __launch_bounds__(kThreads) compose_background_kernel(const float* __restrict__ image, const float* __restrict__ alpha,
                                                                      const float* __restrict__ background, int channels, int64_t n_px,
                                                                      float* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x; p < n_px; p += stride) {
        const float t = __fsub_rn(1.0f, __ldg(alpha + p));
        for (int c = 0; c < channels; ++c) {
            const int64_t i = (int64_t)c * n_px + p;
            out[i] = __fadd_rn(__ldg(image + i), __fmul_rn(t, __ldg(background + i)));
        }
    }
}

// grad_alpha = -sum_c g[c] * background[c];  grad_background[c] = (1 - alpha) * g[c]   (grad_image = g)
__global__ void __launch_bounds__(kThreads) compose_background_backward_kernel(const float* __restrict__ grad_out, const float* __restrict__ alpha,
                                                                               const float* __restrict__ background, int channels,
                                                                               int64_t n_px, float* __restrict__ grad_alpha,
                                                                               float* __restrict__ grad_background) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x; p < n_px; p += stride) {
        const float t = 1.0f - __ldg(alpha + p);
        float dot = 0.0f;
        for (int c = 0; c < channels; ++c) {
            const int64_t i = (int64_t)c * n_px + p;
            const float g = __ldg(grad_out + i);
            if (grad_alpha) dot += g * __ldg(background + i);
            if (grad_background) grad_background[i] = t * g;
        }
        if (grad_alpha) grad_alpha[p] = -dot;
    }
}

// One multisample: acc (+)= sample, the features optionally divided by the sample's alpha first
// (Renderer.py:108-117).
__global__ void __launch_bounds__(kThreads) multisample_accumulate_kernel(float* __restrict__ acc_image, float* __restrict__ acc_depth,
                                                                          float* __restrict__ acc_alpha, const float* __restrict__ image,
                                                                          const float* __restrict__ depth, const float* __restrict__ alpha,
                                                                          int channels, int64_t n_px, bool first, bool unpremultiply) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x; p < n_px; p += stride) {
        const float a = __ldg(alpha + p);
        for (int c = 0; c < channels; ++c) {
            const int64_t i = (int64_t)c * n_px + p;
            float f = __ldg(image + i);
            if (unpremultiply) f = a > 0.0f ? __fdiv_rn(f, a) : 0.0f;
            acc_image[i] = first ? f : __fadd_rn(acc_image[i], f);
        }
        acc_depth[p] = first ? __ldg(depth + p) : __fadd_rn(acc_depth[p], __ldg(depth + p));
        acc_alpha[p] = first ? a : __fadd_rn(acc_alpha[p], a);
    }
}

// After the last multisample (Renderer.py:118-125): scale by 1/n, alpha_sum = clamp(sum of alphas),
// re-multiply by the mean alpha when the features were accumulated un-premultiplied, add the background.
__global__ void __launch_bounds__(kThreads) multisample_resolve_kernel(float* __restrict__ acc_image, float* __restrict__ acc_depth,
                                                                       float* __restrict__ acc_alpha, float* __restrict__ alpha_sum,
                                                                       const float* __restrict__ background, int channels, int64_t n_px,
                                                                       float factor, bool remultiply) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x; p < n_px; p += stride) {
        const float a_sum = acc_alpha[p];
        const float a = __fmul_rn(a_sum, factor);
        alpha_sum[p] = fminf(fmaxf(a_sum, 0.0f), 1.0f);
        acc_alpha[p] = a;
        acc_depth[p] = __fmul_rn(acc_depth[p], factor);
        const float t = __fsub_rn(1.0f, a);
        for (int c = 0; c < channels; ++c) {
            const int64_t i = (int64_t)c * n_px + p;
            float f = __fmul_rn(acc_image[i], factor);
            if (remultiply) f = __fmul_rn(f, a);
            if (background) f = __fadd_rn(f, __fmul_rn(t, __ldg(background + i)));
            acc_image[i] = f;
        }
    }
}

}  // namespace

}  // namespace inpc

using namespace inpc;

extern "C" int inpc_weight_decay_grads(const float* weights, float* grads, int64_t n, int add, void* stream_) {
    if (n == 0) return INPC_OK;
    if (n < 0 || n >= ((int64_t)1 << 32) || !weights || !grads) { set_error("inpc_weight_decay_grads: bad argument"); return INPC_E_INVALID; }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(weights) | reinterpret_cast<uintptr_t>(grads)) & 15u) == 0;
    const int grid = grid_for(n / 4 + 1);
    if (add) weight_decay_kernel<true><<<grid, kThreads, 0, stream>>>(weights, grads, n, vec_ok);
    else weight_decay_kernel<false><<<grid, kThreads, 0, stream>>>(weights, grads, n, vec_ok);
    INPC_LAUNCH_CHECK("weight_decay_kernel");
    return INPC_OK;
}

extern "C" int inpc_spherical_contraction(const float* positions, float* out, int64_t n, void* stream_) {
    if (n == 0) return INPC_OK;
    if (n < 0 || !positions || !out) { set_error("inpc_spherical_contraction: bad argument"); return INPC_E_INVALID; }
    contraction_kernel<<<grid_for(n), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(positions, out, n);
    INPC_LAUNCH_CHECK("contraction_kernel");
    return INPC_OK;
}

extern "C" size_t inpc_cauchy_workspace_bytes(int64_t n) { (void)n; return sizeof(float) * kCauchyMaxBlocks; }

extern "C" int inpc_cauchy_loss(const float* input, const float* target, int64_t n, float* loss, void* partials, void* stream_) {
    if (n <= 0 || n >= ((int64_t)1 << 32) || !input || !target || !loss || !partials) { set_error("inpc_cauchy_loss: bad argument"); return INPC_E_INVALID; }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int grid = grid_for(n);
    if (grid > kCauchyMaxBlocks) grid = kCauchyMaxBlocks;
    cauchy_partial_kernel<<<grid, kThreads, 0, stream>>>(input, target, n, static_cast<float*>(partials));
    INPC_LAUNCH_CHECK("cauchy_partial_kernel");
    cauchy_final_kernel<<<1, 1024, 0, stream>>>(static_cast<const float*>(partials), grid, loss);
    INPC_LAUNCH_CHECK("cauchy_final_kernel");
    return INPC_OK;
}

extern "C" int inpc_cauchy_loss_backward(const float* grad, const float* input, const float* target, int64_t n,
                                         float* grad_input, void* stream_) {
    if (n == 0) return INPC_OK;
    if (n < 0 || n >= ((int64_t)1 << 32) || !grad || !input || !target || !grad_input) { set_error("inpc_cauchy_loss_backward: bad argument"); return INPC_E_INVALID; }
    cauchy_backward_kernel<<<grid_for(n), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(grad, input, target, n, grad_input);
    INPC_LAUNCH_CHECK("cauchy_backward_kernel");
    return INPC_OK;
}

extern "C" int inpc_leaf_stats_reset(uint32_t* stats, int64_t n_leaves, void* stream_) {
    if (n_leaves == 0) return INPC_OK;
    if (n_leaves < 0 || !stats) { set_error("inpc_leaf_stats_reset: bad argument"); return INPC_E_INVALID; }
    INPC_CUDA_TRY(cudaMemsetAsync(stats, 0, 2 * sizeof(uint32_t) * (size_t)n_leaves, static_cast<cudaStream_t>(stream_)));
    return INPC_OK;
}

extern "C" int inpc_leaf_stats_accumulate(const int64_t* indices, const float* weights, int64_t n, uint32_t* stats, int64_t n_leaves,
                                          void* stream_) {
    if (n == 0) return INPC_OK;
    if (n < 0 || n_leaves <= 0 || !indices || !weights || !stats || (reinterpret_cast<uintptr_t>(stats) & 7u)) {
        set_error("inpc_leaf_stats_accumulate: bad argument");
        return INPC_E_INVALID;
    }
    leaf_stats_kernel<<<grid_for(n), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(reinterpret_cast<const long long*>(indices), weights, n, n_leaves,
                                                                                     reinterpret_cast<uint2*>(stats));
    INPC_LAUNCH_CHECK("leaf_stats_kernel");
    return INPC_OK;
}

extern "C" int inpc_leaf_update(float* leaf_weights, float* leaf_subdivision_scores, const uint32_t* stats, int64_t n_leaves, float decay,
                                void* stream_) {
    if (n_leaves == 0) return INPC_OK;
    if (n_leaves < 0 || !leaf_weights || !leaf_subdivision_scores || !stats || (reinterpret_cast<uintptr_t>(stats) & 7u)) {
        set_error("inpc_leaf_update: bad argument");
        return INPC_E_INVALID;
    }
    leaf_update_kernel<<<grid_for(n_leaves), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(leaf_weights, leaf_subdivision_scores,
                                                                                             reinterpret_cast<const uint2*>(stats), n_leaves, decay);
    INPC_LAUNCH_CHECK("leaf_update_kernel");
    return INPC_OK;
}

extern "C" int inpc_compose_background(const float* image, const float* alpha, const float* background, int channels, int64_t n_pixels,
                                       float* out, void* stream_) {
    if (n_pixels == 0 || channels == 0) return INPC_OK;
    if (n_pixels < 0 || channels < 0 || !image || !alpha || !background || !out) { set_error("inpc_compose_background: bad argument"); return INPC_E_INVALID; }
    compose_background_kernel<<<grid_for(n_pixels), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(image, alpha, background, channels, n_pixels, out);
    INPC_LAUNCH_CHECK("compose_background_kernel");
    return INPC_OK;
}

extern "C" int inpc_compose_background_backward(const float* grad_out, const float* alpha, const float* background, int channels,
                                                int64_t n_pixels, float* grad_alpha, float* grad_background, void* stream_) {
    if (n_pixels == 0 || channels == 0 || (!grad_alpha && !grad_background)) return INPC_OK;
    if (n_pixels < 0 || channels < 0 || !grad_out || !alpha || (grad_alpha && !background)) { set_error("inpc_compose_background_backward: bad argument"); return INPC_E_INVALID; }
    compose_background_backward_kernel<<<grid_for(n_pixels), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(grad_out, alpha, background, channels,
                                                                                                             n_pixels, grad_alpha, grad_background);
    INPC_LAUNCH_CHECK("compose_background_backward_kernel");
    return INPC_OK;
}

extern "C" int inpc_multisample_accumulate(float* acc_image, float* acc_depth, float* acc_alpha, const float* image, const float* depth,
                                           const float* alpha, int channels, int64_t n_pixels, int first, int unpremultiply, void* stream_) {
    if (n_pixels == 0) return INPC_OK;
    if (n_pixels < 0 || channels < 0 || !acc_image || !acc_depth || !acc_alpha || !image || !depth || !alpha) { set_error("inpc_multisample_accumulate: bad argument"); return INPC_E_INVALID; }
    multisample_accumulate_kernel<<<grid_for(n_pixels), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(acc_image, acc_depth, acc_alpha, image, depth, alpha,
                                                                                                        channels, n_pixels, first != 0, unpremultiply != 0);
    INPC_LAUNCH_CHECK("multisample_accumulate_kernel");
    return INPC_OK;
}

extern "C" int inpc_multisample_resolve(float* acc_image, float* acc_depth, float* acc_alpha, float* alpha_sum, const float* background,
                                        int channels, int64_t n_pixels, int n_multisamples, int remultiply, void* stream_) {
    if (n_pixels == 0) return INPC_OK;
    if (n_pixels < 0 || channels < 0 || n_multisamples < 1 || !acc_image || !acc_depth || !acc_alpha || !alpha_sum) { set_error("inpc_multisample_resolve: bad argument"); return INPC_E_INVALID; }
    // the factor is the double-precision 1/n rounded to float once, as a python float times an fp32 tensor is
    const float factor = (float)(1.0 / (double)n_multisamples);
    multisample_resolve_kernel<<<grid_for(n_pixels), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(acc_image, acc_depth, acc_alpha, alpha_sum, background,
                                                                                                     channels, n_pixels, factor, remultiply != 0);
    INPC_LAUNCH_CHECK("multisample_resolve_kernel");
    return INPC_OK;
}
