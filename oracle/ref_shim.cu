// TEST INFRASTRUCTURE — not part of the product.
//
// C-ABI shim around the *unmodified* native layer of the reference CUDA backend
// (INPCCudaBackend/INPCCudaBackend/{rasterization,sampling,misc}).  The reference
// sources are compiled where they lie (oracle/Makefile, target `ref`); nothing of them
// is copied here.  This file only supplies what the reference's torch wrappers
// supply (INPCCudaBackend/INPCCudaBackend/rasterization/src/rasterization_api.cu:23-367,
// sampling/src/sampling_api.cu:9-240, misc/src/misc_api.cu:7-83): output zero-fill,
// grow-only scratch blobs standing in for torch's caching allocator, and pointer
// unwrapping.  It is used by the GPU parity tests, by the golden-vector generator
// and by the reference arm of the benchmark.  The product never loads it.
#include "bilinear/forward.h"
#include "bilinear/backward.h"
#include "bilinear/inference.h"
#include "bilinear/inference_preextracted.h"
#include "bilinear/buffer_utils.h"
#include "gaussian/forward.h"
#include "gaussian/backward.h"
#include "gaussian/inference.h"
#include "gaussian/inference_preextracted.h"
#include "rasterization_utils.h"
#include "sampling.h"
#include "misc.h"
#include "pcg32.h"
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <functional>

namespace {

struct Blob {
    char* ptr = nullptr;
    size_t cap = 0;
    size_t used = 0;
    char* grow(size_t n) {
        used = n;
        if (n > cap) {
            if (ptr) cudaFree(ptr);
            cap = n + n / 4 + 4096;
            if (cudaMalloc(&ptr, cap) != cudaSuccess) { ptr = nullptr; cap = 0; }
        }
        return ptr;
    }
};

Blob g_prim, g_tile, g_inst, g_sum, g_misc;
int g_n_instances = 0, g_selector = 0, g_n_primitives = 0, g_mode = 0;
pcg32 g_rng(0);

std::function<char*(size_t)> grower(Blob& b) { return [&b](size_t n) { return b.grow(n); }; }

int last_error() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { fprintf(stderr, "[ref_shim] CUDA error: %s\n", cudaGetErrorString(e)); return (int)e; }
    e = cudaGetLastError();
    return (int)e;
}

}  // namespace

extern "C" {

// forward_wrapper equivalent (rasterization_api.cu:23-107). No device synchronisation
// beyond what the reference performs itself; call inpcref_sync() to check errors.
int inpcref_forward(int mode, const float* positions, const void* features, const float* opacities,
                    const float* w2c, const float* cam_position, float* image, float* alpha,
                    float* blending_weights, int n, int width, int height, float fx, float fy,
                    float cx, float cy, float near_plane, float far_plane) {
    cudaMemsetAsync(blending_weights, 0, sizeof(float) * (size_t)n, 0);
    std::pair<int, int> st;
    g_mode = mode;
    g_n_primitives = n;
    if (mode == 0)
        st = inpc::rasterization::bilinear::forward(grower(g_prim), grower(g_tile), grower(g_inst),
            (const float3*)positions, (const half4*)features, opacities, (const float4*)w2c,
            (const float3*)cam_position, image, alpha, blending_weights, n, width, height, fx, fy, cx, cy,
            near_plane, far_plane);
    else if (mode == 1)
        st = inpc::rasterization::gaussian::forward(grower(g_prim), grower(g_tile), grower(g_inst),
            (const float3*)positions, (const half4*)features, opacities, (const float4*)w2c,
            (const float3*)cam_position, image, alpha, blending_weights, n, width, height, fx, fy, cx, cy,
            near_plane, far_plane);
    else
        return -1;
    g_n_instances = st.first;
    g_selector = st.second;
    return 0;
}

// backward_wrapper equivalent (rasterization_api.cu:109-190): zero-fills the three
// gradient tensors, then runs the reference backward on the blobs of the last forward.
int inpcref_backward(int mode, const float* grad_image, const float* grad_alpha, const float* image,
                     const float* alpha, const float* positions, const float* opacities,
                     const float* cam_position, float* grad_features_view, void* grad_features,
                     float* grad_opacities, int n, int width, int height) {
    cudaMemsetAsync(grad_features_view, 0, sizeof(float) * 4 * (size_t)n, 0);
    cudaMemsetAsync(grad_features, 0, 2 * 36 * (size_t)n, 0);
    cudaMemsetAsync(grad_opacities, 0, sizeof(float) * (size_t)n, 0);
    if (mode == 0)
        inpc::rasterization::bilinear::backward(grad_image, grad_alpha, image, alpha, (const float3*)positions,
            opacities, (const float3*)cam_position, g_prim.ptr, g_tile.ptr, g_inst.ptr,
            (float4*)grad_features_view, (half4*)grad_features, grad_opacities, n, width, height,
            g_n_instances, g_selector);
    else if (mode == 1)
        inpc::rasterization::gaussian::backward(grad_image, grad_alpha, image, alpha, (const float3*)positions,
            opacities, (const float3*)cam_position, g_prim.ptr, g_tile.ptr, g_inst.ptr,
            (float4*)grad_features_view, (half4*)grad_features, grad_opacities, n, width, height,
            g_n_instances, g_selector);
    else
        return -1;
    return 0;
}

// inference_wrapper equivalent (rasterization_api.cu:192-276); features_raw is (n,37) fp16.
int inpcref_render(int mode, const float* positions, const void* features_raw, const float* w2c,
                   const float* cam_position, float* image, float* depth, float* alpha, int n, int width,
                   int height, float fx, float fy, float cx, float cy, float near_plane, float far_plane,
                   float sigma_world, float sigma_cutoff) {
    g_mode = mode;
    g_n_primitives = n;
    if (mode == 0)
        inpc::rasterization::bilinear::inference(grower(g_prim), grower(g_tile), grower(g_inst),
            (const float3*)positions, (const __half*)features_raw, (const float4*)w2c,
            (const float3*)cam_position, image, depth, alpha, n, width, height, fx, fy, cx, cy, near_plane,
            far_plane);
    else if (mode == 1)
        inpc::rasterization::gaussian::inference(grower(g_prim), grower(g_tile), grower(g_inst),
            (const float3*)positions, (const __half*)features_raw, (const float4*)w2c,
            (const float3*)cam_position, image, depth, alpha, n, width, height, fx, fy, cx, cy, near_plane,
            far_plane, sigma_world, sigma_cutoff);
    else
        return -1;
    return 0;
}

// inference_preextracted_wrapper equivalent (rasterization_api.cu:278-367); scales may be null.
int inpcref_render_preextracted(int mode, const float* positions, const void* features,
                                const float* opacities, const float* scales, const float* w2c,
                                const float* cam_position, float* image, float* depth, float* alpha, int n,
                                int width, int height, float fx, float fy, float cx, float cy,
                                float near_plane, float far_plane, float sigma_world, float sigma_cutoff) {
    g_mode = mode;
    g_n_primitives = n;
    if (mode == 0)
        inpc::rasterization::bilinear::inference_preextracted(grower(g_prim), grower(g_tile), grower(g_inst),
            (const float3*)positions, (const half4*)features, opacities, (const float4*)w2c,
            (const float3*)cam_position, image, depth, alpha, n, width, height, fx, fy, cx, cy, near_plane,
            far_plane);
    else if (mode == 1)
        inpc::rasterization::gaussian::inference_preextracted(grower(g_prim), grower(g_tile), grower(g_inst),
            (const float3*)positions, (const half4*)features, opacities, scales, (const float4*)w2c,
            (const float3*)cam_position, image, depth, alpha, n, width, height, fx, fy, cx, cy, near_plane,
            far_plane, sigma_world, sigma_cutoff);
    else
        return -1;
    return 0;
}

int inpcref_sync(void) { return last_error(); }

// blocking device-to-host copy, so that tests can read the intermediate buffers without another
// CUDA binding
int inpcref_copy_to_host(void* dst, const void* src, size_t bytes) {
    return (int)cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost);
}

int inpcref_n_instances(void) { return g_n_instances; }

// Intermediate buffers of the last bilinear/gaussian *training* forward, resolved with the
// reference's own carving code (bilinear/buffer_utils.h:24-115).  which:
//   0 depth keys buffer A   1 depth keys buffer B   2 primitive indices A   3 primitive indices B
//   4 n_touched_tiles       5 screen_bounds (ushort4) 6 screen_coords (float2)
//   7 features_view (float4) 8 depth (float)        9 n_visible (uint)   10 n_instances (uint)
//  11 instance ranges (uint2 per tile)  12 sorted instance primitive indices (selected buffer)
//  13 sorted instance keys buffer A     14 sorted instance keys buffer B
// Only valid for mode 0 (the gaussian blob has one more array); returns null otherwise.
void* inpcref_intermediate(int which, int width, int height) {
    using namespace inpc::rasterization::bilinear;
    if (g_mode != 0 || !g_prim.ptr) return nullptr;
    char* b = g_prim.ptr;
    PerPrimitiveBuffers pp = PerPrimitiveBuffers::from_blob(b, g_n_primitives);
    const int gw = (width + 7) / 8, gh = (height + 7) / 8;
    switch (which) {
        case 0: return pp.depth_keys.d_buffers[0];
        case 1: return pp.depth_keys.d_buffers[1];
        case 2: return pp.primitive_indices.d_buffers[0];
        case 3: return pp.primitive_indices.d_buffers[1];
        case 4: return pp.n_touched_tiles;
        case 5: return pp.screen_bounds;
        case 6: return pp.screen_coords;
        case 7: return pp.features_view;
        case 8: return pp.depth;
        case 9: return pp.n_visible_primitives;
        case 10: return pp.n_instances;
        default: break;
    }
    if (which == 11) {
        char* t = g_tile.ptr;
        return PerTileBuffers::from_blob(t, gw * gh).instance_ranges;
    }
    if (which >= 12 && which <= 14 && g_inst.ptr) {
        char* i = g_inst.ptr;
        const int end_bit = extract_end_bit((uint)(gw * gh - 1));
        PerInstanceBuffers pi = PerInstanceBuffers::from_blob(i, g_n_instances, end_bit);
        if (which == 12) return pi.primitive_indices.d_buffers[g_selector];
        return pi.keys.d_buffers[which - 13];
    }
    return nullptr;
}

// ---- sampler (sampling/src/sampling_api.cu:9-240) ----------------------------------------

void inpcref_sampler_seed(long long seed) { g_rng = pcg32((uint64_t)seed); }

int inpcref_viewpoint_weights(const float* centers, const int* levels, const float* weights,
                              const float* w2c, float* out, unsigned n_cells, unsigned width,
                              unsigned height, float fx, float fy, float cx, float cy, float near_plane,
                              float far_plane, float initial_size) {
    inpc::sampling::compute_viewpoint_weights((const float3*)centers, levels, weights, (const float4*)w2c,
        out, n_cells, width, height, fx, fy, cx, cy, near_plane, far_plane, initial_size);
    return 0;
}

// viewpoint_weights (n_cells floats, receives the CDF), weights_sum (1 float) and counter (1 int)
// are caller-provided scratch, as the torch wrapper allocates them per call.
int inpcref_training_samples(const float* centers, const int* levels, const float* weights,
                             const float* w2c, float* viewpoint_weights, float* weights_sum,
                             float* positions, long long* indices, int* counter, unsigned n_cells,
                             unsigned n_samples, unsigned width, unsigned height, float fx, float fy,
                             float cx, float cy, float near_plane, float far_plane, float initial_size) {
    cudaMemsetAsync(counter, 0, sizeof(int), 0);
    inpc::sampling::create_training_samples(grower(g_sum), (const float3*)centers, levels, weights,
        (const float4*)w2c, viewpoint_weights, weights_sum, (float3*)positions, (int64_t*)indices, counter,
        n_cells, n_samples, width, height, fx, fy, cx, cy, near_plane, far_plane, initial_size, g_rng);
    return 0;
}

// generate_samples_wrapper equivalent; returns the number of samples written (0 if the weight sum <= 0).
int inpcref_samples(const float* centers, const int* levels, const float* weights, const float* w2c,
                    float* viewpoint_weights, float* weights_sum, float* positions, unsigned n_cells,
                    unsigned n_samples, unsigned width, unsigned height, float fx, float fy, float cx,
                    float cy, float near_plane, float far_plane, float initial_size) {
    inpc::sampling::compute_viewpoint_weights((const float3*)centers, levels, weights, (const float4*)w2c,
        viewpoint_weights, n_cells, width, height, fx, fy, cx, cy, near_plane, far_plane, initial_size);
    if (!inpc::sampling::compute_cdf(grower(g_sum), viewpoint_weights, weights_sum, n_cells)) return 0;
    inpc::sampling::create_samples((const float3*)centers, levels, viewpoint_weights, (float3*)positions,
        n_samples, n_cells, initial_size, g_rng);
    return (int)n_samples;
}

// generate_expected_samples_wrapper equivalent, split in two so the caller can size the output:
// phase 1 returns n_created (0 if the weight sum <= 0); phase 2 fills n_created*n_multi positions.
int inpcref_expected_samples_count(const float* centers, const int* levels, const float* weights,
                                   const float* w2c, float* viewpoint_weights, float* weights_sum,
                                   unsigned n_cells, unsigned n_samples, unsigned width, unsigned height,
                                   float fx, float fy, float cx, float cy, float near_plane, float far_plane,
                                   float initial_size) {
    inpc::sampling::compute_viewpoint_weights((const float3*)centers, levels, weights, (const float4*)w2c,
        viewpoint_weights, n_cells, width, height, fx, fy, cx, cy, near_plane, far_plane, initial_size);
    return (int)inpc::sampling::compute_sample_distribution(grower(g_sum), viewpoint_weights, weights_sum,
        n_samples, n_cells);
}

int inpcref_expected_samples_fill(const float* centers, const int* levels, int* cell_indices,
                                  float* positions, unsigned n_created, unsigned n_multi, unsigned n_cells,
                                  float initial_size) {
    inpc::sampling::create_expected_samples((const float3*)centers, levels, g_sum.ptr, cell_indices,
        (float3*)positions, n_created * n_multi, n_created, n_cells, initial_size, g_rng);
    return 0;
}

// ---- misc (misc/src/misc_api.cu:7-83) -----------------------------------------------------

int inpcref_weight_decay(const float* weights, float* grads, unsigned n, int add) {
    if (add) inpc::misc::add_normalized_weight_decay_grads(weights, grads, n);
    else inpc::misc::compute_normalized_weight_decay_grads(weights, grads, n);
    return 0;
}

int inpcref_contraction(const float* positions, float* out, unsigned n) {
    if (n) inpc::misc::spherical_contraction((const float3*)positions, (float3*)out, n);
    return 0;
}

int inpcref_cauchy(const float* input, const float* target, float* elementwise, unsigned n) {
    inpc::misc::cauchy_loss(input, target, elementwise, n);
    return 0;
}

int inpcref_cauchy_backward(const float* grad, const float* input, const float* target, float* grad_input,
                            unsigned n) {
    inpc::misc::cauchy_loss_backward(grad, input, target, grad_input, n);
    return 0;
}

}  // extern "C"
