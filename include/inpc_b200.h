/*
 * inpc_b200 — C ABI of the B200-native (sm_100a) replacement for the INPC CUDA backend.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, i.e. a
 * cudaStream_t; NULL is the legacy default stream).  No torch types cross this boundary.  All
 * functions return 0 on success or a negative INPC_E_* code; inpc_last_error() returns a message
 * for the last failure on the calling thread.  Unless stated otherwise a call only enqueues work
 * on `stream` and returns; the few calls that must read a count back say so.
 *
 * Each declaration cites the interface of the reference project it replaces, as
 * path:line below INPCCudaBackend/INPCCudaBackend/ of nerficg-project/INPC.
 */
#ifndef INPC_B200_H
#define INPC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INPC_OK 0
#define INPC_E_INVALID (-1)   /* bad argument (mode, tile size, null pointer, size out of range) */
#define INPC_E_CUDA (-2)      /* a CUDA runtime call failed; message has the CUDA error string */
#define INPC_E_ALLOC (-3)     /* the allocator callback returned NULL */
#define INPC_E_DEVICE (-4)    /* a kernel reported a failed internal check (bounded wait ran out) */
#define INPC_E_CAPACITY (-5)  /* size beyond a fixed capacity of the called entry point */

#define INPC_MODE_BILINEAR 0
#define INPC_MODE_GAUSSIAN 1

/* Scratch allocator: returns a device pointer to at least `bytes` bytes (256-byte aligned), valid
 * until the matching backward has run.  Replaces the three std::function<char*(size_t)> resize
 * callbacks of rasterization/include/bilinear/forward.h:11-13 (torch_utils.h:6-11). */
typedef void* (*inpc_alloc_fn)(void* user, size_t bytes);

/* Pinhole camera and raster parameters.  `w2c` and `cam_position` stay device pointers exactly as
 * in the reference (rows 0..2 of a row-major 4x4 float matrix; 3 floats).  Mirrors the scalar tail
 * of rasterization/include/bilinear/forward.h:22-30 and RasterizerSettings.as_tuple()
 * (torch_bindings/rasterization.py:20-46). */
typedef struct inpc_view {
    const float* w2c;           /* device, 16 floats */
    const float* cam_position;  /* device, 3 floats */
    int32_t width, height;
    float fx, fy, cx, cy;
    float near_plane, far_plane;
} inpc_view;

/* What forward hands to backward; plain data, no ownership.  Replaces the (n_instances, selector)
 * pair plus the three blob base pointers the reference keeps on the autograd context
 * (torch_bindings/rasterization.py:62-74). */
typedef struct inpc_raster_state {
    void* point_blob;     /* per-point scratch from alloc_point */
    void* instance_blob;  /* per-instance + per-tile scratch from alloc_instance */
    int64_t n_points;
    int64_t n_visible;        /* -1 while the count is still on the device (deferred_counts), see inpc_raster_resolve */
    int64_t n_instances;      /* likewise */
    int32_t tile_size;
    int32_t mode;
    uint32_t depth_key_base;  /* depth bit pattern the sort keys are offsets from: the smallest visible one, or the near plane's when the counts are deferred */
    int32_t depth_key_bits;   /* significant bits of the largest offset */
    int32_t channels;         /* blended channels: 4 for the spherical-harmonics layout, else the feature-row width */
    int32_t deferred_counts;  /* 1: no count was read back; scratch is sized for 4 instances per point */
} inpc_raster_state;

const char* inpc_last_error(void);
/* Library/ABI version as major*10000 + minor*100 + patch. */
int inpc_version(void);

/* Number of kernels this library has launched in the process so far. */
long long inpc_launch_count(void);

/* Per-stage device timing with CUDA events on the caller's stream; off by default.  Stages:
 * 0 sample | 1 preprocess | 2 depth sort | 3 instance emission | 4 tile sort + ranges | 5 blend
 * forward | 6 blend backward | 7 preprocess backward.  inpc_profile_read waits for the recorded
 * events, adds them to running totals and copies min(n, 8) totals (milliseconds, number of timed
 * scopes) out; `reset` != 0 clears the totals afterwards.  Stands in for the reference's only
 * profiling aid, the -lineinfo switch of INPCCudaBackend/setup.py:11,32-33. */
int inpc_profile_enable(int on);
int inpc_profile_read(double* stage_ms, long long* stage_calls, int n, int reset);

/* Device-side status of a call.  A few kernels wait on one another or on a copy engine; every such wait is
 * bounded, and a kernel that gives up stores a flag into the status words of ITS call (words: 0 a
 * radix-sort tile gave up its look-back | 1 some rejection-sampler slots ran out of attempts
 * (informational) | 2 a block gave up waiting for its bulk copy | 3 checked build: a gather index was out
 * of range).  Every entry point that launches such kernels takes a ticket; inpc_last_call_ticket returns
 * the one the calling host thread took last, inpc_call_status copies the four words of a ticket out
 * (`words` may be NULL) and returns INPC_E_DEVICE with a message naming the entry point if words 0, 2 or 3
 * are set, INPC_E_INVALID if the ticket is unknown or older than 1024 calls.  The words live in mapped
 * host memory: reading them needs no device synchronisation, but they are final only once the call's
 * stream has been synchronised.  Independently of this, each entry point first looks at the last eight
 * tickets of its host thread and returns INPC_E_DEVICE if one of them has reported since.
 * The reference has no counterpart (its only check is the debug macro of utils/utils.h:10-17). */
long long inpc_last_call_ticket(void);
int inpc_call_status(long long ticket, unsigned* words);

/* ------------------------------------------------------------------------------------------
 * Rasterizer
 * ---------------------------------------------------------------------------------------- */

/* Training forward: cull/project/SH-evaluate, order by (tile, depth), blend front to back.
 *   positions (n,3) f32 | features (n,36) f16, coefficient-major channel-minor | opacities (n) f32
 *   image (4,H,W) f32 | alpha (H,W) f32 | blending_weights (n) f32 — all three fully written.
 * tile_size is 8 (the reference's tiling; tile ranges comparable with it) or 16.
 * Bilinear mode with 8x8 tiles makes no host synchronisation at all: a splat touches at most 2x2 tiles, so the
 * instance scratch is sized for 4 n instances, the kernels read the two counts from device memory, and
 * state->n_visible / n_instances stay -1 until inpc_raster_resolve is called.  The other combinations read
 * the two counters back once to size the instance scratch (the reference does so twice, with blocking copies:
 * rasterization/src/bilinear/forward.cu:86-89).
 * Replaces inpc::rasterization::{bilinear,gaussian}::forward
 * (rasterization/include/bilinear/forward.h:10-30, gaussian/forward.h:10-30) together with the
 * output zero-fill of forward_wrapper (rasterization/src/rasterization_api.cu:44-46). */
int inpc_rasterize_forward(int mode, int tile_size, const inpc_view* view, int64_t n,
                           const float* positions, const void* features, const float* opacities,
                           float* image, float* alpha, float* blending_weights,
                           inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user,
                           inpc_raster_state* state, void* stream);

/* Training backward for the forward that produced `state`.
 *   grad_image (4,H,W), grad_alpha (H,W), image, alpha: as returned by / upstream of forward
 *   grad_features (n,36) f16 and grad_opacities (n) f32 — fully written (zero rows for culled points)
 *   grad_features_view (n,33) f32, 32-byte aligned — caller scratch: per point four 32-byte slot records
 *     (4 feature + 1 opacity gradient sums) plus one mask word.  A splat's pixels lie in at most four (tile, half-tile) parts; every part stores
 *     its sums into the slot that is its own by construction and the per-point pass adds the written slots in
 *     fixed order, so bilinear gradients on 8x8 tiles involve no floating-point atomics and are bit-identical
 *     from run to run (the reference adds five float atomics per fragment, bilinear/kernels.cu:392-415).  The
 *     other paths use the first (n,4) floats as an atomic accumulation buffer.
 * Replaces inpc::rasterization::{bilinear,gaussian}::backward
 * (rasterization/include/bilinear/backward.h:8-26) together with the three zero-fills of
 * backward_wrapper (rasterization/src/rasterization_api.cu:138-140). */
int inpc_rasterize_backward(const inpc_raster_state* state, const inpc_view* view,
                            const float* grad_image, const float* grad_alpha, const float* image,
                            const float* alpha, const float* positions, const float* opacities,
                            float* grad_features_view, void* grad_features, float* grad_opacities,
                            void* stream);

/* Inference from raw network output: features_raw (n,37) f16 = [opacity logit, 36 SH halves];
 * opacity = 1 - exp(-exp(raw)).  Writes image (4,H,W), depth (H,W), alpha (H,W).
 * sigma_world / sigma_cutoff are used by the gaussian mode only.
 * Replaces inpc::rasterization::{bilinear,gaussian}::inference
 * (rasterization/include/bilinear/inference.h:9-28, gaussian/inference.h:9-30). */
int inpc_render(int mode, int tile_size, const inpc_view* view, int64_t n, const float* positions,
                const void* features_raw, float sigma_world, float sigma_cutoff, float* image,
                float* depth, float* alpha, inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance,
                void* alloc_user, void* stream);

/* Batched inference over several sample sets of one view (bilinear splats, 8x8 tiles): set j = positions[j] (n_points[j],3)
 * f32 and features_raw[j] (n_points[j],37) f16, drawn into images[j] (4,H,W), depths[j] (H,W), alphas[j] (H,W) of the three
 * contiguous output arrays -- bit for bit what n_sets calls of inpc_render give, from ONE launch sequence: the sets are
 * culled and projected together, sorted together (a set's tiles are rows of a stacked tile grid, so the set index rides in
 * the tile key) and blended together.  n_sets <= 8; no host synchronisation.  Replaces the loop over
 * rasterizer.render of the reference's multisampled and ring-buffer inference (Renderer.py:99-125, :139-166,
 * utils.py:145-174). */
int inpc_render_multi(int tile_size, const inpc_view* view, int n_sets, const int64_t* n_points,
                      const float* const* positions, const void* const* features_raw, float* images, float* depths,
                      float* alphas, inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user,
                      void* stream);

/* Inference from a pre-extracted point cloud; `scales` (n) f32 may be NULL (gaussian mode then uses
 * sigma_world for every point).
 * Replaces inpc::rasterization::{bilinear,gaussian}::inference_preextracted
 * (rasterization/include/bilinear/inference_preextracted.h:9-29,
 *  gaussian/inference_preextracted.h:9-32). */
int inpc_render_preextracted(int mode, int tile_size, const inpc_view* view, int64_t n,
                             const float* positions, const void* features, const float* opacities,
                             const float* scales, float sigma_world, float sigma_cutoff, float* image,
                             float* depth, float* alpha, inpc_alloc_fn alloc_point,
                             inpc_alloc_fn alloc_instance, void* alloc_user, void* stream);

/* Feature-row layout (bilinear splats): every point carries `channels` fp32 values (4, 8, 16 or 32;
 * features (n, channels), 16-byte aligned) that are blended as they are, without spherical
 * harmonics, into image (channels,H,W).  alpha (H,W), blending_weights (n), the scratch callbacks
 * and `state` are as in inpc_rasterize_forward.
 * No counterpart in the reference, whose backend only blends the four channels it evaluates from 36
 * SH halves (rasterization/src/rasterization_api.cu:23-107): the ordering is that of
 * rasterization/src/bilinear/forward.cu:59-170 and the per-fragment arithmetic that of
 * rasterization/src/bilinear/kernels.cu:241-313 with the channel count as a parameter, so that a
 * channels/4-fold run of the reference on DC-only coefficients gives the same image. */
int inpc_rasterize_rows_forward(int tile_size, const inpc_view* view, int64_t n, const float* positions,
                                const float* features, int channels, const float* opacities, float* image,
                                float* alpha, float* blending_weights, inpc_alloc_fn alloc_point,
                                inpc_alloc_fn alloc_instance, void* alloc_user, inpc_raster_state* state,
                                void* stream);

/* Backward of inpc_rasterize_rows_forward: grad_image (channels,H,W), grad_alpha (H,W);
 * grad_features (n, channels) f32 and grad_opacities (n) f32 are fully written (zero rows for
 * culled points).  Arithmetic of rasterization/src/bilinear/kernels.cu:315-420 per channel. */
int inpc_rasterize_rows_backward(const inpc_raster_state* state, const inpc_view* view,
                                 const float* grad_image, const float* grad_alpha, const float* image,
                                 const float* alpha, const float* features, float* grad_features,
                                 float* grad_opacities, void* stream);

/* Inference over feature rows: image (channels,H,W), expected depth (H,W), alpha (H,W)
 * (rasterization/src/bilinear/kernels.cu:422-495 with the channel count as a parameter). */
int inpc_render_rows(int tile_size, const inpc_view* view, int64_t n, const float* positions,
                     const float* features, int channels, const float* opacities, float* image, float* depth,
                     float* alpha, inpc_alloc_fn alloc_point, inpc_alloc_fn alloc_instance, void* alloc_user,
                     void* stream);

/* Fills in state->n_visible, n_instances and depth_key_base of a forward that deferred them: one small
 * device-to-host copy on `stream` and a synchronisation of that stream.  A no-op for states whose counts were
 * read back by the forward itself.  The values the reference returns from its blocking copies at
 * rasterization/src/bilinear/forward.cu:86-89. */
int inpc_raster_resolve(inpc_raster_state* state, void* stream);

/* Introspection for parity tests: copies one intermediate array of the forward that produced
 * `state` into `dst` (device pointer, caller-sized).  which: 0 sorted visible point ids (n_visible
 * u32) | 1 sorted depth keys (n_visible u32) | 2 sorted instance point ids (n_instances u32) |
 * 3 tile ranges (2 u32 per tile) | 4 tiles touched per point (n u32) | 5 screen xy (n,2 f32) |
 * 6 depth (n f32) | 7 view-space feature (n,4 f32) | 8 tile bounds x0,x1,y0,y1 (n,4 u16).
 * These are the arrays the reference keeps in PerPrimitiveBuffers / PerInstanceBuffers /
 * PerTileBuffers (rasterization/include/bilinear/buffer_utils.h:24-115). */
int inpc_raster_debug_copy(const inpc_raster_state* state, const inpc_view* view, int which, void* dst,
                           void* stream);

/* Stable least-significant-digit radix sort of (u32 key, u32 value) pairs on bits [0, end_bit),
 * the library's own onesweep.  keys_alt / values_alt are same-sized ping-pong buffers; `workspace`
 * needs inpc_sort_workspace_bytes(n).  *result_in_alt tells which pair holds the result.
 * Replaces the two cub::DeviceRadixSort::SortPairs calls of
 * rasterization/src/bilinear/forward.cu:91-98 and :132-139. */
size_t inpc_sort_workspace_bytes(int64_t n);
int inpc_sort_pairs(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n,
                    int end_bit, void* workspace, int* result_in_alt, void* stream);

/* The same sort for callers that cannot allocate device memory: hosts that run inside someone
 * else's memory budget — an engine plugin handed a fixed arena, a real-time loop where cudaMalloc's
 * implicit synchronisation is not acceptable, a process whose allocator is owned by another
 * framework and must not see foreign allocations.  It takes no workspace argument: its scratch is a
 * fixed array inside the library's device image (about 1 MB, held by every GPU that loads the
 * library until the process exits), and it makes no cudaMalloc / cudaFree / allocating call of any
 * kind, torch's included.  Inputs and outputs are still the caller's.
 *   - Capacity: n <= 1,048,576 pairs; larger n returns INPC_E_CAPACITY with a message.
 *   - The first call on a device resolves the array's device address (once per device, with that
 *     device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array, which still holds the previous call's histograms
 *     and flags; each call clears what it reads, on `stream`.  Two calls whose work overlaps on the
 *     GPU (different streams, no ordering) race on it: serialise them.
 *   - A look-back wait that runs out is recorded inside the array (reporting through pinned memory would
 *     be an allocation); the wait stays bounded.  inpc_sort_pairs_static_status synchronises `stream`,
 *     copies the status words of the last call on the current device out (see inpc_call_status for
 *     their meaning) and returns INPC_E_DEVICE if the look-back word is set; it allocates nothing either.
 * This entry point has no counterpart in the reference. */
int inpc_sort_pairs_static(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt, int64_t n,
                           int end_bit, int* result_in_alt, void* stream);
int inpc_sort_pairs_static_status(void* stream, unsigned* words);

/* Test hook for the bounded look-back wait: inpc_sort_pairs with tile 0 of every pass leaving before it
 * publishes its digit counts and a wait limit of 2^10 polls.  The tiles behind it give up within
 * microseconds, set word 0 of the call's status and finish; every access stays inside the buffers, the
 * output is simply not sorted.  *ticket receives the call's status ticket.  This hook has no counterpart
 * in the reference (cub's look-back spins without a limit). */
int inpc_debug_sort_lookback_timeout(uint32_t* keys, uint32_t* keys_alt, uint32_t* values, uint32_t* values_alt,
                                     int64_t n, int end_bit, void* workspace, long long* ticket, void* stream);

/* ------------------------------------------------------------------------------------------
 * Probability-field sampler
 * ---------------------------------------------------------------------------------------- */

/* Per-leaf sampling weight for one viewpoint.  centers (L,3) f32, levels (L) i32, weights (L) f32,
 * out (L) f32.  Replaces inpc::sampling::compute_viewpoint_weights (sampling/include/sampling.h:11-26). */
int inpc_compute_viewpoint_weights(const inpc_view* view, int64_t n_cells, const float* centers,
                                   const int32_t* levels, const float* weights, float initial_size,
                                   float* out, void* stream);

/* Opaque sampler: a counter-based Philox4x32-10 stream keyed by `seed`; each generate_* call consumes
 * one value of a 64-bit call counter, which is all the state there is.  Replaces
 * struct ProbabilityFieldSampler and its host-side pcg32 (sampling/include/sampling_api.h:26-82). */
typedef struct inpc_sampler inpc_sampler;
inpc_sampler* inpc_sampler_create(int64_t seed);
void inpc_sampler_destroy(inpc_sampler* s);
/* Checkpoint / resume of the stream position (the reference's pcg32 state is not checkpointable). */
uint64_t inpc_sampler_get_counter(const inpc_sampler* s);
void inpc_sampler_set_counter(inpc_sampler* s, uint64_t counter);
/* The rejection sampler of inpc_generate_training_samples bounds its attempts per slot (the reference's loop,
 * sampling/src/sampling_kernels.cu:104-125, is unbounded).  1: some slots of this sampler's last such call
 * ran out and hold their last candidate, a position outside the view frustum; 0: none did; -1: no longer known
 * (more than 1024 status-carrying calls since).  Final once the call's stream has been synchronised. */
int inpc_sampler_exhausted(const inpc_sampler* s);

/* Bytes of device scratch the generate_* calls need for `n_cells` leaves (CDF + scan partials). */
size_t inpc_sampler_workspace_bytes(int64_t n_cells);

/* Visible training samples: positions (n,3) f32, indices (n) i64.  No host synchronisation: when
 * the weight sum is <= 0 the kernel writes zeros / -1 as the reference does
 * (sampling/src/sampling.cu:107-111).  Replaces inpc::sampling::create_training_samples
 * (sampling/include/sampling.h:28-50). */
int inpc_generate_training_samples(inpc_sampler* s, const inpc_view* view, int64_t n_cells,
                                   const float* centers, const int32_t* levels, const float* weights,
                                   float initial_size, int64_t n_samples, float* positions,
                                   int64_t* indices, void* workspace, void* stream);

/* Unconditional samples.  Reads the weight sum back; *n_written is n_samples, or 0 when the sum is
 * <= 0 (the reference then returns an empty tensor, sampling/src/sampling_api.cu:154).
 * Replaces compute_cdf + create_samples (sampling/include/sampling.h:52-66). */
int inpc_generate_samples(inpc_sampler* s, const inpc_view* view, int64_t n_cells, const float* centers,
                          const int32_t* levels, const float* weights, float initial_size,
                          int64_t n_samples, float* positions, int64_t* n_written, void* workspace,
                          void* stream);

/* Expected-count samples in two steps so the caller can size the output.  _count reads one integer
 * back: *n_created = sum over visible leaves of max(1, round(w/sum*n_samples)), 0 if sum <= 0.
 * _fill writes n_created*n_multi positions.  Replaces compute_sample_distribution +
 * create_expected_samples (sampling/include/sampling.h:68-83). */
int inpc_generate_expected_samples_count(inpc_sampler* s, const inpc_view* view, int64_t n_cells,
                                         const float* centers, const int32_t* levels,
                                         const float* weights, float initial_size, int64_t n_samples,
                                         int64_t* n_created, void* workspace, void* stream);
int inpc_generate_expected_samples_fill(inpc_sampler* s, int64_t n_cells, const float* centers,
                                        const int32_t* levels, float initial_size, int64_t n_created,
                                        int64_t n_multi, float* positions, void* workspace, void* stream);

/* Leaf look-up alone: out[i] = min(lower_bound(cdf, u[i]), n_cells-1) as int64.
 * Replaces binary_search (sampling/include/sampling_utils.h:49-69). */
int inpc_draw_leaves(const float* cdf, int64_t n_cells, const float* u, int64_t n, int64_t* out,
                     void* stream);

/* Normalised inclusive CDF of `weights` into `cdf` (fp32), and the plain sum into *sum_out (device,
 * one float).  Replaces the Sum / normalize / InclusiveSum sequence of sampling/src/sampling.cu:97-125. */
int inpc_build_cdf(const float* weights, int64_t n_cells, float* cdf, float* sum_out, void* workspace,
                   void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused misc ops (misc/include/misc.h:7-33)
 * ---------------------------------------------------------------------------------------- */

/* grads (=|+=) factor(level(index)) * weights for the fixed ten-level hash grid layout; `add` != 0
 * accumulates.  Replaces compute_/add_normalized_weight_decay_grads (misc/include/misc.h:9-17). */
int inpc_weight_decay_grads(const float* weights, float* grads, int64_t n, int add, void* stream);
/* Replaces spherical_contraction (misc/include/misc.h:19-22). */
int inpc_spherical_contraction(const float* positions, float* out, int64_t n, void* stream);
/* Mean Cauchy loss into *loss (device, one float), reduction fused; `partials` needs
 * inpc_cauchy_workspace_bytes(n).  Replaces cauchy_loss + the torch .sum()
 * (misc/include/misc.h:24-28, misc/src/misc_api.cu:64). */
size_t inpc_cauchy_workspace_bytes(int64_t n);
int inpc_cauchy_loss(const float* input, const float* target, int64_t n, float* loss, void* partials,
                     void* stream);
/* grad (device, one float) is the upstream scalar.  Replaces cauchy_loss_backward (misc.h:29-33). */
int inpc_cauchy_loss_backward(const float* grad, const float* input, const float* target, int64_t n,
                              float* grad_input, void* stream);

/* ------------------------------------------------------------------------------------------
 * Probability-field update (the consumer of blending_weights; Modules/ProbabilityField.py:146-157)
 * ---------------------------------------------------------------------------------------- */

/* Per-leaf maximum and minimum of the blending weights of the samples drawn from each leaf, over any
 * number of views / ranks.  `stats` holds two uint32 per leaf, 8-byte aligned: {bit pattern of the
 * maximum, 0x7FFFFFFF - bit pattern of the minimum}; weights are non-negative, so both words only grow
 * and one MAX all-reduce of the int32 view of the whole buffer reduces it across ranks; all-zero means
 * "no sample".  Reset once, accumulate per view, all-reduce, then apply inpc_leaf_update.
 * indices < 0 are skipped.
 * Replaces the two scatter_reduce_ calls (amax / amin, include_self=False) of
 * Modules/ProbabilityField.py:152-155. */
int inpc_leaf_stats_reset(uint32_t* stats, int64_t n_leaves, void* stream);
int inpc_leaf_stats_accumulate(const int64_t* indices, const float* weights, int64_t n, uint32_t* stats,
                               int64_t n_leaves, void* stream);
/* leaf_weights = max(leaf_weights * decay, max_sampled);
 * scores = max(scores * decay, clamp(max_sampled - min_sampled, 0, 1)); decay is 0.9968 in the reference.
 * Replaces Modules/ProbabilityField.py:148-149 and :156-157. */
int inpc_leaf_update(float* leaf_weights, float* leaf_subdivision_scores, const uint32_t* stats,
                     int64_t n_leaves, float decay, void* stream);

/* Structural updates of the octree probability field (the reference does them in torch:
 * Modules/ProbabilityField.py:159-165 prune, :217-257 subdivide).  Both are two calls: *_count
 * selects and scans (kind 0 = prune: values are the leaf weights, a leaf is KEPT when weight >
 * threshold; kind 1 = subdivide: values are the subdivision scores, a leaf is SPLIT when score >
 * threshold and level < max_level) and returns the number of selected leaves to the host (it
 * synchronises the stream); the caller sizes the outputs and calls the matching *_fill with the same
 * arguments and workspace (inpc_leaf_select_workspace_bytes(n) bytes).
 *   prune output:     n_selected leaves, old order kept.
 *   subdivide output: n - n_selected unsplit leaves in their old order, then 8 children per split
 *                     leaf in leaf order; child k sits at centre +- initial_size / 2^(level + 2) per
 *                     axis with (x, y, z) signs from bits (k&1, k&2, k&4), has level + 1, the parent's
 *                     weight and score 0.  The reference's cap on the leaf count (16,777,216,
 *                     ProbabilityField.py:222-224) is the caller's check between the two calls. */
size_t inpc_leaf_select_workspace_bytes(int64_t n_leaves);
int inpc_leaf_select_count(int kind, const float* values, const int32_t* levels, int64_t n, float threshold,
                           int max_level, void* workspace, int64_t* n_selected, void* stream);
int inpc_leaf_prune_fill(const float* centers, const int32_t* levels, const float* weights, const float* scores,
                         int64_t n, float threshold, const void* workspace, float* out_centers,
                         int32_t* out_levels, float* out_weights, float* out_scores, void* stream);
int inpc_leaf_subdivide_fill(const float* centers, const int32_t* levels, const float* weights,
                             const float* scores, int64_t n, float threshold, int max_level, float initial_size,
                             int64_t n_selected, const void* workspace, float* out_centers, int32_t* out_levels,
                             float* out_weights, float* out_scores, void* stream);

/* Image composition directly after the blend; images are (channels, H, W) planar fp32, alpha and
 * depth (H, W); n_pixels = H*W.  The reference does these with chains of torch element-wise ops.
 *   compose_background          out = image + (1 - alpha) * background            (Renderer.py:80)
 *   compose_background_backward grad_alpha = -sum_c g_c * background_c, grad_background = (1 - alpha) * g;
 *                               either output may be NULL; grad_image is grad_out itself
 *   multisample_accumulate      acc (+)= one multisample's image / depth / alpha; with `unpremultiply`
 *                               the features are divided by the sample's alpha first (0 where alpha
 *                               is 0)                                             (Renderer.py:108-117)
 *   multisample_resolve         after the last sample: image, depth, alpha *= 1/n; alpha_sum =
 *                               clamp(sum, 0, 1); with `remultiply` image *= alpha; with a background
 *                               image += (1 - alpha) * background                 (Renderer.py:118-125)
 * Each product and sum is rounded separately, so results equal the torch chain bit for bit. */
int inpc_compose_background(const float* image, const float* alpha, const float* background, int channels,
                            int64_t n_pixels, float* out, void* stream);
int inpc_compose_background_backward(const float* grad_out, const float* alpha, const float* background,
                                     int channels, int64_t n_pixels, float* grad_alpha, float* grad_background,
                                     void* stream);
int inpc_multisample_accumulate(float* acc_image, float* acc_depth, float* acc_alpha, const float* image,
                                const float* depth, const float* alpha, int channels, int64_t n_pixels, int first,
                                int unpremultiply, void* stream);
int inpc_multisample_resolve(float* acc_image, float* acc_depth, float* acc_alpha, float* alpha_sum,
                             const float* background, int channels, int64_t n_pixels, int n_multisamples,
                             int remultiply, void* stream);

/* Global point cloud extraction (Modules/ProbabilityField.py:121-144, utils.py:36-64).
 *   inpc_draw_leaf_counts  counts[leaf] = how many of n_samples multinomial draws (with replacement,
 *                          probability proportional to weights) fell into the leaf; replaces
 *                          torch.multinomial + torch.bincount (ProbabilityField.py:129-130) with the
 *                          sampler's Philox stream.  Synchronises the stream once (zero-sum check).
 *   inpc_halton_samples    n_total = sum(counts) positions, leaf by leaf: the h-th sample of a leaf is
 *                          centre - cell/2 + halton(h + 1; bases 2, 3, 5) * cell, a leaf with one
 *                          sample puts it at its centre; bit-identical to compute_halton_coords +
 *                          ProbabilityField.py:131-140 (the Halton elements are formed in double
 *                          precision and stored as float32 as there).
 *   inpc_morton_order      out = positions sorted by a 30-bit Morton code (10 bits per axis) inside
 *                          the cube [box_lo, box_lo + box_extent]^3 (box_lo: 3 HOST floats); stable.
 *                          Stands in for NeRFICG's CudaUtils.MortonEncoding.morton_encode + argsort
 *                          (ProbabilityField.py:141-143), which is not part of the reference tree:
 *                          the code width and the box are this library's choice.
 * `workspace`: inpc_sampler_workspace_bytes(n_cells) for the first two, inpc_morton_workspace_bytes(n)
 * for the third. */
int inpc_draw_leaf_counts(inpc_sampler* s, int64_t n_cells, const float* weights, int64_t n_samples,
                          uint32_t* counts, void* workspace, void* stream);
int inpc_halton_samples(const uint32_t* counts, int64_t n_cells, const float* centers, const int32_t* levels,
                        float initial_size, int64_t n_total, float* positions, void* workspace, void* stream);
size_t inpc_morton_workspace_bytes(int64_t n);
int inpc_morton_order(const float* positions, int64_t n, const float* box_lo, float box_extent, float* out,
                      void* workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INPC_B200_H */
