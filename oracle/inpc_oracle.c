/*
 * TEST INFRASTRUCTURE — CPU restatement ("oracle") of the INPC CUDA backend hot path.
 *
 * Only the test-suite, the smoke check and the cpu-baseline / reference legs of the benchmark
 * may load this library.  The product (inpc_b200) never calls it and has no CPU fallback.
 *
 * Each function restates, in plain scalar C, what the reference's CUDA kernels compute; the
 * reference file:line it follows (paths relative to INPCCudaBackend/INPCCudaBackend/ of the
 * reference project) is cited per function.  The reference ships no CPU implementation, no tests
 * and no golden vectors for this path, so parity is pinned by outputs of the reference's own CUDA
 * backend (built unmodified into oracle/_ref and run on a B200): committed as fixtures under
 * tests/golden/ and checked by tests/test_oracle_golden.py on the CPU, and compared live by the
 * GPU tests.
 *
 * Exactness: integer stages (depth keys, tile bounds, ordering, ranges, CDF look-ups, both random
 * generators) are bit-exact restatements.  Floating point follows the reference expression by
 * expression with the fused multiply-adds nvcc forms made explicit; rsqrtf/expf/exp2f/__expf are
 * the host libm here, so images, weights and gradients agree to rounding, not bit for bit.
 * Accumulations that the reference performs with float atomics in unspecified order (blending
 * weights, per-point gradients) are summed in double and rounded once.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 half_t;

typedef struct {
    float w2c[16];   /* row-major 4x4, rows 0..2 used */
    float cam[3];    /* camera position in world space */
    int width, height;
    float fx, fy, cx, cy, near_plane, far_plane;
} orc_camera;

enum { ORC_BILINEAR = 0, ORC_GAUSSIAN = 1 };
/* which of the three preprocess kernels of the reference is restated */
enum { ORC_TRAIN = 0, ORC_RAW37 = 1, ORC_PREEXTRACTED = 2 };

/* How nvcc contracts r.x*p.x + r.y*p.y + r.z*p.z + r.w (default -fmad=true).  Variant 1 reproduces
 * the reference backend's depth and screen coordinates bit for bit (tests/golden); the others are
 * kept so that the golden test can show that the fixture tells them apart. */
static int g_contract = 1;
void orc_set_contract(int v) { g_contract = v; }

static inline float affine_row(const float* r, const float* p) {
    float t;
    switch (g_contract) {
        case 0: /* first product rounded, the others fused onto it, then + w */
            t = r[0] * p[0];
            t = fmaf(r[1], p[1], t);
            t = fmaf(r[2], p[2], t);
            return t + r[3];
        default:
        case 1: /* second product rounded, first fused onto it, third fused, then + w */
            t = r[1] * p[1];
            t = fmaf(r[0], p[0], t);
            t = fmaf(r[2], p[2], t);
            return t + r[3];
        case 2: /* no contraction at all */
            t = r[0] * p[0] + r[1] * p[1];
            t = t + r[2] * p[2];
            return t + r[3];
        case 3: /* everything fused, w included */
            t = fmaf(r[2], p[2], r[3]);
            t = fmaf(r[1], p[1], t);
            return fmaf(r[0], p[0], t);
    }
}

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline float satf(float x) { return x < 0.0f ? 0.0f : (x > 1.0f ? 1.0f : x); }
static inline float clampf(float x, float lo, float hi) { return fminf(fmaxf(x, lo), hi); }

/* __float2int_rd / __float2int_ru: round toward -inf / +inf, saturating, NaN -> 0 */
static inline int f2i_rd(float x) {
    if (x != x) return 0;
    double f = floor((double)x);
    if (f < -2147483648.0) return INT32_MIN;
    if (f > 2147483647.0) return INT32_MAX;
    return (int)f;
}
static inline int f2i_ru(float x) {
    if (x != x) return 0;
    double f = ceil((double)x);
    if (f < -2147483648.0) return INT32_MIN;
    if (f > 2147483647.0) return INT32_MAX;
    return (int)f;
}
static inline uint32_t umin(uint32_t a, uint32_t b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

int orc_end_bit(uint32_t n) { /* rasterization/include/rasterization_utils.h:3-13: bit length of n */
    int b = 0;
    while (n) { ++b; n >>= 1; }
    return b;
}

/* ------------------------------------------------------------------------------------------
 * SH degree-2 evaluation along the view ray: rasterization/include/sh_utils.cuh:6-23 (forward),
 * :44-62 (backward).  `h` points at 36 halves laid out coefficient-major, channel-minor.
 * ---------------------------------------------------------------------------------------- */
static void sh_basis(const float* p, const float* cam, float* b) {
    const float vx = p[0] - cam[0], vy = p[1] - cam[1], vz = p[2] - cam[2];
    const float inv = 1.0f / sqrtf(vx * vx + vy * vy + vz * vz);
    const float x = vx * inv, y = vy * inv, z = vz * inv;
    b[0] = 0.28209479177387814f;
    b[1] = -0.48860251190291987f * y;
    b[2] = 0.48860251190291987f * z;
    b[3] = -0.48860251190291987f * x;
    b[4] = 1.0925484305920792f * (x * y);
    b[5] = -1.0925484305920792f * (y * z);
    b[6] = 0.94617469575755997f * (z * z) - 0.31539156525251999f;
    b[7] = -1.0925484305920792f * (x * z);
    b[8] = 0.54627421529603959f * (x * x) - 0.54627421529603959f * (y * y);
}

static void sh_forward(const float* p, const float* cam, const half_t* h, float* out4) {
    float b[9];
    sh_basis(p, cam, b);
    for (int c = 0; c < 4; ++c) {
        float acc = b[0] * (float)h[c];
        for (int k = 1; k < 9; ++k) acc += b[k] * (float)h[4 * k + c];
        out4[c] = acc;
    }
}

static void sh_backward(const float* p, const float* cam, const float* g4, half_t* gh) {
    float b[9];
    sh_basis(p, cam, b);
    for (int k = 0; k < 9; ++k)
        for (int c = 0; c < 4; ++c) gh[4 * k + c] = (half_t)(b[k] * g4[c]);
}

/* ------------------------------------------------------------------------------------------
 * Preprocess: cull, project, tile bounds, view-dependent feature.
 *   bilinear  rasterization/src/bilinear/kernels.cu:11-84 (train / pre-extracted), :106-184 (raw 37)
 *   gaussian  rasterization/src/gaussian/kernels.cu:11-111, :113-217, :219-324
 * Outputs are per input point (no compaction); n_touched==0 marks a culled point and leaves the
 * other per-point outputs at zero.  `tile` is the tile edge (8 in the reference).
 * `features` is (n,36) halves for TRAIN/PREEXTRACTED and (n,37) for RAW37.
 * ---------------------------------------------------------------------------------------- */
void orc_preprocess(int mode, int variant, const orc_camera* cam, int tile, int64_t n,
                    const float* positions, const half_t* features, const float* opacities,
                    const float* scales, float sigma_world, float sigma_cutoff,
                    uint32_t* n_touched, uint16_t* bounds, float* screen, float* feat_view,
                    float* depth_out, float* opacity_out, float* conic_out) {
    const uint32_t gw = (uint32_t)((cam->width + tile - 1) / tile);
    const uint32_t gh = (uint32_t)((cam->height + tile - 1) / tile);
    const float tf = (float)tile;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        n_touched[i] = 0;
        memset(bounds + 4 * i, 0, 8);
        screen[2 * i] = screen[2 * i + 1] = 0.0f;
        memset(feat_view + 4 * i, 0, 16);
        depth_out[i] = 0.0f;
        if (opacity_out) opacity_out[i] = 0.0f;
        if (conic_out) conic_out[3 * i] = conic_out[3 * i + 1] = conic_out[3 * i + 2] = 0.0f;

        const float* p = positions + 3 * i;
        const float depth = affine_row(cam->w2c + 8, p);
        if (depth < cam->near_plane || depth > cam->far_plane) continue;
        const float x = affine_row(cam->w2c + 0, p) / depth;
        const float y = affine_row(cam->w2c + 4, p) / depth;
        const float sx = fmaf(x, cam->fx, cam->cx);
        const float sy = fmaf(y, cam->fy, cam->cy);

        float ex = 0.5f, ey = 0.5f, conic[3] = {0, 0, 0};
        if (mode == ORC_GAUSSIAN) {
            float var;
            float k = 3.0f;
            if (variant == ORC_TRAIN) {
                var = (0.3f * 0.3f * 0.5f * 0.5f) / (cam->fx * cam->fy);
            } else {
                k = sigma_cutoff;
                if (variant == ORC_PREEXTRACTED && scales) var = scales[i] * scales[i];
                else var = sigma_world * sigma_world;
            }
            const float j00 = cam->fx / depth;
            const float j02 = -j00 * clampf(x, -1.3f * cam->cx / cam->fx, 1.3f * cam->cx / cam->fx);
            const float j11 = cam->fy / depth;
            const float j12 = -j11 * clampf(y, -1.3f * cam->cy / cam->fy, 1.3f * cam->cy / cam->fy);
            float cxx = var * fmaf(j02, j02, j00 * j00);
            float cxy = var * (j02 * j12);
            float cyy = var * fmaf(j12, j12, j11 * j11);
            cxx += 0.16f;
            cyy += 0.16f;
            const float det = fmaf(cxx, cyy, -(cxy * cxy));
            if (det == 0.0f) continue;
            const float rdet = 1.0f / det;
            conic[0] = cyy * rdet;
            conic[1] = -cxy * rdet;
            conic[2] = cxx * rdet;
            ex = fmaf(k, sqrtf(cxx), -0.5f);
            ey = fmaf(k, sqrtf(cyy), -0.5f);
        }
        const uint32_t x0 = umin(gw, (uint32_t)imax(0, f2i_rd((sx - ex) / tf)));
        const uint32_t x1 = umin(gw, (uint32_t)imax(0, f2i_ru((sx + ex) / tf)));
        const uint32_t y0 = umin(gh, (uint32_t)imax(0, f2i_rd((sy - ey) / tf)));
        const uint32_t y1 = umin(gh, (uint32_t)imax(0, f2i_ru((sy + ey) / tf)));
        const uint32_t nt = (x1 - x0) * (y1 - y0);
        if (nt == 0) continue;

        n_touched[i] = nt;
        bounds[4 * i + 0] = (uint16_t)x0;
        bounds[4 * i + 1] = (uint16_t)x1;
        bounds[4 * i + 2] = (uint16_t)y0;
        bounds[4 * i + 3] = (uint16_t)y1;
        screen[2 * i] = sx;
        screen[2 * i + 1] = sy;
        depth_out[i] = depth;
        if (variant == ORC_RAW37) {
            const half_t* h = features + 37 * i;
            sh_forward(p, cam->cam, h + 1, feat_view + 4 * i);
            /* opacity = 1 - exp(-exp(raw)), bilinear/kernels.cu:144 (fast-math exp on the GPU) */
            if (opacity_out) opacity_out[i] = 1.0f - expf(-expf((float)h[0]));
        } else {
            sh_forward(p, cam->cam, features + 36 * i, feat_view + 4 * i);
            if (opacity_out && opacities) opacity_out[i] = opacities[i];
        }
        if (conic_out) { conic_out[3 * i] = conic[0]; conic_out[3 * i + 1] = conic[1]; conic_out[3 * i + 2] = conic[2]; }
    }
}

/* ------------------------------------------------------------------------------------------
 * Ordering: rasterization/src/bilinear/forward.cu:86-141 with kernels.cu:186-239.
 * Visible points are taken in index order (one legal outcome of the reference's atomic
 * compaction), stably sorted by the bit pattern of their depth, expanded row-major over their
 * tile bounds, and stably sorted by tile.  ranges[2*t..] = [first, last+1) or (0,0).
 * Call orc_order_counts first to size sorted_points (V) and inst_* (I).
 * ---------------------------------------------------------------------------------------- */
void orc_order_counts(int64_t n, const uint32_t* n_touched, int64_t* n_visible, int64_t* n_instances) {
    int64_t v = 0, t = 0;
    for (int64_t i = 0; i < n; ++i)
        if (n_touched[i]) { ++v; t += n_touched[i]; }
    *n_visible = v;
    *n_instances = t;
}

static void radix_sort_pairs(uint64_t* keys, uint32_t* vals, int64_t n, int bits) {
    if (n <= 1) return;
    uint64_t* k2 = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)n);
    uint32_t* v2 = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)n);
    for (int shift = 0; shift < bits; shift += 11) {
        int64_t hist[2049];
        memset(hist, 0, sizeof(hist));
        for (int64_t i = 0; i < n; ++i) hist[((keys[i] >> shift) & 2047) + 1]++;
        for (int d = 0; d < 2048; ++d) hist[d + 1] += hist[d];
        for (int64_t i = 0; i < n; ++i) {
            const int64_t dst = hist[(keys[i] >> shift) & 2047]++;
            k2[dst] = keys[i];
            v2[dst] = vals[i];
        }
        uint64_t* tk = keys; keys = k2; k2 = tk;
        uint32_t* tv = vals; vals = v2; v2 = tv;
    }
    /* an odd number of passes leaves the result in the scratch pair: copy back */
    const int passes = (bits + 10) / 11;
    if (passes & 1) {
        memcpy(k2, keys, sizeof(uint64_t) * (size_t)n);
        memcpy(v2, vals, sizeof(uint32_t) * (size_t)n);
        free(keys);
        free(vals);
    } else {
        free(k2);
        free(v2);
    }
}

void orc_order(int64_t n, int tile, int width, int height, const uint32_t* n_touched,
               const uint16_t* bounds, const float* depth, uint32_t* sorted_points,
               uint32_t* inst_point, uint32_t* inst_tile, uint32_t* ranges) {
    const uint32_t gw = (uint32_t)((width + tile - 1) / tile);
    const uint32_t gh = (uint32_t)((height + tile - 1) / tile);
    int64_t v = 0, total = 0;
    for (int64_t i = 0; i < n; ++i)
        if (n_touched[i]) { ++v; total += n_touched[i]; }
    uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(v > total ? v : total) + 8);
    int64_t j = 0;
    for (int64_t i = 0; i < n; ++i)
        if (n_touched[i]) { keys[j] = f2u(depth[i]); sorted_points[j] = (uint32_t)i; ++j; }
    radix_sort_pairs(keys, sorted_points, v, 32);
    int64_t o = 0;
    for (int64_t s = 0; s < v; ++s) {
        const uint32_t i = sorted_points[s];
        const uint16_t* b = bounds + 4 * (int64_t)i;
        for (uint32_t ty = b[2]; ty < b[3]; ++ty)
            for (uint32_t tx = b[0]; tx < b[1]; ++tx) {
                keys[o] = (uint64_t)ty * gw + tx;
                inst_point[o] = i;
                ++o;
            }
    }
    radix_sort_pairs(keys, inst_point, total, orc_end_bit(gw * gh - 1) > 0 ? orc_end_bit(gw * gh - 1) : 1);
    memset(ranges, 0, sizeof(uint32_t) * 2 * (size_t)gw * gh);
    for (int64_t s = 0; s < total; ++s) {
        const uint32_t t = (uint32_t)keys[s];
        inst_tile[s] = t;
        if (s == 0 || (uint32_t)keys[s - 1] != t) ranges[2 * t] = (uint32_t)s;
        if (s == total - 1 || (uint32_t)keys[s + 1] != t) ranges[2 * t + 1] = (uint32_t)(s + 1);
    }
    free(keys);
}

/* ------------------------------------------------------------------------------------------
 * Per-fragment weight of point j at pixel centre (pcx, pcy); returns 0 when the reference skips it.
 *   bilinear: kernels.cu:286-290    gaussian: gaussian/kernels.cu:447-453 (threshold argument)
 * ---------------------------------------------------------------------------------------- */
static inline int frag_weight(int mode, const float* s, const float* conic, float pcx, float pcy,
                              float g_threshold, float* w) {
    if (mode == ORC_BILINEAR) {
        const float dx = fabsf(s[0] - pcx), dy = fabsf(s[1] - pcy);
        if (dx >= 1.0f || dy >= 1.0f) return 0;
        *w = satf(1.0f - dx) * satf(1.0f - dy);
        return 1;
    }
    const float dx = s[0] - pcx, dy = s[1] - pcy;
    const float q = -0.5f * (conic[0] * dx * dx + conic[2] * dy * dy) - conic[1] * dx * dy;
    if (q > 0.0f) return 0;
    const float g = expf(q);
    if (g < g_threshold) return 0;
    *w = g;
    return 1;
}

#define ORC_T_EPS 1e-4f
#define ORC_TRAIN_G_THRESHOLD 0.01110899653f

/* Blend forward: bilinear/kernels.cu:241-313, gaussian/kernels.cu:401-474.
 * image is (4,H,W), alpha (H,W), blending_weights (n) — all fully written. */
void orc_blend_forward(int mode, const orc_camera* cam, int tile, int64_t n, const uint32_t* ranges,
                       const uint32_t* inst_point, const float* screen, const float* feat_view,
                       const float* opacity, const float* conic, float* image, float* alpha,
                       float* blending_weights) {
    const int W = cam->width, H = cam->height;
    const int gw = (W + tile - 1) / tile, gh = (H + tile - 1) / tile;
    const int64_t P = (int64_t)W * H;
    double* bw_acc = (double*)calloc((size_t)(n > 0 ? n : 1), sizeof(double));
#pragma omp parallel for schedule(dynamic, 4)
    for (int t = 0; t < gw * gh; ++t) {
        const int tx = t % gw, ty = t / gw;
        const uint32_t r0 = ranges[2 * t], r1 = ranges[2 * t + 1];
        for (int ly = 0; ly < tile; ++ly)
            for (int lx = 0; lx < tile; ++lx) {
                const int px = tx * tile + lx, py = ty * tile + ly;
                if (px >= W || py >= H) continue;
                const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
                float C[4] = {0, 0, 0, 0}, T = 1.0f;
                for (uint32_t s = r0; s < r1; ++s) {
                    const uint32_t i = inst_point[s];
                    float w;
                    if (!frag_weight(mode, screen + 2 * (int64_t)i, conic ? conic + 3 * (int64_t)i : 0, pcx, pcy,
                                     ORC_TRAIN_G_THRESHOLD, &w))
                        continue;
                    const float a = opacity[i] * w;
                    const float bw = T * a;
                    if (bw > 0.0f) {
                        const double add = (double)(bw * w);
#pragma omp atomic
                        bw_acc[i] += add;
                    }
                    for (int c = 0; c < 4; ++c) C[c] = fmaf(bw, feat_view[4 * (int64_t)i + c], C[c]);
                    T *= 1.0f - a;
                    if (T < ORC_T_EPS) break;
                }
                const int64_t pi = (int64_t)py * W + px;
                for (int c = 0; c < 4; ++c) image[c * P + pi] = C[c];
                alpha[pi] = T < ORC_T_EPS ? 1.0f : 1.0f - T;
            }
    }
    for (int64_t i = 0; i < n; ++i) blending_weights[i] = (float)bw_acc[i];
    free(bw_acc);
}

/* Blend backward: bilinear/kernels.cu:315-420, gaussian/kernels.cu:476-579.
 * grad_feat_view (n,4) and grad_opacity (n) are fully written (zero where untouched). */
void orc_blend_backward(int mode, const orc_camera* cam, int tile, int64_t n, const uint32_t* ranges,
                        const uint32_t* inst_point, const float* screen, const float* feat_view,
                        const float* opacity, const float* conic, const float* grad_image,
                        const float* grad_alpha, const float* image, const float* alpha,
                        float* grad_feat_view, float* grad_opacity) {
    const int W = cam->width, H = cam->height;
    const int gw = (W + tile - 1) / tile, gh = (H + tile - 1) / tile;
    const int64_t P = (int64_t)W * H;
    double* gf = (double*)calloc((size_t)(n > 0 ? 4 * n : 1), sizeof(double));
    double* go = (double*)calloc((size_t)(n > 0 ? n : 1), sizeof(double));
#pragma omp parallel for schedule(dynamic, 4)
    for (int t = 0; t < gw * gh; ++t) {
        const int tx = t % gw, ty = t / gw;
        const uint32_t r0 = ranges[2 * t], r1 = ranges[2 * t + 1];
        for (int ly = 0; ly < tile; ++ly)
            for (int lx = 0; lx < tile; ++lx) {
                const int px = tx * tile + lx, py = ty * tile + ly;
                if (px >= W || py >= H) continue;
                const int64_t pi = (int64_t)py * W + px;
                const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
                float g[4], Cfin[4], Crun[4] = {0, 0, 0, 0};
                for (int c = 0; c < 4; ++c) { g[c] = grad_image[c * P + pi]; Cfin[c] = image[c * P + pi]; }
                const float K = grad_alpha[pi] * (1.0f - alpha[pi]);
                float T = 1.0f;
                for (uint32_t s = r0; s < r1; ++s) {
                    const uint32_t i = inst_point[s];
                    float w;
                    if (!frag_weight(mode, screen + 2 * (int64_t)i, conic ? conic + 3 * (int64_t)i : 0, pcx, pcy,
                                     ORC_TRAIN_G_THRESHOLD, &w))
                        continue;
                    const float a = opacity[i] * w;
                    const float bw = T * a;
                    const float* f = feat_view + 4 * (int64_t)i;
                    if (bw > 0.0f)
                        for (int c = 0; c < 4; ++c) {
                            const double add = (double)(bw * g[c]);
#pragma omp atomic
                            gf[4 * (int64_t)i + c] += add;
                        }
                    for (int c = 0; c < 4; ++c) Crun[c] = fmaf(bw, f[c], Crun[c]);
                    const float oma = 1.0f - a;
                    const float r = 1.0f / fmaxf(oma, 1e-8f);
                    float dot = 0.0f;
                    for (int c = 0; c < 4; ++c) dot = fmaf(fmaf(T, f[c], (Crun[c] - Cfin[c]) * r), g[c], dot);
                    const float dalpha = dot + K * r;
                    const float dop = dalpha * w;
                    if (dop != 0.0f) {
                        const double add = (double)dop;
#pragma omp atomic
                        go[i] += add;
                    }
                    T *= oma;
                    if (T < ORC_T_EPS) break;
                }
            }
    }
    for (int64_t i = 0; i < 4 * n; ++i) grad_feat_view[i] = (float)gf[i];
    for (int64_t i = 0; i < n; ++i) grad_opacity[i] = (float)go[i];
    free(gf);
    free(go);
}

/* SH chain rule per touched point: bilinear/kernels.cu:86-104 + sh_utils.cuh:44-62.
 * grad_features is (n,36) halves, zero rows for culled points. */
void orc_preprocess_backward(const orc_camera* cam, int64_t n, const float* positions,
                             const uint32_t* n_touched, const float* grad_feat_view, half_t* grad_features) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        if (!n_touched[i]) { memset(grad_features + 36 * i, 0, 72); continue; }
        sh_backward(positions + 3 * i, cam->cam, grad_feat_view + 4 * i, grad_features + 36 * i);
    }
}

/* Inference blend with expected depth: bilinear/kernels.cu:422-495, gaussian/kernels.cu:581-660.
 * g_threshold is exp(-sigma_cutoff^2/2) for the gaussian mode (gaussian/inference.cu:171). */
void orc_blend_inference(int mode, const orc_camera* cam, int tile, const uint32_t* ranges,
                         const uint32_t* inst_point, const float* screen, const float* feat_view,
                         const float* opacity, const float* depth, const float* conic, float g_threshold,
                         float* image, float* depth_image, float* alpha) {
    const int W = cam->width, H = cam->height;
    const int gw = (W + tile - 1) / tile, gh = (H + tile - 1) / tile;
    const int64_t P = (int64_t)W * H;
#pragma omp parallel for schedule(dynamic, 4)
    for (int t = 0; t < gw * gh; ++t) {
        const int tx = t % gw, ty = t / gw;
        const uint32_t r0 = ranges[2 * t], r1 = ranges[2 * t + 1];
        for (int ly = 0; ly < tile; ++ly)
            for (int lx = 0; lx < tile; ++lx) {
                const int px = tx * tile + lx, py = ty * tile + ly;
                if (px >= W || py >= H) continue;
                const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
                float C[4] = {0, 0, 0, 0}, Z = 0.0f, T = 1.0f;
                for (uint32_t s = r0; s < r1; ++s) {
                    const uint32_t i = inst_point[s];
                    float w;
                    if (!frag_weight(mode, screen + 2 * (int64_t)i, conic ? conic + 3 * (int64_t)i : 0, pcx, pcy,
                                     g_threshold, &w))
                        continue;
                    const float a = opacity[i] * w;
                    const float bw = T * a;
                    for (int c = 0; c < 4; ++c) C[c] = fmaf(bw, feat_view[4 * (int64_t)i + c], C[c]);
                    Z = fmaf(bw, depth[i], Z);
                    T *= 1.0f - a;
                    if (T < ORC_T_EPS) break;
                }
                const int64_t pi = (int64_t)py * W + px;
                const float A = 1.0f - T;
                for (int c = 0; c < 4; ++c) image[c * P + pi] = C[c];
                depth_image[pi] = A > 0.0f ? Z / A : 0.0f;
                alpha[pi] = T < ORC_T_EPS ? 1.0f : A;
            }
    }
}

/* ==========================================================================================
 * Sampler
 * ======================================================================================== */

/* The sampler of the product spells out every fused multiply-add, and so does this restatement:
 * all sampler values are reproduced bit for bit.  (The reference leaves contraction to nvcc; its
 * values agree to rounding.) */
static inline float affine_fused(const float* r, const float* p) {
    return fmaf(r[2], p[2], fmaf(r[1], p[1], fmaf(r[0], p[0], r[3])));
}

/* Leaf weight for one viewpoint: sampling/src/sampling_kernels.cu:9-64. */
static int in_frustum(const orc_camera* cam, const float* p, float* z_out) {
    const float vx = affine_fused(cam->w2c + 0, p);
    const float vy = affine_fused(cam->w2c + 4, p);
    const float z = affine_fused(cam->w2c + 8, p);
    const float inv = 1.0f / (z + 1e-8f);
    const float x = fmaf(vx * inv, cam->fx, cam->cx);
    const float y = fmaf(vy * inv, cam->fy, cam->cy);
    if (z_out) *z_out = z;
    return (z >= cam->near_plane) & (z <= cam->far_plane) & (x >= 0.0f) & (x < (float)cam->width) &
           (y >= 0.0f) & (y < (float)cam->height);
}

void orc_viewpoint_weights(const orc_camera* cam, int64_t n_cells, const float* centers, const int* levels,
                           const float* weights, float initial_size, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t l = 0; l < n_cells; ++l) {
        const float* c = centers + 3 * l;
        float z;
        int valid = in_frustum(cam, c, &z);
        if (!valid) {
            const float hs = initial_size / ldexpf(1.0f, levels[l] + 1);
            for (int k = 0; k < 8 && !valid; ++k) {
                const float q[3] = {fmaf(hs, (k & 4) ? 1.0f : -1.0f, c[0]), fmaf(hs, (k & 2) ? 1.0f : -1.0f, c[1]),
                                    fmaf(hs, (k & 1) ? 1.0f : -1.0f, c[2])};
                valid |= in_frustum(cam, q, 0);
            }
        }
        float w = 0.0f;
        if (valid) {
            const float ds = fmaxf(fabsf(z - cam->near_plane) / cam->far_plane, 1e-8f);
            /* 2^(level/2) exactly; the reference's exp2f(level*0.5f) agrees within exp2f's 2 ulp */
            const float ss = ldexpf((levels[l] & 1) ? 1.41421356237309504880f : 1.0f, levels[l] >> 1);
            w = 1.0f / (ds * ss) * weights[l];
        }
        out[l] = w;
    }
}

/* CDF: sampling/src/sampling.cu:97-125 computes sum, w * (1/sum) and an fp32 inclusive scan with CUB,
 * whose summation order is unspecified.  The product instead takes every weight as a 39-bit
 * fixed-point fraction of the largest weight and scans integers, which is exact in any order:
 *   q_i = trunc(w_i / w_max * 2^39), P_i = q_0 + .. + q_i, cdf_i = float(P_i / P_last),
 *   sum = float(P_last * 2^-39 * w_max).   Returns that sum (<= 0: no CDF). */
float orc_build_cdf(int64_t n_cells, const float* vw, float* cdf) {
    float w_max = 0.0f;
    for (int64_t l = 0; l < n_cells; ++l) w_max = fmaxf(w_max, vw[l]);
    if (!(w_max > 0.0f)) return 0.0f;
    uint64_t total = 0;
    for (int64_t l = 0; l < n_cells; ++l) total += vw[l] > 0.0f ? (uint64_t)((vw[l] / w_max) * 549755813888.0f) : 0u;
    uint64_t run = 0;
    if (cdf)
        for (int64_t l = 0; l < n_cells; ++l) {
            run += vw[l] > 0.0f ? (uint64_t)((vw[l] / w_max) * 549755813888.0f) : 0u;
            cdf[l] = (float)((double)run / (double)total);
        }
    return (float)((double)total * (1.0 / 549755813888.0) * (double)w_max);
}

/* sampling/include/sampling_utils.h:49-69: first index with cdf[idx] >= u, clamped to n-1. */
static inline uint32_t lower_bound_clamped(const float* cdf, float u, uint32_t n) {
    uint32_t first = 0, count = n;
    while (count > 0) {
        const uint32_t step = count / 2;
        if (cdf[first + step] < u) { first += step + 1; count -= step + 1; }
        else count = step;
    }
    return first < n - 1 ? first : n - 1;
}

void orc_draw_leaves(const float* cdf, uint32_t n_cells, const float* u, int64_t n, int64_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (int64_t)lower_bound_clamped(cdf, u[i], n_cells);
}

/* 23 random mantissa bits -> [0,1): sampling/include/pcg32.h:105-114 */
static inline float bits_to_unit_float(uint32_t r) { return u2f((r >> 9) | 0x3f800000u) - 1.0f; }

/* ---- PCG32 (sampling/include/pcg32.h:55-70, 147-168): LCG-64 state, XSH-RR output ---------- */
typedef struct { uint64_t state, inc; } orc_pcg32;
#define ORC_PCG_MULT 0x5851f42d4c957f2dULL

static uint32_t pcg_next(orc_pcg32* g) {
    const uint64_t old = g->state;
    g->state = old * ORC_PCG_MULT + g->inc;
    const uint32_t xs = (uint32_t)(((old >> 18u) ^ old) >> 27u);
    const uint32_t rot = (uint32_t)(old >> 59u);
    return (xs >> rot) | (xs << ((32u - rot) & 31u));
}
void orc_pcg_seed(orc_pcg32* g, uint64_t initstate, uint64_t initseq) {
    g->state = 0;
    g->inc = (initseq << 1u) | 1u;
    pcg_next(g);
    g->state += initstate;
    pcg_next(g);
}
void orc_pcg_advance(orc_pcg32* g, uint64_t delta) {
    uint64_t cm = ORC_PCG_MULT, cp = g->inc, am = 1, ap = 0;
    while (delta) {
        if (delta & 1) { am *= cm; ap = ap * cm + cp; }
        cp = (cm + 1) * cp;
        cm *= cm;
        delta >>= 1;
    }
    g->state = am * g->state + ap;
}
uint32_t orc_pcg_next_uint(orc_pcg32* g) { return pcg_next(g); }

static inline void jitter_position(const float* center, int level, float initial_size, const float* j3,
                                   int fused, float* out) {
    const float scale = 1.0f / ldexpf(1.0f, level) * initial_size;
    for (int k = 0; k < 3; ++k) {
        const float off = j3[k] - 0.5f;
        out[k] = fused ? fmaf(off, scale, center[k]) : center[k] + off * scale;
    }
}

/* Reference deterministic draw, one per output slot: sampling_kernels.cu:128-150.  `g` is the host
 * generator *before* the call; it is advanced by 4n as sampling.cu:208 does.  u_out (optional)
 * receives the CDF uniforms, leaf_out (optional) the drawn leaves. */
void orc_ref_create_samples(orc_pcg32* g, const float* cdf, uint32_t n_cells, const float* centers,
                            const int* levels, float initial_size, int64_t n, int fused, float* positions,
                            float* u_out, int64_t* leaf_out) {
    for (int64_t i = 0; i < n; ++i) {
        orc_pcg32 r = *g;
        /* the kernel multiplies in 32 bits: sample_idx * 4 wraps at 2^32 */
        orc_pcg_advance(&r, (uint64_t)(uint32_t)((uint32_t)i * 4u));
        const float u = bits_to_unit_float(pcg_next(&r));
        const uint32_t l = lower_bound_clamped(cdf, u, n_cells);
        float j[3];
        for (int k = 0; k < 3; ++k) j[k] = bits_to_unit_float(pcg_next(&r));
        jitter_position(centers + 3 * (int64_t)l, levels[l], initial_size, j, fused, positions + 3 * i);
        if (u_out) u_out[i] = u;
        if (leaf_out) leaf_out[i] = l;
    }
    orc_pcg_advance(g, (uint64_t)(uint32_t)((uint32_t)n * 4u));
}

/* Expected-sample mode: counts (sampling_kernels.cu:152-169), repeat-interleave (:171-183),
 * jitter (:185-205).  counts[] is written; returns n_created. */
int64_t orc_expected_counts(int64_t n_cells, const float* vw, float sum, uint32_t n_samples, int* counts) {
    int64_t total = 0;
    const float norm = 1.0f / sum;
    for (int64_t l = 0; l < n_cells; ++l) {
        int c = 0;
        if (vw[l] > 0.0f) {
            c = (int)nearbyintf(vw[l] * norm * (float)n_samples);
            if (c < 1) c = 1;
        }
        counts[l] = c;
        total += c;
    }
    return total;
}

void orc_ref_expected_samples(orc_pcg32* g, int64_t n_cells, const int* counts, const float* centers,
                              const int* levels, float initial_size, int64_t n_created, int64_t n_multi,
                              int fused, float* positions) {
    int* cell = (int*)malloc(sizeof(int) * (size_t)(n_created > 0 ? n_created : 1));
    int64_t o = 0;
    for (int64_t l = 0; l < n_cells; ++l)
        for (int k = 0; k < counts[l]; ++k) cell[o++] = (int)l;
    const int64_t total = n_created * n_multi;
    for (int64_t i = 0; i < total; ++i) {
        const int l = cell[i % n_created];
        orc_pcg32 r = *g;
        orc_pcg_advance(&r, (uint64_t)(uint32_t)((uint32_t)i * 3u));
        float j[3];
        for (int k = 0; k < 3; ++k) j[k] = bits_to_unit_float(pcg_next(&r));
        jitter_position(centers + 3 * (int64_t)l, levels[l], initial_size, j, fused, positions + 3 * i);
    }
    orc_pcg_advance(g, (uint64_t)(uint32_t)((uint32_t)total * 3u));
    free(cell);
}

/* ---- Philox4x32-10 (Salmon et al., SC'11): the counter-based stream of the B200 sampler ---- */
void orc_philox4x32(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* Stream layout of the B200 sampler: counter = (slot lo, attempt | slot hi << 20 ... ) is fixed in
 * one place so that the CUDA kernel and this restatement cannot drift apart:
 *   ctr = { slot (low 32 bits), attempt, call (low 32), call (high 32) }, key = seed (lo, hi)
 *   out[0] -> CDF uniform, out[1..3] -> jitter x, y, z.   */
static inline void philox_draw(uint64_t seed, uint64_t call, uint32_t slot, uint32_t attempt, float u[4]) {
    const uint32_t ctr[4] = {slot, attempt, (uint32_t)call, (uint32_t)(call >> 32)};
    const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t o[4];
    orc_philox4x32(ctr, key, o);
    for (int k = 0; k < 4; ++k) u[k] = bits_to_unit_float(o[k]);
}

#define ORC_MAX_ATTEMPTS 4096

/* Training samples, B200 design: one output slot per thread, redraw until the jittered position
 * passes the frustum test of sampling_kernels.cu:106-113 (z, then x, then y).  Same distribution as
 * the reference's ticketed rejection loop (:77-126) but reproducible: slot s always holds the
 * first accepted attempt of stream (seed, call, s).  Returns the number of slots that ran out of
 * attempts (they keep their last candidate). */
int64_t orc_training_samples(const orc_camera* cam, uint64_t seed, uint64_t call, const float* cdf,
                             uint32_t n_cells, const float* centers, const int* levels, float initial_size,
                             int64_t n, float* positions, int64_t* indices) {
    int64_t exhausted = 0;
#pragma omp parallel for schedule(static) reduction(+ : exhausted)
    for (int64_t s = 0; s < n; ++s) {
        uint32_t l = 0;
        float pos[3] = {0, 0, 0};
        int ok = 0;
        for (uint32_t a = 0; a < ORC_MAX_ATTEMPTS && !ok; ++a) {
            float u[4];
            philox_draw(seed, call, (uint32_t)s, a, u);
            l = lower_bound_clamped(cdf, u[0], n_cells);
            jitter_position(centers + 3 * (int64_t)l, levels[l], initial_size, u + 1, 1, pos);
            const float z = affine_fused(cam->w2c + 8, pos);
            if (z < cam->near_plane || z > cam->far_plane) continue;
            const float inv = 1.0f / (z + 1e-8f);
            const float x = fmaf(affine_fused(cam->w2c + 0, pos) * inv, cam->fx, cam->cx);
            if (x < 0.0f || x >= (float)cam->width) continue;
            const float y = fmaf(affine_fused(cam->w2c + 4, pos) * inv, cam->fy, cam->cy);
            if (y < 0.0f || y >= (float)cam->height) continue;
            ok = 1;
        }
        if (!ok) ++exhausted;
        positions[3 * s] = pos[0]; positions[3 * s + 1] = pos[1]; positions[3 * s + 2] = pos[2];
        indices[s] = (int64_t)l;
    }
    return exhausted;
}

/* Unconditional draws (generate_samples), Philox stream, attempt fixed at 0. */
void orc_samples(uint64_t seed, uint64_t call, const float* cdf, uint32_t n_cells, const float* centers,
                 const int* levels, float initial_size, int64_t n, float* positions, int64_t* indices) {
#pragma omp parallel for schedule(static)
    for (int64_t s = 0; s < n; ++s) {
        float u[4];
        philox_draw(seed, call, (uint32_t)s, 0, u);
        const uint32_t l = lower_bound_clamped(cdf, u[0], n_cells);
        jitter_position(centers + 3 * (int64_t)l, levels[l], initial_size, u + 1, 1, positions + 3 * s);
        if (indices) indices[s] = (int64_t)l;
    }
}

/* Expected samples, Philox stream: slot i jitters inside leaf cell[i % n_created] with out[1..3]. */
void orc_expected_samples(uint64_t seed, uint64_t call, int64_t n_cells, const int* counts,
                          const float* centers, const int* levels, float initial_size, int64_t n_created,
                          int64_t n_multi, float* positions) {
    int* cell = (int*)malloc(sizeof(int) * (size_t)(n_created > 0 ? n_created : 1));
    int64_t o = 0;
    for (int64_t l = 0; l < n_cells; ++l)
        for (int k = 0; k < counts[l]; ++k) cell[o++] = (int)l;
    const int64_t total = n_created * n_multi;
    for (int64_t i = 0; i < total; ++i) {
        const int l = cell[i % n_created];
        float u[4];
        philox_draw(seed, call, (uint32_t)i, 0, u);
        jitter_position(centers + 3 * (int64_t)l, levels[l], initial_size, u + 1, 1, positions + 3 * i);
    }
    free(cell);
}

/* ==========================================================================================
 * Misc fused ops: misc/src/misc_kernels.cu
 * ======================================================================================== */

/* :49-66 */
void orc_spherical_contraction(int64_t n, const float* p, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        const float* q = p + 3 * i;
        const float len2 = fmaxf(fmaf(q[2], q[2], fmaf(q[1], q[1], q[0] * q[0])), 1.0f);
        const float s = (sqrtf(len2) * 2.0f - 1.0f) / len2 * 0.25f;
        for (int k = 0; k < 3; ++k) out[3 * i + k] = satf(fmaf(s, q[k], 0.5f));
    }
}

/* :68-79 — returns the mean-reduced loss; elementwise (optional) receives the per-element terms */
double orc_cauchy_loss(int64_t n, const float* input, const float* target, float* elementwise) {
    double sum = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        const float d = input[i] - target[i];
        const float e = log1pf(d * d * 12.5f) / (float)(uint32_t)n;
        if (elementwise) elementwise[i] = e;
        sum += e;
    }
    return sum;
}

/* :81-94 */
void orc_cauchy_loss_backward(int64_t n, float grad, const float* input, const float* target, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        const float d = input[i] - target[i];
        const float den = (float)(uint32_t)n * fmaf(12.5f * d, d, 1.0f);
        out[i] = 25.0f * d / fmaxf(den, 1.0e-12f) * grad;
    }
}

/* :6-47 — per-hash-level factor 0.2/len(level), zero below index 6144 */
float orc_weight_decay_factor(uint32_t idx) {
    static const uint32_t edge[11] = {210917376u, 177362944u, 143808512u, 110254080u, 76699648u, 43145216u,
                                      9590784u,   1202176u,   153600u,    22528u,     6144u};
    for (int k = 0; k < 10; ++k)
        if (idx >= edge[k + 1]) return 0.1f * 2.0f / (float)(edge[k] - edge[k + 1]);
    return 0.0f;
}

void orc_weight_decay(int64_t n, const float* weights, float* grads, int add) {
    for (int64_t i = 0; i < n; ++i) {
        const float f = orc_weight_decay_factor((uint32_t)i);
        if (add) grads[i] = fmaf(f, weights[i], grads[i]);
        else grads[i] = f * weights[i];
    }
}
