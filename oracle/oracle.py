"""TEST INFRASTRUCTURE — numpy front-end of the CPU oracle (oracle/inpc_oracle.c).

Only tests/, the smoke check and the cpu-baseline / reference legs of bench.py import this module.
The product package never does; it has no CPU path.

Every function works on host numpy arrays and mirrors one entry point of the reference backend
(INPCCudaBackend/INPCCudaBackend/torch_bindings/{rasterization,sampling,misc}.py) so that parity
tests read like calls into the reference.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libinpc_oracle.so"

BILINEAR, GAUSSIAN = 0, 1
TRAIN, RAW37, PREEXTRACTED = 0, 1, 2


def build(force: bool = False) -> Path:
    """Compile the C restatement with gcc (a second or two)."""
    src = _HERE / "inpc_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["make", "-s", "-C", str(_HERE), "oracle"])
    return _LIB_PATH


class _Cam(C.Structure):
    _fields_ = [("w2c", C.c_float * 16), ("cam", C.c_float * 3), ("width", C.c_int), ("height", C.c_int),
                ("fx", C.c_float), ("fy", C.c_float), ("cx", C.c_float), ("cy", C.c_float),
                ("near_plane", C.c_float), ("far_plane", C.c_float)]


class _Pcg(C.Structure):
    _fields_ = [("state", C.c_uint64), ("inc", C.c_uint64)]


@dataclass
class Camera:
    """Pinhole camera as the reference bindings read it from a NeRFICG `View`
    (torch_bindings/rasterization.py:116-128): +z forward, +x right, +y down."""
    w2c: np.ndarray            # (4,4) float32 row-major
    position: np.ndarray       # (3,) float32
    width: int
    height: int
    focal_x: float
    focal_y: float
    center_x: float
    center_y: float
    near_plane: float = 0.01
    far_plane: float = 100.0

    def c(self) -> _Cam:
        s = _Cam()
        w = np.ascontiguousarray(self.w2c, dtype=np.float32).reshape(16)
        for i in range(16):
            s.w2c[i] = float(w[i])
        p = np.asarray(self.position, dtype=np.float32).reshape(3)
        for i in range(3):
            s.cam[i] = float(p[i])
        s.width, s.height = int(self.width), int(self.height)
        s.fx, s.fy, s.cx, s.cy = self.focal_x, self.focal_y, self.center_x, self.center_y
        s.near_plane, s.far_plane = self.near_plane, self.far_plane
        return s


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(_LIB_PATH))
        _lib.orc_build_cdf.restype = C.c_float
        _lib.orc_cauchy_loss.restype = C.c_double
        _lib.orc_weight_decay_factor.restype = C.c_float
        _lib.orc_expected_counts.restype = C.c_int64
        _lib.orc_training_samples.restype = C.c_int64
        _lib.orc_pcg_next_uint.restype = C.c_uint32
    return _lib


def set_threads(n: int) -> None:
    os.environ["OMP_NUM_THREADS"] = str(n)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


@dataclass
class ForwardState:
    mode: int
    tile: int
    cam: Camera
    n: int
    positions: np.ndarray
    opacity: np.ndarray
    n_touched: np.ndarray
    bounds: np.ndarray
    screen: np.ndarray
    feat_view: np.ndarray
    depth: np.ndarray
    conic: np.ndarray | None
    sorted_points: np.ndarray
    inst_point: np.ndarray
    inst_tile: np.ndarray
    ranges: np.ndarray
    image: np.ndarray | None = None
    alpha: np.ndarray | None = None
    blending_weights: np.ndarray | None = None
    extra: dict = field(default_factory=dict)


def preprocess_and_order(mode, variant, cam: Camera, positions, features, opacities=None, scales=None,
                         sigma_world=0.0, sigma_cutoff=3.0, tile=8) -> ForwardState:
    L = lib()
    positions = _f32(positions).reshape(-1, 3)
    n = positions.shape[0]
    feats = np.ascontiguousarray(features, dtype=np.float16)
    assert feats.shape == (n, 37 if variant == RAW37 else 36), feats.shape
    opac = None if opacities is None else _f32(opacities).reshape(-1)
    sc = None if scales is None else _f32(scales).reshape(-1)
    n_touched = np.zeros(n, np.uint32)
    bounds = np.zeros((n, 4), np.uint16)
    screen = np.zeros((n, 2), np.float32)
    feat_view = np.zeros((n, 4), np.float32)
    depth = np.zeros(n, np.float32)
    opacity_out = np.zeros(n, np.float32)
    conic = np.zeros((n, 3), np.float32) if mode == GAUSSIAN else None
    cc = cam.c()
    L.orc_preprocess(C.c_int(mode), C.c_int(variant), C.byref(cc), C.c_int(tile), C.c_int64(n), _p(positions),
                     _p(feats), _p(opac), _p(sc), C.c_float(sigma_world), C.c_float(sigma_cutoff), _p(n_touched),
                     _p(bounds), _p(screen), _p(feat_view), _p(depth), _p(opacity_out), _p(conic))
    nv, ni = C.c_int64(0), C.c_int64(0)
    L.orc_order_counts(C.c_int64(n), _p(n_touched), C.byref(nv), C.byref(ni))
    gw, gh = -(-cam.width // tile), -(-cam.height // tile)
    sorted_points = np.zeros(max(nv.value, 1), np.uint32)
    inst_point = np.zeros(max(ni.value, 1), np.uint32)
    inst_tile = np.zeros(max(ni.value, 1), np.uint32)
    ranges = np.zeros((gw * gh, 2), np.uint32)
    L.orc_order(C.c_int64(n), C.c_int(tile), C.c_int(cam.width), C.c_int(cam.height), _p(n_touched), _p(bounds),
                _p(depth), _p(sorted_points), _p(inst_point), _p(inst_tile), _p(ranges))
    return ForwardState(mode, tile, cam, n, positions, opacity_out, n_touched, bounds, screen, feat_view, depth,
                        conic, sorted_points[:nv.value], inst_point[:ni.value], inst_tile[:ni.value], ranges)


def rasterize_forward(mode, cam: Camera, positions, features, opacities, tile=8) -> ForwardState:
    """INPCRasterizer.forward (torch_bindings/rasterization.py:136-149)."""
    st = preprocess_and_order(mode, TRAIN, cam, positions, features, opacities, tile=tile)
    L = lib()
    H, W = cam.height, cam.width
    st.image = np.zeros((4, H, W), np.float32)
    st.alpha = np.zeros((1, H, W), np.float32)
    st.blending_weights = np.zeros(st.n, np.float32)
    cc = cam.c()
    L.orc_blend_forward(C.c_int(mode), C.byref(cc), C.c_int(tile), C.c_int64(st.n), _p(st.ranges), _p(st.inst_point),
                        _p(st.screen), _p(st.feat_view), _p(st.opacity), _p(st.conic), _p(st.image), _p(st.alpha),
                        _p(st.blending_weights))
    return st


def rasterize_backward(st: ForwardState, grad_image, grad_alpha):
    """_Rasterize.backward (torch_bindings/rasterization.py:80-101): returns
    grad_features (n,36) float16, grad_opacities (n,1) float32 and the intermediate (n,4) view gradient."""
    L = lib()
    gi = _f32(grad_image).reshape(4, st.cam.height, st.cam.width)
    ga = _f32(grad_alpha).reshape(1, st.cam.height, st.cam.width)
    gfv = np.zeros((st.n, 4), np.float32)
    go = np.zeros((st.n, 1), np.float32)
    gfeat = np.zeros((st.n, 36), np.float16)
    cc = st.cam.c()
    L.orc_blend_backward(C.c_int(st.mode), C.byref(cc), C.c_int(st.tile), C.c_int64(st.n), _p(st.ranges),
                         _p(st.inst_point), _p(st.screen), _p(st.feat_view), _p(st.opacity), _p(st.conic), _p(gi),
                         _p(ga), _p(st.image), _p(st.alpha), _p(gfv), _p(go))
    L.orc_preprocess_backward(C.byref(cc), C.c_int64(st.n), _p(st.positions), _p(st.n_touched), _p(gfv), _p(gfeat))
    return gfeat, go, gfv


def _inference(st: ForwardState, sigma_cutoff):
    L = lib()
    H, W = st.cam.height, st.cam.width
    image = np.zeros((4, H, W), np.float32)
    depth = np.zeros((1, H, W), np.float32)
    alpha = np.zeros((1, H, W), np.float32)
    thr = float(np.exp(np.float32(-0.5) * np.float32(sigma_cutoff) * np.float32(sigma_cutoff)))
    cc = st.cam.c()
    L.orc_blend_inference(C.c_int(st.mode), C.byref(cc), C.c_int(st.tile), _p(st.ranges), _p(st.inst_point),
                          _p(st.screen), _p(st.feat_view), _p(st.opacity), _p(st.depth), _p(st.conic),
                          C.c_float(thr), _p(image), _p(depth), _p(alpha))
    st.image, st.alpha = image, alpha
    st.extra["depth_image"] = depth
    return image, depth, alpha


def render(mode, cam: Camera, positions, features_raw, sigma_world, sigma_cutoff, tile=8):
    """INPCRasterizer.render (torch_bindings/rasterization.py:151-167); sigma_world is the product
    sigma_world_scale * 0.05 / focal_y that the binding forms."""
    st = preprocess_and_order(mode, RAW37, cam, positions, features_raw, None, None, sigma_world, sigma_cutoff, tile)
    return _inference(st, sigma_cutoff) + (st,)


def render_preextracted(mode, cam: Camera, positions, features, opacities, scales, sigma_world, sigma_cutoff,
                        tile=8):
    """INPCRasterizer.render_preextracted (torch_bindings/rasterization.py:169-189)."""
    st = preprocess_and_order(mode, PREEXTRACTED, cam, positions, features, opacities, scales, sigma_world,
                              sigma_cutoff, tile)
    return _inference(st, sigma_cutoff) + (st,)


# ----------------------------------------------------------------------------- feature rows
# (n, C) fp32 features blended as they are.  The blend treats channels independently, so C channels
# are C/4 runs of the four-channel restatement over the same ordering: exactly the "C/4 reference
# passes" by which the reference itself can be run on such input.

def _rows_state(cam: Camera, positions, opacities, tile) -> ForwardState:
    n = np.asarray(positions).reshape(-1, 3).shape[0]
    return preprocess_and_order(BILINEAR, TRAIN, cam, positions, np.zeros((n, 36), np.float16), opacities, tile=tile)


def rasterize_rows_forward(cam: Camera, positions, features, opacities, tile=8) -> ForwardState:
    feats = _f32(features)
    n, ch = feats.shape
    assert ch % 4 == 0
    st = _rows_state(cam, positions, opacities, tile)
    L = lib()
    H, W = cam.height, cam.width
    st.image = np.zeros((ch, H, W), np.float32)
    st.alpha = np.zeros((1, H, W), np.float32)
    st.blending_weights = np.zeros(n, np.float32)
    st.extra["features"] = feats
    cc = cam.c()
    for g in range(ch // 4):
        fv = np.ascontiguousarray(feats[:, 4 * g:4 * g + 4])
        img = np.zeros((4, H, W), np.float32)
        L.orc_blend_forward(C.c_int(BILINEAR), C.byref(cc), C.c_int(tile), C.c_int64(n), _p(st.ranges), _p(st.inst_point),
                            _p(st.screen), _p(fv), _p(st.opacity), None, _p(img), _p(st.alpha), _p(st.blending_weights))
        st.image[4 * g:4 * g + 4] = img
    return st


def rasterize_rows_backward(st: ForwardState, grad_image, grad_alpha):
    """grad_features (n,C) float32 and grad_opacities (n,1) float32.  The opacity gradient is linear in
    (grad_image, grad_alpha): channel group g contributes through its own four gradient planes, the
    alpha term is added once (with group 0)."""
    L = lib()
    feats = st.extra["features"]
    n, ch = feats.shape
    H, W = st.cam.height, st.cam.width
    gi = _f32(grad_image).reshape(ch, H, W)
    ga = _f32(grad_alpha).reshape(1, H, W)
    gf = np.zeros((n, ch), np.float32)
    go = np.zeros((n, 1), np.float64)
    cc = st.cam.c()
    for g in range(ch // 4):
        fv = np.ascontiguousarray(feats[:, 4 * g:4 * g + 4])
        gfv = np.zeros((n, 4), np.float32)
        gop = np.zeros((n, 1), np.float32)
        gig = np.ascontiguousarray(gi[4 * g:4 * g + 4])
        gag = ga if g == 0 else np.zeros_like(ga)
        img = np.ascontiguousarray(st.image[4 * g:4 * g + 4])
        L.orc_blend_backward(C.c_int(BILINEAR), C.byref(cc), C.c_int(st.tile), C.c_int64(n), _p(st.ranges),
                             _p(st.inst_point), _p(st.screen), _p(fv), _p(st.opacity), None, _p(gig), _p(gag), _p(img),
                             _p(st.alpha), _p(gfv), _p(gop))
        gf[:, 4 * g:4 * g + 4] = gfv
        go += gop
    return gf, go.astype(np.float32)


def render_rows(cam: Camera, positions, features, opacities, tile=8):
    feats = _f32(features)
    n, ch = feats.shape
    st = _rows_state(cam, positions, opacities, tile)
    L = lib()
    H, W = cam.height, cam.width
    image = np.zeros((ch, H, W), np.float32)
    depth = np.zeros((1, H, W), np.float32)
    alpha = np.zeros((1, H, W), np.float32)
    cc = cam.c()
    for g in range(ch // 4):
        fv = np.ascontiguousarray(feats[:, 4 * g:4 * g + 4])
        img = np.zeros((4, H, W), np.float32)
        L.orc_blend_inference(C.c_int(BILINEAR), C.byref(cc), C.c_int(tile), _p(st.ranges), _p(st.inst_point), _p(st.screen),
                              _p(fv), _p(st.opacity), _p(st.depth), None, C.c_float(0.0), _p(img), _p(depth), _p(alpha))
        image[4 * g:4 * g + 4] = img
    return image, depth, alpha, st


# ----------------------------------------------------------------------------- sampler

def viewpoint_weights(cam: Camera, centers, levels, weights, initial_size):
    """compute_viewpoint_weights (torch_bindings/sampling.py:9-34)."""
    centers = _f32(centers).reshape(-1, 3)
    levels = np.ascontiguousarray(levels, dtype=np.int32)
    weights = _f32(weights)
    out = np.zeros(centers.shape[0], np.float32)
    cc = cam.c()
    lib().orc_viewpoint_weights(C.byref(cc), C.c_int64(centers.shape[0]), _p(centers), _p(levels), _p(weights),
                                C.c_float(initial_size), _p(out))
    return out


def build_cdf(vw):
    vw = _f32(vw)
    cdf = np.zeros_like(vw)
    s = lib().orc_build_cdf(C.c_int64(vw.shape[0]), _p(vw), _p(cdf))
    return cdf, float(s)


def draw_leaves(cdf, u):
    cdf, u = _f32(cdf), _f32(u)
    out = np.zeros(u.shape[0], np.int64)
    lib().orc_draw_leaves(_p(cdf), C.c_uint32(cdf.shape[0]), _p(u), C.c_int64(u.shape[0]), _p(out))
    return out


def philox4x32(ctr, key):
    c = (C.c_uint32 * 4)(*[int(x) & 0xFFFFFFFF for x in ctr])
    k = (C.c_uint32 * 2)(*[int(x) & 0xFFFFFFFF for x in key])
    o = (C.c_uint32 * 4)()
    lib().orc_philox4x32(c, k, o)
    return [int(x) for x in o]


def training_samples(cam: Camera, seed, call, cdf, centers, levels, initial_size, n):
    cdf, centers = _f32(cdf), _f32(centers).reshape(-1, 3)
    levels = np.ascontiguousarray(levels, dtype=np.int32)
    pos = np.zeros((n, 3), np.float32)
    idx = np.zeros(n, np.int64)
    cc = cam.c()
    ex = lib().orc_training_samples(C.byref(cc), C.c_uint64(seed), C.c_uint64(call), _p(cdf), C.c_uint32(cdf.shape[0]),
                                    _p(centers), _p(levels), C.c_float(initial_size), C.c_int64(n), _p(pos), _p(idx))
    return pos, idx, int(ex)


def samples(seed, call, cdf, centers, levels, initial_size, n):
    cdf, centers = _f32(cdf), _f32(centers).reshape(-1, 3)
    levels = np.ascontiguousarray(levels, dtype=np.int32)
    pos = np.zeros((n, 3), np.float32)
    idx = np.zeros(n, np.int64)
    lib().orc_samples(C.c_uint64(seed), C.c_uint64(call), _p(cdf), C.c_uint32(cdf.shape[0]), _p(centers), _p(levels),
                      C.c_float(initial_size), C.c_int64(n), _p(pos), _p(idx))
    return pos, idx


def expected_counts(vw, vw_sum, n_samples):
    vw = _f32(vw)
    counts = np.zeros(vw.shape[0], np.int32)
    total = lib().orc_expected_counts(C.c_int64(vw.shape[0]), _p(vw), C.c_float(vw_sum), C.c_uint32(n_samples),
                                      _p(counts))
    return counts, int(total)


def expected_samples(seed, call, counts, centers, levels, initial_size, n_multi):
    counts = np.ascontiguousarray(counts, dtype=np.int32)
    centers = _f32(centers).reshape(-1, 3)
    levels = np.ascontiguousarray(levels, dtype=np.int32)
    n_created = int(counts.sum())
    pos = np.zeros((n_created * n_multi, 3), np.float32)
    lib().orc_expected_samples(C.c_uint64(seed), C.c_uint64(call), C.c_int64(counts.shape[0]), _p(counts),
                               _p(centers), _p(levels), C.c_float(initial_size), C.c_int64(n_created),
                               C.c_int64(n_multi), _p(pos))
    return pos


class RefPcg:
    """The reference's host-side pcg32 (sampling/include/pcg32.h:42-201), for restating its
    deterministic sampler variants."""

    def __init__(self, seed: int):
        self.g = _Pcg()
        lib().orc_pcg_seed(C.byref(self.g), C.c_uint64(seed), C.c_uint64(1))

    def next_uint(self) -> int:
        return int(lib().orc_pcg_next_uint(C.byref(self.g)))

    def create_samples(self, cdf, centers, levels, initial_size, n, fused=True):
        cdf, centers = _f32(cdf), _f32(centers).reshape(-1, 3)
        levels = np.ascontiguousarray(levels, dtype=np.int32)
        pos = np.zeros((n, 3), np.float32)
        u = np.zeros(n, np.float32)
        leaf = np.zeros(n, np.int64)
        lib().orc_ref_create_samples(C.byref(self.g), _p(cdf), C.c_uint32(cdf.shape[0]), _p(centers), _p(levels),
                                     C.c_float(initial_size), C.c_int64(n), C.c_int(int(fused)), _p(pos), _p(u),
                                     _p(leaf))
        return pos, u, leaf

    def expected_samples(self, counts, centers, levels, initial_size, n_multi, fused=True):
        counts = np.ascontiguousarray(counts, dtype=np.int32)
        centers = _f32(centers).reshape(-1, 3)
        levels = np.ascontiguousarray(levels, dtype=np.int32)
        n_created = int(counts.sum())
        pos = np.zeros((n_created * n_multi, 3), np.float32)
        lib().orc_ref_expected_samples(C.byref(self.g), C.c_int64(counts.shape[0]), _p(counts), _p(centers),
                                       _p(levels), C.c_float(initial_size), C.c_int64(n_created), C.c_int64(n_multi),
                                       C.c_int(int(fused)), _p(pos))
        return pos


# ----------------------------------------------------------------------------- misc

def spherical_contraction(p):
    p = _f32(p).reshape(-1, 3)
    out = np.zeros_like(p)
    lib().orc_spherical_contraction(C.c_int64(p.shape[0]), _p(p), _p(out))
    return out


def cauchy_loss(inp, tgt):
    inp, tgt = _f32(inp).reshape(-1), _f32(tgt).reshape(-1)
    return float(lib().orc_cauchy_loss(C.c_int64(inp.shape[0]), _p(inp), _p(tgt), None))


def cauchy_loss_backward(grad, inp, tgt):
    shape = np.shape(inp)
    inp, tgt = _f32(inp).reshape(-1), _f32(tgt).reshape(-1)
    out = np.zeros_like(inp)
    lib().orc_cauchy_loss_backward(C.c_int64(inp.shape[0]), C.c_float(grad), _p(inp), _p(tgt), _p(out))
    return out.reshape(shape)


def weight_decay(weights, grads=None, offset_check=None):
    w = _f32(weights).reshape(-1)
    add = grads is not None
    g = _f32(grads).reshape(-1).copy() if add else np.zeros_like(w)
    lib().orc_weight_decay(C.c_int64(w.shape[0]), _p(w), _p(g), C.c_int(int(add)))
    return g


def weight_decay_factor(idx: int) -> float:
    return float(lib().orc_weight_decay_factor(C.c_uint32(idx)))


# ----------------------------------------------------------------------------- octree structure
# numpy restatements of the reference's torch code (no native kernel exists for these in the reference)

def leaf_update(leaf_weights, leaf_scores, indices, weights, decay=np.float32(0.9968)):
    """ProbabilityField.update (Modules/ProbabilityField.py:146-157)."""
    lw = _f32(leaf_weights) * np.float32(decay)
    ls = _f32(leaf_scores) * np.float32(decay)
    w = _f32(weights).reshape(-1)
    idx = np.asarray(indices, dtype=np.int64).reshape(-1)
    mx = np.zeros_like(lw)
    mn = np.full_like(lw, np.inf)
    np.maximum.at(mx, idx, w)
    np.minimum.at(mn, idx, w)
    mn[np.isinf(mn)] = 0.0
    return np.maximum(lw, mx), np.maximum(ls, np.clip(mx - mn, 0.0, 1.0))


def leaf_prune(centers, levels, weights, scores, threshold):
    """ProbabilityField.prune (Modules/ProbabilityField.py:159-165)."""
    mask = _f32(weights) > np.float32(threshold)
    return (_f32(centers).reshape(-1, 3)[mask], np.asarray(levels, np.int32)[mask], _f32(weights)[mask], _f32(scores)[mask])


def leaf_subdivide(centers, levels, weights, scores, threshold, initial_size, max_level=6, max_leaves=16_777_216):
    """ProbabilityField.subdivide (Modules/ProbabilityField.py:217-257); None when the cap would be exceeded."""
    centers = _f32(centers).reshape(-1, 3)
    levels = np.asarray(levels, np.int32)
    weights, scores = _f32(weights), _f32(scores)
    valid = (scores > np.float32(threshold)) & (levels < max_level)
    nv = int(valid.sum())
    if nv * 8 + (centers.shape[0] - nv) > max_leaves:
        return None
    new_centers = np.repeat(centers[valid], 8, axis=0)
    new_levels = np.repeat(levels[valid] + 1, 8)
    new_weights = np.repeat(weights[valid], 8)
    offset = (np.float32(initial_size) / (2 ** (new_levels.astype(np.int64) + 1)).astype(np.float32)).astype(np.float32)
    new_centers[0::2, 0] -= offset[0::2]
    new_centers[1::2, 0] += offset[1::2]
    for k in range(4):
        if k < 2:
            new_centers[k::4, 1] -= offset[k::4]
        else:
            new_centers[k::4, 1] += offset[k::4]
    for k in range(8):
        if k < 4:
            new_centers[k::8, 2] -= offset[k::8]
        else:
            new_centers[k::8, 2] += offset[k::8]
    return (np.concatenate([centers[~valid], new_centers]), np.concatenate([levels[~valid], new_levels]),
            np.concatenate([weights[~valid], new_weights]), np.concatenate([scores[~valid], np.zeros_like(new_weights)]))


# ----------------------------------------------------------------------------- image composition
# numpy restatements of the reference renderer's torch element-wise chains (one rounding per op)

def compose_background(image, alpha, background):
    """Renderer.py:80: feature_image + (1 - alpha_image) * background."""
    image, alpha, background = _f32(image), _f32(alpha), _f32(background)
    return image + (np.float32(1.0) - alpha.reshape(1, *image.shape[1:])) * background


def multisample_resolve(samples, background, premultiplied=True):
    """Renderer.py:105-125 for a list of (feature_image, depth_image, alpha_image) multisamples.
    Returns feature_image, depth, alpha, alpha_sum."""
    n = max(1, len(samples))
    fi = di = ai = None
    for k, (f, d, a) in enumerate(samples):
        f, d, a = _f32(f).copy(), _f32(d).copy(), _f32(a).copy()
        if not premultiplied and n > 1:
            with np.errstate(divide="ignore", invalid="ignore"):
                f = np.where(a > 0.0, f / a, np.float32(0.0)).astype(np.float32)
        if k == 0:
            fi, di, ai = f, d, a
        else:
            fi += f
            di += d
            ai += a
    factor = np.float32(1.0 / n)
    fi *= factor
    di *= factor
    alpha_sum = np.clip(ai, 0.0, 1.0)
    ai = ai * factor
    if not premultiplied and n > 1:
        fi *= ai
    if background is not None:
        fi += (np.float32(1.0) - ai) * _f32(background)
    return fi, di, ai, alpha_sum


# ----------------------------------------------------------------------------- global point cloud

def halton_element(index: int, base: int) -> float:
    """utils.py:36-46 (double precision, as Python floats)."""
    result, f, i = 0.0, 1.0 / base, index
    while i > 0:
        result += f * (i % base)
        i //= base
        f /= base
    return result


def halton_samples(counts, centers, levels, initial_size):
    """ProbabilityField.py:131-140 with utils.py:49-64: `counts[l]` quasi-random positions per leaf."""
    counts = np.asarray(counts, dtype=np.int64)
    centers = _f32(centers).reshape(-1, 3)
    levels = np.asarray(levels, dtype=np.int64)
    cell = np.repeat(np.arange(counts.shape[0]), counts)
    offsets = np.cumsum(counts) - counts
    h = np.arange(int(counts.sum())) - offsets[cell]
    table = np.zeros((int(h.max()) + 1 if h.size else 0, 3), np.float32)
    for i in range(table.shape[0]):
        for j, base in enumerate((2, 3, 5)):
            table[i, j] = halton_element(i + 1, base)
    coords = table[h]
    cell_size = (np.float32(initial_size) / (2 ** levels[cell]).astype(np.float32)).astype(np.float32)[:, None]
    initial = centers[cell]
    samples = initial - (cell_size / np.float32(2)) + coords * cell_size
    single = np.repeat(counts == 1, counts)
    samples[single] = initial[single]
    return samples.astype(np.float32)
