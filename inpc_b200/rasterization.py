"""Host-side mirror of the reference rasterizer bindings
(INPCCudaBackend/INPCCudaBackend/torch_bindings/rasterization.py): same class names, call
signatures, tensor shapes/dtypes and return values, on top of the C ABI of libinpc_b200.

PyTorch supplies device memory, the current stream and autograd plumbing only; every computation
is a kernel of the shared library.
"""
from __future__ import annotations

import ctypes as C
import warnings
from enum import Enum
from typing import Any, NamedTuple

import torch
from torch.autograd.function import once_differentiable

from . import _cabi

# Tile edge used by the blend: 8 is the reference's tiling (its tile ranges and per-tile lists) and
# also the faster one on B200; 16 halves the number of duplicated instances.  Images, weights and
# gradients do not depend on it beyond summation order.
DEFAULT_TILE_SIZE = 8


class RasterizerMode(Enum):
    BILINEAR = 0
    GAUSSIAN = 1


class RasterizerSettings(NamedTuple):
    w2c: torch.Tensor
    cam_position: torch.Tensor
    mode: RasterizerMode
    width: int
    height: int
    focal_x: float
    focal_y: float
    center_x: float
    center_y: float
    near_plane: float
    far_plane: float

    def as_tuple(self) -> tuple:
        return (self.w2c, self.cam_position, self.mode.value, self.width, self.height, self.focal_x, self.focal_y,
                self.center_x, self.center_y, self.near_plane, self.far_plane)


def _cuda_f32(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32, got {t.dtype}")
    return t.contiguous()


def _cuda_f16(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.float16:
        raise TypeError(f"{name} must be float16, got {t.dtype}")
    return t.contiguous()


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None or t.numel() == 0 else t.data_ptr())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _ViewArg:
    """Keeps the device tensors of an `inpc_view` alive while the struct is in use."""

    def __init__(self, s: RasterizerSettings, device: torch.device):
        self.w2c = _cuda_f32(s.w2c.to(device), "w2c")
        self.pos = _cuda_f32(s.cam_position.to(device), "cam_position")
        if self.w2c.numel() != 16 or self.pos.numel() != 3:
            raise ValueError("w2c must have 16 elements and cam_position 3")
        self.c = _cabi.View(self.w2c.data_ptr(), self.pos.data_ptr(), int(s.width), int(s.height), float(s.focal_x),
                            float(s.focal_y), float(s.center_x), float(s.center_y), float(s.near_plane),
                            float(s.far_plane))


class _Blobs:
    """Scratch allocator handed to the C ABI: torch byte tensors, kept alive by this object.  Plays
    the role of the three growable byte tensors of the reference's forward_wrapper
    (rasterization/src/rasterization_api.cu:47-52)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.point: torch.Tensor | None = None
        self.instance: torch.Tensor | None = None
        self.error: BaseException | None = None
        self.cb_point = _cabi.ALLOC_FN(self._alloc_point)
        self.cb_instance = _cabi.ALLOC_FN(self._alloc_instance)

    def _alloc(self, nbytes: int) -> torch.Tensor:
        return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=self.device)

    def _alloc_point(self, _user, nbytes):
        try:
            self.point = self._alloc(nbytes)
            return self.point.data_ptr()
        except BaseException as e:  # surfaced by the caller after the C call returns INPC_E_ALLOC
            self.error = e
            return 0

    def _alloc_instance(self, _user, nbytes):
        try:
            self.instance = self._alloc(nbytes)
            return self.instance.data_ptr()
        except BaseException as e:
            self.error = e
            return 0


def _check(status: int, blobs: _Blobs | None = None) -> None:
    if blobs is not None:
        # the ctypes callbacks hold bound methods of `blobs`: drop them, or the reference cycle keeps
        # the scratch tensors alive until the cyclic garbage collector runs
        blobs.cb_point = blobs.cb_instance = None
    if status != 0 and blobs is not None and blobs.error is not None:
        raise blobs.error
    _cabi.check(status)


def resolve_counts(state) -> None:
    """Fills in `n_visible` / `n_instances` of a state whose forward left them on the device (one small copy and a
    synchronisation of the current stream)."""
    _check(_cabi.lib().inpc_raster_resolve(C.byref(state), _stream()))


def forward_with_state(positions: torch.Tensor, features: torch.Tensor, opacities: torch.Tensor,
                       rasterizer_settings: RasterizerSettings, tile_size: int = DEFAULT_TILE_SIZE, resolve: bool = True):
    """Training forward without autograd; also returns the C state and the scratch blobs.  `resolve` fetches the
    visible / instance counts (a host synchronisation the autograd path does without)."""
    positions = _cuda_f32(positions, "positions")
    features = _cuda_f16(features, "features")
    opacities = _cuda_f32(opacities, "opacities")
    n = positions.shape[0]
    if positions.dim() != 2 or positions.shape[1] != 3:
        raise ValueError(f"positions must be (N,3), got {tuple(positions.shape)}")
    if features.shape != (n, 36):
        raise ValueError(f"features must be (N,36), got {tuple(features.shape)}")
    if opacities.numel() != n:
        raise ValueError(f"opacities must hold N={n} values, got {tuple(opacities.shape)}")
    dev = positions.device
    s = rasterizer_settings
    with torch.cuda.device(dev):
        view = _ViewArg(s, dev)
        image = torch.empty((4, s.height, s.width), dtype=torch.float32, device=dev)
        alpha = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
        blending_weights = torch.empty((n,), dtype=torch.float32, device=dev)
        blobs = _Blobs(dev)
        state = _cabi.RasterState()
        _check(_cabi.lib().inpc_rasterize_forward(
            s.mode.value, int(tile_size), C.byref(view.c), n, _ptr(positions), _ptr(features), _ptr(opacities),
            _ptr(image), _ptr(alpha), _ptr(blending_weights), blobs.cb_point, blobs.cb_instance, None,
            C.byref(state), _stream()), blobs)
        if resolve:
            resolve_counts(state)
    return image, alpha, blending_weights, state, blobs, (positions, opacities)


class _Rasterize(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, positions: torch.Tensor, features: torch.Tensor, opacities: torch.Tensor,
                rasterizer_settings: RasterizerSettings, tile_size: int = DEFAULT_TILE_SIZE):
        image, alpha, blending_weights, state, blobs, (positions, opacities) = forward_with_state(
            positions, features, opacities, rasterizer_settings, tile_size, resolve=False)
        ctx.save_for_backward(image, alpha, positions, opacities, blobs.point, blobs.instance)
        ctx.rasterizer_settings = rasterizer_settings
        ctx.raster_state = state
        ctx.n_instances = int(state.n_instances)
        ctx.mark_non_differentiable(blending_weights)
        ctx.set_materialize_grads(False)
        return image, alpha, blending_weights

    @staticmethod
    @once_differentiable
    def backward(ctx: Any, grad_image: torch.Tensor, grad_alpha: torch.Tensor, _):
        image, alpha, positions, opacities, point_blob, instance_blob = ctx.saved_tensors
        s = ctx.rasterizer_settings
        dev = positions.device
        n = positions.shape[0]
        # set_materialize_grads(False): an unused output arrives as None
        grad_image = torch.zeros_like(image) if grad_image is None else _cuda_f32(grad_image, "grad_image")
        grad_alpha = torch.zeros_like(alpha) if grad_alpha is None else _cuda_f32(grad_alpha, "grad_alpha")
        with torch.cuda.device(dev):
            view = _ViewArg(s, dev)
            grad_features_view = torch.empty((n, 33), dtype=torch.float32, device=dev)   # per-point gradient slots
            grad_features = torch.empty((n, 36), dtype=torch.float16, device=dev)
            grad_opacities = torch.empty((n, 1), dtype=torch.float32, device=dev)
            _check(_cabi.lib().inpc_rasterize_backward(
                C.byref(ctx.raster_state), C.byref(view.c), _ptr(grad_image), _ptr(grad_alpha), _ptr(image),
                _ptr(alpha), _ptr(positions), _ptr(opacities), _ptr(grad_features_view), _ptr(grad_features),
                _ptr(grad_opacities), _stream()))
        return None, grad_features, grad_opacities, None, None


def _check_rows(positions, features, opacities):
    positions = _cuda_f32(positions, "positions")
    features = _cuda_f32(features, "features")
    opacities = _cuda_f32(opacities, "opacities")
    n = positions.shape[0]
    if positions.dim() != 2 or positions.shape[1] != 3:
        raise ValueError(f"positions must be (N,3), got {tuple(positions.shape)}")
    if features.dim() != 2 or features.shape[0] != n or features.shape[1] not in (4, 8, 16, 32):
        raise ValueError(f"features must be (N,C) with C in (4, 8, 16, 32), got {tuple(features.shape)}")
    if opacities.numel() != n:
        raise ValueError(f"opacities must hold N={n} values, got {tuple(opacities.shape)}")
    return positions, features, opacities


class _RasterizeRows(torch.autograd.Function):
    """Bilinear training rasterisation of (N,C) fp32 feature rows into a (C,H,W) image."""

    @staticmethod
    def forward(ctx: Any, positions: torch.Tensor, features: torch.Tensor, opacities: torch.Tensor,
                rasterizer_settings: RasterizerSettings, tile_size: int = DEFAULT_TILE_SIZE):
        positions, features, opacities = _check_rows(positions, features, opacities)
        n, channels = features.shape
        dev = positions.device
        s = rasterizer_settings
        with torch.cuda.device(dev):
            view = _ViewArg(s, dev)
            image = torch.empty((channels, s.height, s.width), dtype=torch.float32, device=dev)
            alpha = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            blending_weights = torch.empty((n,), dtype=torch.float32, device=dev)
            blobs = _Blobs(dev)
            state = _cabi.RasterState()
            _check(_cabi.lib().inpc_rasterize_rows_forward(
                int(tile_size), C.byref(view.c), n, _ptr(positions), _ptr(features), int(channels), _ptr(opacities),
                _ptr(image), _ptr(alpha), _ptr(blending_weights), blobs.cb_point, blobs.cb_instance, None,
                C.byref(state), _stream()), blobs)
        ctx.save_for_backward(image, alpha, features, blobs.point, blobs.instance)
        ctx.rasterizer_settings = rasterizer_settings
        ctx.raster_state = state
        ctx.mark_non_differentiable(blending_weights)
        ctx.set_materialize_grads(False)
        return image, alpha, blending_weights

    @staticmethod
    @once_differentiable
    def backward(ctx: Any, grad_image: torch.Tensor, grad_alpha: torch.Tensor, _):
        image, alpha, features, point_blob, instance_blob = ctx.saved_tensors
        s = ctx.rasterizer_settings
        dev = features.device
        grad_image = torch.zeros_like(image) if grad_image is None else _cuda_f32(grad_image, "grad_image")
        grad_alpha = torch.zeros_like(alpha) if grad_alpha is None else _cuda_f32(grad_alpha, "grad_alpha")
        with torch.cuda.device(dev):
            view = _ViewArg(s, dev)
            grad_features = torch.empty_like(features)
            grad_opacities = torch.empty((features.shape[0], 1), dtype=torch.float32, device=dev)
            _check(_cabi.lib().inpc_rasterize_rows_backward(
                C.byref(ctx.raster_state), C.byref(view.c), _ptr(grad_image), _ptr(grad_alpha), _ptr(image),
                _ptr(alpha), _ptr(features), _ptr(grad_features), _ptr(grad_opacities), _stream()))
        return None, grad_features, grad_opacities, None, None


class INPCRasterizer(torch.nn.Module):
    """Drop-in for the reference's INPCRasterizer (torch_bindings/rasterization.py:104-189)."""

    def __init__(self, tile_size: int = DEFAULT_TILE_SIZE) -> None:
        super().__init__()
        if tile_size not in (8, 16):
            raise ValueError("tile_size must be 8 or 16")
        self.tile_size = tile_size

    @staticmethod
    def extract_settings(view, mode: int) -> RasterizerSettings:
        cam = view.camera
        for attr in ("width", "height", "focal_x", "focal_y", "center_x", "center_y", "near_plane", "far_plane"):
            if not hasattr(cam, attr):
                raise NotImplementedError(f"camera without `{attr}`: only perspective cameras are supported")
        if getattr(cam, "distortion", None) is not None:
            warnings.warn("rasterizer ignores all distortion parameters")
        try:
            rasterizer_mode = RasterizerMode(mode)
        except ValueError:
            warnings.warn(f"invalid rasterizer mode {mode}, defaulting to BILINEAR")
            rasterizer_mode = RasterizerMode.BILINEAR
        return RasterizerSettings(view.w2c, view.position, rasterizer_mode, cam.width, cam.height, cam.focal_x,
                                  cam.focal_y, cam.center_x, cam.center_y, cam.near_plane, cam.far_plane)

    @staticmethod
    def extract_base_sigma_world(camera) -> float:
        if not hasattr(camera, "focal_y"):
            raise NotImplementedError
        return 0.05 / camera.focal_y  # screen-space sigma of 5 px at the default near plane (0.01)

    def forward(self, view, mode: int, positions: torch.Tensor, features: torch.Tensor, opacities: torch.Tensor):
        return _Rasterize.apply(positions, features, opacities, self.extract_settings(view, mode), self.tile_size)

    def _render_common(self, positions):
        positions = _cuda_f32(positions, "positions")
        if positions.dim() != 2 or positions.shape[1] != 3:
            raise ValueError(f"positions must be (N,3), got {tuple(positions.shape)}")
        return positions

    @torch.no_grad()
    def render(self, view, mode: int, positions: torch.Tensor, features_raw: torch.Tensor, sigma_world_scale: float,
               sigma_cutoff: float):
        s = self.extract_settings(view, mode)
        positions = self._render_common(positions)
        features_raw = _cuda_f16(features_raw, "features_raw")
        n = positions.shape[0]
        if features_raw.shape != (n, 37):
            raise ValueError(f"features_raw must be (N,37), got {tuple(features_raw.shape)}")
        dev = positions.device
        with torch.cuda.device(dev):
            varg = _ViewArg(s, dev)
            image = torch.empty((4, s.height, s.width), dtype=torch.float32, device=dev)
            depth = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            alpha = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            blobs = _Blobs(dev)
            _check(_cabi.lib().inpc_render(
                s.mode.value, self.tile_size, C.byref(varg.c), n, _ptr(positions), _ptr(features_raw),
                float(sigma_world_scale * self.extract_base_sigma_world(view.camera)), float(sigma_cutoff),
                _ptr(image), _ptr(depth), _ptr(alpha), blobs.cb_point, blobs.cb_instance, None, _stream()), blobs)
            # the blobs must outlive the kernels already enqueued on this stream
            for b in (blobs.point, blobs.instance):
                if b is not None:
                    b.record_stream(torch.cuda.current_stream())
        return image, depth, alpha

    @torch.no_grad()
    def render_multi(self, view, sample_sets):
        """Bilinear inference over several sample sets `(positions (N_j,3) f32, features_raw (N_j,37) f16)` of one view
        in ONE launch sequence: returns images (k,4,H,W), depths (k,1,H,W), alphas (k,1,H,W), set by set bit for bit what
        `render` gives.  Needs 8x8 tiles and at most 8 sets."""
        if self.tile_size != 8:
            raise ValueError("render_multi needs tile_size 8")
        s = self.extract_settings(view, 0)
        sets = [(self._render_common(p), _cuda_f16(f, "features_raw")) for p, f in sample_sets]
        k = len(sets)
        if not 1 <= k <= 8:
            raise ValueError(f"render_multi takes 1 to 8 sample sets, got {k}")
        for p, f in sets:
            if f.shape != (p.shape[0], 37):
                raise ValueError(f"features_raw must be (N,37), got {tuple(f.shape)}")
        dev = sets[0][0].device
        with torch.cuda.device(dev):
            varg = _ViewArg(s, dev)
            images = torch.empty((k, 4, s.height, s.width), dtype=torch.float32, device=dev)
            depths = torch.empty((k, 1, s.height, s.width), dtype=torch.float32, device=dev)
            alphas = torch.empty((k, 1, s.height, s.width), dtype=torch.float32, device=dev)
            n_points = (C.c_int64 * k)(*[p.shape[0] for p, _ in sets])
            pos_ptrs = (C.c_void_p * k)(*[p.data_ptr() if p.numel() else 0 for p, _ in sets])
            feat_ptrs = (C.c_void_p * k)(*[f.data_ptr() if f.numel() else 0 for _, f in sets])
            blobs = _Blobs(dev)
            _check(_cabi.lib().inpc_render_multi(self.tile_size, C.byref(varg.c), k, n_points, pos_ptrs, feat_ptrs, _ptr(images),
                                                 _ptr(depths), _ptr(alphas), blobs.cb_point, blobs.cb_instance, None, _stream()), blobs)
            for b in (blobs.point, blobs.instance):
                if b is not None:
                    b.record_stream(torch.cuda.current_stream())
        return images, depths, alphas

    @torch.no_grad()
    def render_preextracted(self, view, mode: int, positions: torch.Tensor, features: torch.Tensor,
                            opacities: torch.Tensor, scales: torch.Tensor | None = None,
                            sigma_world_scale: float = 1.0, sigma_cutoff: float = 3.0):
        s = self.extract_settings(view, mode)
        positions = self._render_common(positions)
        features = _cuda_f16(features, "features")
        opacities = _cuda_f32(opacities, "opacities")
        n = positions.shape[0]
        if features.shape != (n, 36):
            raise ValueError(f"features must be (N,36), got {tuple(features.shape)}")
        if opacities.numel() != n:
            raise ValueError(f"opacities must hold N={n} values")
        if scales is not None and scales.numel() == 0:
            scales = None
        if scales is not None:
            scales = _cuda_f32(scales, "scales")
            if scales.numel() != n:
                raise ValueError(f"scales must hold N={n} values")
        dev = positions.device
        with torch.cuda.device(dev):
            varg = _ViewArg(s, dev)
            image = torch.empty((4, s.height, s.width), dtype=torch.float32, device=dev)
            depth = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            alpha = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            blobs = _Blobs(dev)
            _check(_cabi.lib().inpc_render_preextracted(
                s.mode.value, self.tile_size, C.byref(varg.c), n, _ptr(positions), _ptr(features), _ptr(opacities),
                _ptr(scales), float(sigma_world_scale * self.extract_base_sigma_world(view.camera)),
                float(sigma_cutoff), _ptr(image), _ptr(depth), _ptr(alpha), blobs.cb_point, blobs.cb_instance, None,
                _stream()), blobs)
            for b in (blobs.point, blobs.instance):
                if b is not None:
                    b.record_stream(torch.cuda.current_stream())
        return image, depth, alpha


    def forward_rows(self, view, positions: torch.Tensor, features: torch.Tensor, opacities: torch.Tensor):
        """Bilinear training forward over (N,C) fp32 feature rows, C in (4, 8, 16, 32): the features are
        blended as they are into a (C,H,W) image (differentiable w.r.t. features and opacities).  The
        reference has no such layout; its only one is 36 SH halves -> 4 channels (`forward`)."""
        return _RasterizeRows.apply(positions, features, opacities, self.extract_settings(view, 0), self.tile_size)

    @torch.no_grad()
    def render_rows(self, view, positions: torch.Tensor, features: torch.Tensor, opacities: torch.Tensor):
        """Bilinear inference over (N,C) fp32 feature rows: image (C,H,W), expected depth, alpha."""
        s = self.extract_settings(view, 0)
        positions, features, opacities = _check_rows(positions, features, opacities)
        n, channels = features.shape
        dev = positions.device
        with torch.cuda.device(dev):
            varg = _ViewArg(s, dev)
            image = torch.empty((channels, s.height, s.width), dtype=torch.float32, device=dev)
            depth = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            alpha = torch.empty((1, s.height, s.width), dtype=torch.float32, device=dev)
            blobs = _Blobs(dev)
            _check(_cabi.lib().inpc_render_rows(
                self.tile_size, C.byref(varg.c), n, _ptr(positions), _ptr(features), int(channels), _ptr(opacities),
                _ptr(image), _ptr(depth), _ptr(alpha), blobs.cb_point, blobs.cb_instance, None, _stream()), blobs)
            for b in (blobs.point, blobs.instance):
                if b is not None:
                    b.record_stream(torch.cuda.current_stream())
        return image, depth, alpha


def debug_arrays(ctx_or_state, view_settings: RasterizerSettings, point_blob: torch.Tensor,
                 instance_blob: torch.Tensor) -> dict:
    """Copies the intermediate arrays of a forward out of its blobs (parity tests)."""
    state = ctx_or_state
    dev = point_blob.device
    s = view_settings
    gw = -(-s.width // state.tile_size)
    gh = -(-s.height // state.tile_size)
    n, nv, ni = int(state.n_points), int(state.n_visible), int(state.n_instances)
    out = {
        "sorted_points": torch.empty(nv, dtype=torch.int32, device=dev),
        "sorted_depth_keys": torch.empty(nv, dtype=torch.int32, device=dev),
        "inst_point": torch.empty(ni, dtype=torch.int32, device=dev),
        "ranges": torch.empty((gw * gh, 2), dtype=torch.int32, device=dev),
        "n_touched": torch.empty(n, dtype=torch.int32, device=dev),
        "screen": torch.empty((n, 2), dtype=torch.float32, device=dev),
        "depth": torch.empty(n, dtype=torch.float32, device=dev),
        "feat_view": torch.empty((n, 4), dtype=torch.float32, device=dev),
        "bounds": torch.empty((n, 4), dtype=torch.int16, device=dev),
    }
    order = ["sorted_points", "sorted_depth_keys", "inst_point", "ranges", "n_touched", "screen", "depth",
             "feat_view", "bounds"]
    with torch.cuda.device(dev):
        varg = _ViewArg(s, dev)
        for which, name in enumerate(order):
            if out[name].numel() == 0:
                continue
            _check(_cabi.lib().inpc_raster_debug_copy(C.byref(state), C.byref(varg.c), which, _ptr(out[name]),
                                                      _stream()))
        torch.cuda.current_stream().synchronize()
    return out
