"""Host-side mirror of the reference sampler bindings
(INPCCudaBackend/INPCCudaBackend/torch_bindings/sampling.py): `compute_viewpoint_weights` and the
`ProbabilityFieldSampler` module with its three generate_* methods, on top of libinpc_b200.

The random stream is a counter-based Philox4x32-10 keyed by the seed; its whole state is one 64-bit
call counter, exposed through `get_rng_state` / `set_rng_state` and the module's state dict so that
a resumed run continues the stream (the reference's pcg32 state cannot be checkpointed).
"""
from __future__ import annotations

import ctypes as C
import warnings

import torch

from . import _cabi
from .rasterization import _cuda_f32, _ptr, _stream


def _check_view(view) -> None:
    cam = view.camera
    for attr in ("width", "height", "focal_x", "focal_y", "center_x", "center_y", "near_plane", "far_plane"):
        if not hasattr(cam, attr):
            raise NotImplementedError(f"camera without `{attr}`: only perspective cameras are supported")
    if getattr(cam, "distortion", None) is not None:
        raise NotImplementedError("camera distortion is not supported by the sampler")


class _ViewArg:
    def __init__(self, view, device: torch.device):
        cam = view.camera
        self.w2c = _cuda_f32(view.w2c.to(device), "w2c")
        if self.w2c.numel() != 16:
            raise ValueError("w2c must have 16 elements")
        pos = getattr(view, "position", None)
        self.pos = None if pos is None else _cuda_f32(pos.to(device), "position")
        self.c = _cabi.View(self.w2c.data_ptr(), 0 if self.pos is None else self.pos.data_ptr(), int(cam.width),
                            int(cam.height), float(cam.focal_x), float(cam.focal_y), float(cam.center_x),
                            float(cam.center_y), float(cam.near_plane), float(cam.far_plane))


def _leaf_args(centers: torch.Tensor, levels: torch.Tensor, weights: torch.Tensor):
    centers = _cuda_f32(centers, "centers")
    weights = _cuda_f32(weights, "weights")
    if not levels.is_cuda or levels.dtype != torch.int32:
        raise TypeError(f"levels must be a CUDA int32 tensor, got {levels.dtype} on {levels.device}")
    levels = levels.contiguous()
    n = centers.shape[0]
    if centers.dim() != 2 or centers.shape[1] != 3 or levels.numel() != n or weights.numel() != n:
        raise ValueError("centers must be (L,3) with L levels and L weights")
    return centers, levels, weights, n


def compute_viewpoint_weights(centers: torch.Tensor, levels: torch.Tensor, weights: torch.Tensor, view,
                              initial_size: float) -> torch.Tensor:
    _check_view(view)
    centers, levels, weights, n = _leaf_args(centers, levels, weights)
    dev = centers.device
    with torch.cuda.device(dev):
        varg = _ViewArg(view, dev)
        out = torch.empty((n,), dtype=torch.float32, device=dev)
        _cabi.check(_cabi.lib().inpc_compute_viewpoint_weights(C.byref(varg.c), n, _ptr(centers), _ptr(levels),
                                                               _ptr(weights), float(initial_size), _ptr(out),
                                                               _stream()))
    return out


class ProbabilityFieldSampler(torch.nn.Module):
    def __init__(self, seed: int) -> None:
        super().__init__()
        self.seed = int(seed)
        self._handle = C.c_void_p(_cabi.lib().inpc_sampler_create(self.seed))
        if not self._handle:
            raise _cabi.InpcError("inpc_sampler_create failed")

    def __del__(self):
        try:
            h = self.__dict__.get("_handle")
            if h:
                self.__dict__["_handle"] = None
                _cabi.lib().inpc_sampler_destroy(h)
        except Exception:
            pass

    # ---- checkpoint / resume of the stream position
    def get_rng_state(self) -> int:
        return int(_cabi.lib().inpc_sampler_get_counter(self._handle))

    def set_rng_state(self, counter: int) -> None:
        _cabi.lib().inpc_sampler_set_counter(self._handle, int(counter))

    def get_extra_state(self):
        return {"seed": self.seed, "counter": self.get_rng_state()}

    def set_extra_state(self, state) -> None:
        if state and int(state.get("seed", self.seed)) == self.seed:
            self.set_rng_state(int(state["counter"]))

    def last_call_exhausted(self) -> bool | None:
        """True if some slots of the last `generate_training_samples` call ran out of rejection attempts (they
        hold their last candidate, a position outside the view frustum), False if none did, None if no longer known.
        Final once the stream of that call has been synchronised; reading it does not synchronise."""
        r = int(_cabi.lib().inpc_sampler_exhausted(self._handle))
        return None if r < 0 else bool(r)

    def _workspace(self, n_cells: int, dev: torch.device) -> torch.Tensor:
        nbytes = int(_cabi.lib().inpc_sampler_workspace_bytes(n_cells))
        return torch.empty(nbytes, dtype=torch.uint8, device=dev)

    def draw_leaf_counts(self, weights: torch.Tensor, n_samples: int) -> torch.Tensor:
        """Number of draws per leaf of `n_samples` multinomial draws with probabilities proportional to
        `weights` (torch.multinomial + bincount of Modules/ProbabilityField.py:129-130), int32 (L)."""
        if not weights.is_cuda or weights.dtype != torch.float32:
            raise TypeError("weights must be a CUDA float32 tensor")
        weights = weights.contiguous()
        n, dev = weights.numel(), weights.device
        with torch.cuda.device(dev):
            counts = torch.empty(n, dtype=torch.int32, device=dev)
            ws = self._workspace(n, dev)
            _cabi.check(_cabi.lib().inpc_draw_leaf_counts(self._handle, n, _ptr(weights), int(n_samples), _ptr(counts), _ptr(ws),
                                                          _stream()))
            ws.record_stream(torch.cuda.current_stream())
        return counts

    def generate_training_samples(self, centers: torch.Tensor, levels: torch.Tensor, weights: torch.Tensor, view,
                                  n_samples: int, initial_size: float) -> tuple[torch.Tensor, torch.Tensor]:
        _check_view(view)
        centers, levels, weights, n = _leaf_args(centers, levels, weights)
        dev = centers.device
        if self.last_call_exhausted():
            # the previous call's flag, read without waiting for anything: by now it is normally final
            warnings.warn("the previous generate_training_samples call left sample slots unfilled (rejection attempts "
                          "exhausted): they hold positions outside the view frustum")
        with torch.cuda.device(dev):
            varg = _ViewArg(view, dev)
            positions = torch.empty((n_samples, 3), dtype=torch.float32, device=dev)
            indices = torch.empty((n_samples,), dtype=torch.int64, device=dev)
            ws = self._workspace(n, dev)
            _cabi.check(_cabi.lib().inpc_generate_training_samples(
                self._handle, C.byref(varg.c), n, _ptr(centers), _ptr(levels), _ptr(weights), float(initial_size),
                int(n_samples), _ptr(positions), _ptr(indices), _ptr(ws), _stream()))
            ws.record_stream(torch.cuda.current_stream())
        return positions, indices

    def generate_samples(self, centers: torch.Tensor, levels: torch.Tensor, weights: torch.Tensor, view,
                         n_samples: int, initial_size: float) -> torch.Tensor:
        _check_view(view)
        centers, levels, weights, n = _leaf_args(centers, levels, weights)
        dev = centers.device
        with torch.cuda.device(dev):
            varg = _ViewArg(view, dev)
            positions = torch.empty((n_samples, 3), dtype=torch.float32, device=dev)
            ws = self._workspace(n, dev)
            written = C.c_int64(0)
            _cabi.check(_cabi.lib().inpc_generate_samples(
                self._handle, C.byref(varg.c), n, _ptr(centers), _ptr(levels), _ptr(weights), float(initial_size),
                int(n_samples), _ptr(positions), C.byref(written), _ptr(ws), _stream()))
            ws.record_stream(torch.cuda.current_stream())
        if written.value == 0 and n_samples > 0:
            return torch.empty((0, 3), dtype=torch.float32, device=dev)
        return positions

    def generate_expected_samples(self, centers: torch.Tensor, levels: torch.Tensor, weights: torch.Tensor, view,
                                  n_samples: int, n_multi: int, initial_size: float) -> torch.Tensor:
        _check_view(view)
        centers, levels, weights, n = _leaf_args(centers, levels, weights)
        dev = centers.device
        with torch.cuda.device(dev):
            varg = _ViewArg(view, dev)
            ws = self._workspace(n, dev)
            created = C.c_int64(0)
            _cabi.check(_cabi.lib().inpc_generate_expected_samples_count(
                self._handle, C.byref(varg.c), n, _ptr(centers), _ptr(levels), _ptr(weights), float(initial_size),
                int(n_samples), C.byref(created), _ptr(ws), _stream()))
            if created.value == 0 or n_multi <= 0:
                return torch.empty((0, 3), dtype=torch.float32, device=dev)
            positions = torch.empty((created.value * int(n_multi), 3), dtype=torch.float32, device=dev)
            _cabi.check(_cabi.lib().inpc_generate_expected_samples_fill(
                self._handle, n, _ptr(centers), _ptr(levels), float(initial_size), created.value, int(n_multi),
                _ptr(positions), _ptr(ws), _stream()))
            ws.record_stream(torch.cuda.current_stream())
        return positions


def halton_samples(counts: torch.Tensor, centers: torch.Tensor, levels: torch.Tensor, initial_size: float) -> torch.Tensor:
    """Quasi-random positions, `counts[l]` per leaf, leaf by leaf: the Halton placement of
    `ProbabilityField.extract_global` (Modules/ProbabilityField.py:131-140 with utils.py:36-64)."""
    if not counts.is_cuda or counts.dtype != torch.int32:
        raise TypeError("counts must be a CUDA int32 tensor")
    centers, levels, _, n = _leaf_args(centers, levels, torch.empty(centers.shape[0], dtype=torch.float32, device=centers.device))
    if counts.numel() != n:
        raise ValueError(f"counts must hold one entry per leaf ({n}), got {counts.numel()}")
    counts = counts.contiguous()
    total = int(counts.sum().item())
    dev = centers.device
    with torch.cuda.device(dev):
        positions = torch.empty((total, 3), dtype=torch.float32, device=dev)
        ws = torch.empty(int(_cabi.lib().inpc_sampler_workspace_bytes(n)), dtype=torch.uint8, device=dev)
        _cabi.check(_cabi.lib().inpc_halton_samples(_ptr(counts), n, _ptr(centers), _ptr(levels), float(initial_size), total,
                                                    _ptr(positions), _ptr(ws), _stream()))
        ws.record_stream(torch.cuda.current_stream())
    return positions


def morton_order(positions: torch.Tensor) -> torch.Tensor:
    """`positions` (N,3) reordered along a 30-bit Morton curve through their bounding cube (the role of
    morton_encode + argsort in Modules/ProbabilityField.py:141-143)."""
    positions = positions.contiguous()
    if not positions.is_cuda or positions.dtype != torch.float32 or positions.dim() != 2 or positions.shape[1] != 3:
        raise TypeError("positions must be a CUDA float32 (N,3) tensor")
    n = positions.shape[0]
    if n == 0:
        return positions.clone()
    lo = positions.amin(dim=0)
    extent = float((positions.amax(dim=0) - lo).max().item())
    extent = extent * (1.0 + 1e-6) if extent > 0 else 1.0
    box_lo = (C.c_float * 3)(*[float(v) for v in lo.tolist()])
    dev = positions.device
    with torch.cuda.device(dev):
        out = torch.empty_like(positions)
        ws = torch.empty(int(_cabi.lib().inpc_morton_workspace_bytes(n)), dtype=torch.uint8, device=dev)
        _cabi.check(_cabi.lib().inpc_morton_order(_ptr(positions), n, box_lo, extent, _ptr(out), _ptr(ws), _stream()))
        ws.record_stream(torch.cuda.current_stream())
    return out


def extract_global(sampler: "ProbabilityFieldSampler", centers: torch.Tensor, levels: torch.Tensor, weights: torch.Tensor, views,
                   n_samples: int, initial_size: float, use_morton_order: bool = True) -> torch.Tensor:
    """`ProbabilityField.extract_global` (Modules/ProbabilityField.py:121-144): leaf weights = maximum of
    the viewpoint weights over `views` (the level-weighted occupancy when `views` is empty), multinomial
    sample counts per leaf, Halton placement inside every leaf, optional Morton order."""
    centers, levels, weights, n = _leaf_args(centers, levels, weights)
    if views:
        global_weights = torch.zeros_like(weights)
        for view in views:
            torch.maximum(compute_viewpoint_weights(centers, levels, weights, view, initial_size), global_weights, out=global_weights)
    else:
        global_weights = weights * torch.exp2(-levels * 0.5)             # ProbabilityField.get_current_weights(None)
    counts = sampler.draw_leaf_counts(global_weights, n_samples)
    positions = halton_samples(counts, centers, levels, initial_size)
    return morton_order(positions) if use_morton_order else positions


def build_cdf(weights: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Normalised inclusive CDF and plain sum of `weights` (both on the device)."""
    weights = _cuda_f32(weights, "weights")
    n = weights.numel()
    dev = weights.device
    with torch.cuda.device(dev):
        cdf = torch.empty_like(weights)
        total = torch.empty((1,), dtype=torch.float32, device=dev)
        ws = torch.empty(int(_cabi.lib().inpc_sampler_workspace_bytes(n)), dtype=torch.uint8, device=dev)
        _cabi.check(_cabi.lib().inpc_build_cdf(_ptr(weights), n, _ptr(cdf), _ptr(total), _ptr(ws), _stream()))
        ws.record_stream(torch.cuda.current_stream())
    return cdf, total


def draw_leaves(cdf: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """out[i] = min(lower_bound(cdf, u[i]), L-1) as int64."""
    cdf, u = _cuda_f32(cdf, "cdf"), _cuda_f32(u, "u")
    dev = cdf.device
    with torch.cuda.device(dev):
        out = torch.empty((u.numel(),), dtype=torch.int64, device=dev)
        _cabi.check(_cabi.lib().inpc_draw_leaves(_ptr(cdf), cdf.numel(), _ptr(u), u.numel(), _ptr(out), _stream()))
    return out
