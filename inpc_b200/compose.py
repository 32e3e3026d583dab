"""Image composition directly after the blend: background compose for training and multisample
accumulation for inference (reference: Renderer.py:80 and :105-125, chains of torch element-wise ops;
here one kernel of libinpc_b200 each, bit-identical results)."""
from __future__ import annotations

from typing import Any

import torch
from torch.autograd.function import once_differentiable

from . import _cabi
from .rasterization import _cuda_f32, _ptr, _stream


def _planes(image, alpha, name="image"):
    image = _cuda_f32(image, name)
    alpha = _cuda_f32(alpha, "alpha")
    if image.dim() != 3 or alpha.numel() != image.shape[1] * image.shape[2]:
        raise ValueError(f"{name} must be (C,H,W) and alpha (1,H,W) or (H,W); got {tuple(image.shape)} and {tuple(alpha.shape)}")
    return image, alpha


class _ComposeBackground(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, image: torch.Tensor, alpha: torch.Tensor, background: torch.Tensor):
        image, alpha = _planes(image, alpha)
        background = _cuda_f32(background, "background")
        if background.shape != image.shape:
            raise ValueError(f"background must have the image's shape {tuple(image.shape)}, got {tuple(background.shape)}")
        out = torch.empty_like(image)
        with torch.cuda.device(image.device):
            _cabi.check(_cabi.lib().inpc_compose_background(_ptr(image), _ptr(alpha), _ptr(background), image.shape[0],
                                                            image.shape[1] * image.shape[2], _ptr(out), _stream()))
        ctx.save_for_backward(alpha, background)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx: Any, grad_out: torch.Tensor):
        alpha, background = ctx.saved_tensors
        grad_out = _cuda_f32(grad_out, "grad_out")
        need_alpha, need_bg = ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        grad_alpha = torch.empty_like(alpha) if need_alpha else None
        grad_bg = torch.empty_like(background) if need_bg else None
        if need_alpha or need_bg:
            with torch.cuda.device(grad_out.device):
                _cabi.check(_cabi.lib().inpc_compose_background_backward(
                    _ptr(grad_out), _ptr(alpha), _ptr(background), grad_out.shape[0], grad_out.shape[1] * grad_out.shape[2],
                    _ptr(grad_alpha), _ptr(grad_bg), _stream()))
        return grad_out, grad_alpha, grad_bg


def compose_background(image: torch.Tensor, alpha: torch.Tensor, background: torch.Tensor) -> torch.Tensor:
    """`image + (1 - alpha) * background` (Renderer.py:80), differentiable in all three arguments."""
    return _ComposeBackground.apply(image, alpha, background)


class MultisampleAccumulator:
    """Running sums over the multisamples of one frame and their resolve (Renderer.py:105-125).

        acc = MultisampleAccumulator(n_multisamples, average_with_premultiplied_alpha=True)
        for ...: acc.add(*rasterizer.render(...))
        feature_image, depth, alpha, alpha_sum = acc.resolve(background)
    """

    def __init__(self, n_multisamples: int, average_with_premultiplied_alpha: bool = True) -> None:
        self.n = max(1, int(n_multisamples))
        self.unpremultiply = (not average_with_premultiplied_alpha) and self.n > 1
        self.count = 0
        self.image = self.depth = self.alpha = None

    @torch.no_grad()
    def add(self, image: torch.Tensor, depth: torch.Tensor, alpha: torch.Tensor) -> None:
        image, alpha = _planes(image, alpha)
        depth = _cuda_f32(depth, "depth")
        if depth.numel() != alpha.numel():
            raise ValueError("depth and alpha must have the same number of pixels")
        if self.count >= self.n:
            raise RuntimeError(f"already holds {self.n} multisamples")
        first = self.count == 0
        if first:
            self.image, self.depth, self.alpha = torch.empty_like(image), torch.empty_like(depth), torch.empty_like(alpha)
        elif image.shape != self.image.shape:
            raise ValueError("all multisamples must have the same shape")
        with torch.cuda.device(image.device):
            _cabi.check(_cabi.lib().inpc_multisample_accumulate(
                _ptr(self.image), _ptr(self.depth), _ptr(self.alpha), _ptr(image), _ptr(depth), _ptr(alpha), image.shape[0],
                alpha.numel(), int(first), int(self.unpremultiply), _stream()))
        self.count += 1

    @torch.no_grad()
    def resolve(self, background: torch.Tensor | None = None):
        """Returns (feature_image, depth, alpha, alpha_sum); the accumulator is empty afterwards."""
        if self.count != self.n:
            raise RuntimeError(f"{self.count} of {self.n} multisamples were added")
        if background is not None:
            background = _cuda_f32(background, "background")
            if background.shape != self.image.shape:
                raise ValueError("background must have the image's shape")
        alpha_sum = torch.empty_like(self.alpha)
        with torch.cuda.device(self.image.device):
            _cabi.check(_cabi.lib().inpc_multisample_resolve(
                _ptr(self.image), _ptr(self.depth), _ptr(self.alpha), _ptr(alpha_sum), _ptr(background), self.image.shape[0],
                self.alpha.numel(), self.n, int(self.unpremultiply), _stream()))
        out = (self.image, self.depth, self.alpha, alpha_sum)
        self.image = self.depth = self.alpha = None
        self.count = 0
        return out


class MultisamplingRingBuffer:
    """Sample sets of the last `size` frames (utils.py:145-174): every frame appends one new set and
    re-rasterises all cached ones, so a frame costs one sampling / shading pass instead of `size`.
    Same behaviour as the reference class, including its start-up rule (a slot that has not been
    filled yet yields the first set)."""

    def __init__(self) -> None:
        self.size = 0
        self.positions: list | None = None
        self.features: list | None = None
        self.current_idx = 0
        self.read_idx = 0

    def append(self, positions: torch.Tensor, features: torch.Tensor, new_size: int) -> None:
        if self.size != new_size:
            self.current_idx = 0
            self.size = new_size
            self.positions = [None] * new_size
            self.features = [None] * new_size
        self.positions[self.current_idx] = positions
        self.features[self.current_idx] = features
        self.current_idx = (self.current_idx + 1) % self.size
        self.read_idx = 0

    def get_next(self):
        if self.positions[self.read_idx] is None:
            return self.positions[0], self.features[0]
        positions, features = self.positions[self.read_idx], self.features[self.read_idx]
        self.read_idx += 1
        return positions, features


_SIDE_STREAMS: dict = {}


def _side_streams(device: torch.device, n: int) -> list:
    """`n` persistent side streams of `device`.  They are created once: torch's caching allocator keeps a
    pool of blocks per stream, so fresh streams on every call would allocate from the driver every time."""
    pool = _SIDE_STREAMS.setdefault((device.type, device.index), [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device=device))
    return pool[:n]


@torch.no_grad()
def render_multisampled(rasterizer, view, mode: int, sample_sets, background: torch.Tensor | None = None,
                        sigma_world_scale: float = 1.0, sigma_cutoff: float = 3.0,
                        average_with_premultiplied_alpha: bool = True, n_streams: int = 1, batched: bool = False):
    """Inference over several sample sets of one view (Renderer.py:99-125 and :139-166): every set
    `(positions, features_raw)` is rasterised with `rasterizer.render`, the results are averaged and
    composed over `background`.  `sample_sets` is a list of pairs or a filled `MultisamplingRingBuffer`.
    With `n_streams > 1` the sets are rasterised concurrently on that many CUDA streams (they are
    independent; the accumulation order, and hence the result, stays that of the list).  `batched` (bilinear splats,
    8x8 tiles, at most 8 sets) renders all sets with one `render_multi` call instead: same bits, one launch sequence;
    with `n_streams > 1` as well, the sets are split into that many groups (of two sets at least), one batched call each.
    Returns (feature_image, depth, alpha, alpha_sum)."""
    if isinstance(sample_sets, MultisamplingRingBuffer):
        ring = sample_sets
        sets = [ring.get_next() for _ in range(ring.size)]
    else:
        sets = list(sample_sets)
    acc = MultisampleAccumulator(len(sets), average_with_premultiplied_alpha)
    if batched and mode == 0 and 2 <= len(sets) <= 8 and getattr(rasterizer, "tile_size", 0) == 8:
        # one launch sequence per group of sets (culled, sorted and blended together), then the same accumulation, set by set
        n_groups = max(1, min(n_streams, len(sets) // 2))
        if n_groups == 1:
            images, depths, alphas = rasterizer.render_multi(view, sets)
            for j in range(len(sets)):
                acc.add(images[j], depths[j], alphas[j])
            return acc.resolve(background)
        main = torch.cuda.current_stream()
        streams = _side_streams(sets[0][0].device, n_groups)
        bounds = [len(sets) * g // n_groups for g in range(n_groups + 1)]
        rendered = []
        for g, s in enumerate(streams):
            s.wait_stream(main)
            with torch.cuda.stream(s):
                rendered.append(rasterizer.render_multi(view, sets[bounds[g]:bounds[g + 1]]))
        for s in streams:
            main.wait_stream(s)
        for images, depths, alphas in rendered:
            for t in (images, depths, alphas):
                t.record_stream(main)
            for j in range(images.shape[0]):
                acc.add(images[j], depths[j], alphas[j])
        return acc.resolve(background)
    if n_streams <= 1 or len(sets) < 2:
        for positions, features_raw in sets:
            acc.add(*rasterizer.render(view, mode, positions, features_raw, sigma_world_scale, sigma_cutoff))
        return acc.resolve(background)
    main = torch.cuda.current_stream()
    streams = _side_streams(sets[0][0].device, min(n_streams, len(sets)))
    for s in streams:
        s.wait_stream(main)
    rendered = []
    for k, (positions, features_raw) in enumerate(sets):
        with torch.cuda.stream(streams[k % len(streams)]):
            rendered.append(rasterizer.render(view, mode, positions, features_raw, sigma_world_scale, sigma_cutoff))
    for s in streams:
        main.wait_stream(s)
    for images in rendered:
        for t in images:
            t.record_stream(main)
        acc.add(*images)
    return acc.resolve(background)
