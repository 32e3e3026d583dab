"""Fused update of the octree probability field from one step's samples: the consumer of the
rasterizer's `blending_weights` (reference: Modules/ProbabilityField.py:146-157, called from
Trainer.py:167-168).  The reference does it with two `scatter_reduce_` calls and four element-wise
ops; here it is two kernels of libinpc_b200, and the per-leaf statistics can be accumulated over
several views and reduced across ranks before they are applied."""
from __future__ import annotations

import ctypes as C

import torch

from . import _cabi
from .rasterization import _cuda_f32, _ptr, _stream

DECAY = 0.9968


MIN_FLIP = 0x7FFFFFFF


def decode_statistics(stats: torch.Tensor):
    """(max_sampled, min_sampled) as float tensors from a packed (L,2) int32 statistics buffer; leaves
    without a sample read 0 / 0, as the update treats them."""
    mx = stats[:, 0].contiguous().view(torch.float32)
    flipped = stats[:, 1]
    mn = (MIN_FLIP - flipped).to(torch.int32).contiguous().view(torch.float32)
    return mx, torch.where(flipped == 0, torch.zeros_like(mn), mn)


class LeafStatistics:
    """Running per-leaf max / min of blending weights.  One (L,2) int32 buffer: {bit pattern of the
    maximum, 0x7FFFFFFF - bit pattern of the minimum}.  Weights are non-negative, so both columns only
    grow and a single `MAX` all-reduce reduces the buffer across ranks exactly; zero = no sample."""

    def __init__(self, n_leaves: int, device) -> None:
        self.stats = torch.empty((n_leaves, 2), dtype=torch.int32, device=device)
        self.reset()

    @property
    def max_sampled(self) -> torch.Tensor:
        return decode_statistics(self.stats)[0]

    @property
    def min_sampled(self) -> torch.Tensor:
        return decode_statistics(self.stats)[1]

    def reset(self) -> None:
        with torch.cuda.device(self.stats.device):
            _cabi.check(_cabi.lib().inpc_leaf_stats_reset(_ptr(self.stats), self.stats.shape[0], _stream()))

    def accumulate(self, indices: torch.Tensor, weights: torch.Tensor) -> None:
        if not indices.is_cuda or indices.dtype != torch.int64:
            raise TypeError("indices must be a CUDA int64 tensor")
        weights = _cuda_f32(weights.reshape(-1), "weights")
        indices = indices.contiguous()
        if indices.numel() != weights.numel():
            raise ValueError("indices and weights must have the same number of elements")
        with torch.cuda.device(self.stats.device):
            _cabi.check(_cabi.lib().inpc_leaf_stats_accumulate(_ptr(indices), _ptr(weights), indices.numel(), _ptr(self.stats),
                                                               self.stats.shape[0], _stream()))

    def all_reduce(self, group=None) -> None:
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return
        dist.all_reduce(self.stats, op=dist.ReduceOp.MAX, group=group)


def update(leaf_weights: torch.Tensor, leaf_subdivision_scores: torch.Tensor, stats: LeafStatistics,
           decay: float = DECAY) -> None:
    """In-place `ProbabilityField.update` from accumulated statistics."""
    for t, name in ((leaf_weights, "leaf_weights"), (leaf_subdivision_scores, "leaf_subdivision_scores")):
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous CUDA float32 tensor")
    with torch.cuda.device(leaf_weights.device):
        _cabi.check(_cabi.lib().inpc_leaf_update(_ptr(leaf_weights), _ptr(leaf_subdivision_scores), _ptr(stats.stats),
                                                 leaf_weights.numel(), float(decay), _stream()))


def update_from_samples(leaf_weights: torch.Tensor, leaf_subdivision_scores: torch.Tensor, indices: torch.Tensor,
                        weights: torch.Tensor, decay: float = DECAY) -> None:
    """Drop-in for `ProbabilityField.update(indices, weights)` on the module's two leaf buffers."""
    stats = LeafStatistics(leaf_weights.numel(), leaf_weights.device)
    stats.accumulate(indices, weights)
    update(leaf_weights, leaf_subdivision_scores, stats, decay)


MAX_LEVEL = 6                 # ProbabilityField.py:220
MAX_LEAVES = 16_777_216       # 256^3, ProbabilityField.py:222-224


def _leaf_arrays(centers, levels, weights, scores):
    n = weights.numel()
    for t, name, dt in ((centers, "leaf_centers", torch.float32), (levels, "leaf_levels", torch.int32),
                        (weights, "leaf_weights", torch.float32), (scores, "leaf_subdivision_scores", torch.float32)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor")
        if t.dtype != dt:
            raise TypeError(f"{name} must be {dt}, got {t.dtype}")
    if centers.shape != (n, 3) or levels.numel() != n or scores.numel() != n:
        raise ValueError("leaf arrays must describe the same number of leaves: centers (L,3), levels / weights / scores (L)")
    return centers.contiguous(), levels.contiguous(), weights.contiguous(), scores.contiguous(), n


def _select(kind, values, levels, n, threshold, max_level, device):
    lib = _cabi.lib()
    ws = torch.empty(int(lib.inpc_leaf_select_workspace_bytes(n)), dtype=torch.uint8, device=device)
    count = C.c_int64(0)
    _cabi.check(lib.inpc_leaf_select_count(kind, _ptr(values), _ptr(levels), n, float(threshold), int(max_level), _ptr(ws),
                                           C.byref(count), _stream()))
    return ws, int(count.value)


def prune(leaf_centers, leaf_levels, leaf_weights, leaf_subdivision_scores, threshold: float):
    """`ProbabilityField.prune` (Modules/ProbabilityField.py:159-165): the leaves with weight > threshold,
    in their old order, as four new tensors (centers, levels, weights, scores)."""
    centers, levels, weights, scores, n = _leaf_arrays(leaf_centers, leaf_levels, leaf_weights, leaf_subdivision_scores)
    dev = weights.device
    with torch.cuda.device(dev):
        ws, kept = _select(0, weights, levels, n, threshold, 0, dev)
        out = (torch.empty((kept, 3), dtype=torch.float32, device=dev), torch.empty(kept, dtype=torch.int32, device=dev),
               torch.empty(kept, dtype=torch.float32, device=dev), torch.empty(kept, dtype=torch.float32, device=dev))
        if kept:
            _cabi.check(_cabi.lib().inpc_leaf_prune_fill(_ptr(centers), _ptr(levels), _ptr(weights), _ptr(scores), n,
                                                         float(threshold), _ptr(ws), *[_ptr(o) for o in out], _stream()))
            ws.record_stream(torch.cuda.current_stream())
    return out


def subdivide(leaf_centers, leaf_levels, leaf_weights, leaf_subdivision_scores, threshold: float, initial_size: float,
              max_level: int = MAX_LEVEL, max_leaves: int = MAX_LEAVES):
    """`ProbabilityField.subdivide` (Modules/ProbabilityField.py:217-257): leaves with score > threshold
    and level < max_level are replaced by their eight children, appended after the unsplit leaves.
    Returns the four new tensors, or None when the octree would exceed `max_leaves` (the reference
    then leaves the octree as it is)."""
    centers, levels, weights, scores, n = _leaf_arrays(leaf_centers, leaf_levels, leaf_weights, leaf_subdivision_scores)
    dev = weights.device
    with torch.cuda.device(dev):
        ws, split = _select(1, scores, levels, n, threshold, max_level, dev)
        total = n + 7 * split
        if total > max_leaves:
            return None
        out = (torch.empty((total, 3), dtype=torch.float32, device=dev), torch.empty(total, dtype=torch.int32, device=dev),
               torch.empty(total, dtype=torch.float32, device=dev), torch.empty(total, dtype=torch.float32, device=dev))
        if n:
            _cabi.check(_cabi.lib().inpc_leaf_subdivide_fill(_ptr(centers), _ptr(levels), _ptr(weights), _ptr(scores), n,
                                                             float(threshold), int(max_level), float(initial_size), split,
                                                             _ptr(ws), *[_ptr(o) for o in out], _stream()))
            ws.record_stream(torch.cuda.current_stream())
    return out
