"""View-sharded batch step: the one place where the path spans several GPUs.

A batch of camera views is split across ranks (rank r takes views r, r+G, r+2G, ...); each view's
sample -> rasterize -> backward chain is independent and runs on the rank's own GPU.  Per batch the
ranks exchange two fp32 buffers with ONE NCCL all-reduce each (over NVLink / NVSwitch; in-switch
reduction when NCCL picks NVLS): a per-leaf statistic of the probability field and the gradient
buffer of the appearance field.  The reference has no multi-GPU code (one view per optimizer step
on one GPU); correctness here means: the reduced buffers equal what one GPU accumulates over the
same views.

The appearance network itself (tiny-cuda-nn in the reference) is outside this library, so its
gradient buffer is stood in for by a fixed scatter of the per-point gradients into `n_appearance`
slots; the per-leaf statistic is the sum of blending weights per leaf (the quantity the
reference's `ProbabilityField.update` reduces with max/min).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def partition_views(n_views: int, rank: int, world_size: int) -> list[int]:
    """Indices of the views rank `rank` renders: round-robin, so per-rank counts differ by at most one."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return list(range(rank, n_views, world_size))


@dataclass
class BatchBuffers:
    leaf: torch.Tensor         # (n_leaves,) fp32
    appearance: torch.Tensor   # (n_appearance,) fp32

    def zero_(self) -> None:
        self.leaf.zero_()
        self.appearance.zero_()


def accumulate_view(buffers: BatchBuffers, leaf_indices: torch.Tensor, blending_weights: torch.Tensor,
                    grad_features: torch.Tensor, grad_opacities: torch.Tensor) -> None:
    """Adds one view's contribution to the two buffers (device-side, no synchronisation).  The
    appearance stand-in folds the per-point opacity gradient and the DC feature gradient of the
    first channel into `n_appearance` slots."""
    valid = leaf_indices >= 0
    buffers.leaf.index_add_(0, leaf_indices.clamp_min(0), blending_weights * valid)
    n_app = buffers.appearance.numel()
    n = grad_opacities.numel()
    per_point = grad_opacities.reshape(-1) + grad_features[:, 0].float()
    if n % n_app == 0:
        buffers.appearance.add_(per_point.view(n // n_app, n_app).sum(dim=0))
    else:
        slot = torch.arange(n, device=per_point.device) % n_app
        buffers.appearance.index_add_(0, slot, per_point)


def allreduce_buffers(buffers: BatchBuffers, group=None) -> None:
    """SUM all-reduce of both buffers across the ranks of `group` (no-op without a process group)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    dist.all_reduce(buffers.leaf, op=dist.ReduceOp.SUM, group=group)
    dist.all_reduce(buffers.appearance, op=dist.ReduceOp.SUM, group=group)


class ViewShardedTrainer:
    """Runs sample -> rasterize -> backward for this rank's share of a batch of views."""

    def __init__(self, tree, features: torch.Tensor, opacities: torch.Tensor, n_samples: int, seed: int,
                 n_appearance: int = 1 << 22, tile_size: int = 8, mode: int = 0):
        from .rasterization import INPCRasterizer
        from .sampling import ProbabilityFieldSampler
        self.tree = tree
        self.features = features
        self.opacities = opacities
        self.n_samples = int(n_samples)
        self.mode = mode
        self.sampler = ProbabilityFieldSampler(seed)
        self.rasterizer = INPCRasterizer(tile_size=tile_size)
        dev = features.device
        self.buffers = BatchBuffers(torch.zeros(tree.centers.shape[0], dtype=torch.float32, device=dev),
                                    torch.zeros(n_appearance, dtype=torch.float32, device=dev))

    def run_view(self, view, grad_image: torch.Tensor, grad_alpha: torch.Tensor, view_index: int | None = None):
        """One view, forward and backward.  `view_index` pins the random stream to the view, so the
        result does not depend on which rank renders it."""
        t = self.tree
        if view_index is not None:
            self.sampler.set_rng_state(view_index)
        positions, indices = self.sampler.generate_training_samples(t.centers, t.levels, t.weights, view, self.n_samples,
                                                                    t.initial_size)
        feats = self.features.detach().requires_grad_(True)
        opac = self.opacities.detach().requires_grad_(True)
        image, alpha, blending_weights = self.rasterizer(view, self.mode, positions, feats, opac)
        torch.autograd.backward([image, alpha], [grad_image, grad_alpha])
        accumulate_view(self.buffers, indices, blending_weights, feats.grad, opac.grad)
        return image, alpha, blending_weights, feats.grad, opac.grad

    def run_batch(self, views, grads, rank: int = 0, world_size: int = 1, group=None):
        """All views of this rank's shard, then the one exchange step.  `grads` is one
        (grad_image, grad_alpha) pair used for every view, or a list with one pair per view."""
        self.buffers.zero_()
        out = None
        for vi in partition_views(len(views), rank, world_size):
            gi, ga = grads if isinstance(grads[0], torch.Tensor) else grads[vi]
            out = self.run_view(views[vi], gi, ga, view_index=vi)
        allreduce_buffers(self.buffers, group)
        return out
