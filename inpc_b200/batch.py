"""View-sharded batch step: the one place where the path spans several GPUs.

A batch of camera views is split across ranks (rank r takes views r, r+G, r+2G, ...); each view's
sample -> rasterize -> backward chain is independent and runs on the rank's own GPU.  Per batch the
ranks exchange two buffers with one NCCL all-reduce each (over NVLink / NVSwitch; in-switch
reduction when NCCL picks NVLS): the packed per-leaf max / min of the blending weights (MAX) that the
probability-field update consumes, and the gradient buffer of the appearance field (SUM).  The reference has no multi-GPU code (one view per optimizer step
on one GPU); correctness here means: the reduced buffers equal what one GPU accumulates over the
same views.

The appearance network itself (tiny-cuda-nn in the reference) is outside this library, so its
gradient buffer is stood in for by a fixed fold of the per-point opacity gradients into
`n_appearance` slots.
"""
from __future__ import annotations

import torch


def partition_views(n_views: int, rank: int, world_size: int) -> list[int]:
    """Indices of the views rank `rank` renders: round-robin, so per-rank counts differ by at most one."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return list(range(rank, n_views, world_size))


class BatchBuffers:
    """What a batch exchanges: packed per-leaf max / min of the blending weights (reduced with MAX,
    exactly what the reference's `ProbabilityField.update` needs) and the appearance gradient buffer
    (reduced with SUM)."""

    def __init__(self, n_leaves: int, n_appearance: int, device) -> None:
        self.appearance = torch.zeros(n_appearance, dtype=torch.float32, device=device)
        self.device = torch.device(device)
        if self.device.type == "cuda":
            from .probability_field import LeafStatistics
            self.leaf = LeafStatistics(n_leaves, device)
        else:   # host-side tests of the exchange logic: same buffers, filled by the caller
            self.leaf = _HostLeafStatistics(n_leaves)

    def zero_(self) -> None:
        self.leaf.reset()
        self.appearance.zero_()


class _HostLeafStatistics:
    """CPU mirror of `probability_field.LeafStatistics` (same packed buffer) for the host-side tests of
    the exchange logic."""
    MIN_FLIP = 0x7FFFFFFF

    def __init__(self, n_leaves: int) -> None:
        self.stats = torch.zeros((n_leaves, 2), dtype=torch.int32)

    @property
    def max_sampled(self) -> torch.Tensor:
        from .probability_field import decode_statistics
        return decode_statistics(self.stats)[0]

    @property
    def min_sampled(self) -> torch.Tensor:
        from .probability_field import decode_statistics
        return decode_statistics(self.stats)[1]

    def reset(self) -> None:
        self.stats.zero_()

    def accumulate(self, indices: torch.Tensor, weights: torch.Tensor) -> None:
        valid = indices >= 0
        idx = indices[valid]
        bits = weights.reshape(-1)[valid].clamp_min(0).contiguous().view(torch.int32)
        mx, flipped = self.stats[:, 0].clone(), self.stats[:, 1].clone()
        mx.scatter_reduce_(0, idx, bits, reduce="amax", include_self=True)
        flipped.scatter_reduce_(0, idx, self.MIN_FLIP - bits, reduce="amax", include_self=True)
        self.stats[:, 0], self.stats[:, 1] = mx, flipped

    def all_reduce(self, group=None) -> None:
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return
        dist.all_reduce(self.stats, op=dist.ReduceOp.MAX, group=group)


def accumulate_view(buffers: BatchBuffers, leaf_indices: torch.Tensor, blending_weights: torch.Tensor,
                    grad_features: torch.Tensor, grad_opacities: torch.Tensor, appearance: torch.Tensor | None = None,
                    overwrite: bool = False) -> None:
    """Adds one view's contribution to the buffers (device-side, no synchronisation).  The appearance
    stand-in folds the per-point opacity gradient into `n_appearance` slots.  `appearance` redirects
    that sum to a private partial buffer (views running concurrently on several streams must not
    read-modify-write one buffer; the leaf statistics are updated with atomics and need no such care);
    `overwrite` stores the view's sum instead of adding it (the first view of a partial buffer: no zero-fill)."""
    buffers.leaf.accumulate(leaf_indices, blending_weights)
    target = buffers.appearance if appearance is None else appearance
    n_app = target.numel()
    per_point = grad_opacities.reshape(-1)
    n = per_point.numel()
    if n % n_app == 0:
        if overwrite:
            torch.sum(per_point.view(n // n_app, n_app), dim=0, out=target)
        else:
            target.add_(per_point.view(n // n_app, n_app).sum(dim=0))
    else:
        if overwrite:
            target.zero_()
        slot = torch.arange(n, device=per_point.device) % n_app
        target.index_add_(0, slot, per_point)


def allreduce_buffers(buffers: BatchBuffers, group=None) -> None:
    """The one exchange step of a batch: MAX of the packed leaf statistics, SUM of the appearance buffer."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    buffers.leaf.all_reduce(group)
    dist.all_reduce(buffers.appearance, op=dist.ReduceOp.SUM, group=group)


class ViewShardedTrainer:
    """Runs sample -> rasterize -> backward for this rank's share of a batch of views.

    The views of a shard are independent, and most kernels of the chain are bound by latency rather than
    by bandwidth, so the shard is software-pipelined over `n_streams` CUDA streams: view k runs on stream
    k mod n_streams and overlaps with its neighbours (measured on B200, 2^23 samples per view: 2.24 ms
    per view on one stream, 1.95 on two, 1.89 on three, 1.88 on four; four also divides the 8 or 16
    views a rank gets from a 64-view batch on 8 or 4 GPUs evenly)."""

    def __init__(self, tree, features: torch.Tensor, opacities: torch.Tensor, n_samples: int, seed: int,
                 n_appearance: int = 1 << 22, tile_size: int = 8, mode: int = 0, n_streams: int = 4):
        from .rasterization import INPCRasterizer
        from .sampling import ProbabilityFieldSampler
        self.tree = tree
        self.features = features
        self.opacities = opacities
        self.n_samples = int(n_samples)
        self.mode = mode
        self.sampler = ProbabilityFieldSampler(seed)
        self.rasterizer = INPCRasterizer(tile_size=tile_size)
        self.buffers = BatchBuffers(tree.centers.shape[0], n_appearance, features.device)
        self.n_streams = max(1, int(n_streams))
        self._streams: list | None = None
        self._appearance_parts: list | None = None

    def _pipeline(self):
        if self._streams is None:
            dev = self.features.device
            self._streams = [torch.cuda.Stream(device=dev) for _ in range(self.n_streams)]
            # one row per stream: the views of a stream add into their own row
            self._appearance_parts = torch.zeros((self.n_streams, self.buffers.appearance.numel()), dtype=torch.float32, device=dev)
        return self._streams, self._appearance_parts

    def run_view(self, view, grad_image: torch.Tensor, grad_alpha: torch.Tensor, view_index: int | None = None,
                 appearance: torch.Tensor | None = None, overwrite: bool = False, grads_ready=None):
        """One view, forward and backward.  `view_index` pins the random stream to the view, so the
        result does not depend on which rank renders it.  `grads_ready` (a CUDA event) is waited for between the
        forward and the backward pass: upstream gradients that are still being copied do not hold up the forward."""
        t = self.tree
        if view_index is not None:
            self.sampler.set_rng_state(view_index)
        positions, indices = self.sampler.generate_training_samples(t.centers, t.levels, t.weights, view, self.n_samples,
                                                                    t.initial_size)
        feats = self.features.detach().requires_grad_(True)
        opac = self.opacities.detach().requires_grad_(True)
        image, alpha, blending_weights = self.rasterizer(view, self.mode, positions, feats, opac)
        if grads_ready is not None:
            torch.cuda.current_stream().wait_event(grads_ready)
        torch.autograd.backward([image, alpha], [grad_image, grad_alpha])
        accumulate_view(self.buffers, indices, blending_weights, feats.grad, opac.grad, appearance, overwrite)
        return image, alpha, blending_weights, feats.grad, opac.grad

    def run_batch(self, views, grads, rank: int = 0, world_size: int = 1, group=None, inputs=None):
        """All views of this rank's shard and the exchange step.  `grads` is one (grad_image, grad_alpha) pair
        used for every view, or a list with one pair per view.  `inputs(view_index, stream)`, if given, supplies
        (view, grad_image, grad_alpha) of a view instead -- e.g. copied from host memory on a stream of the
        caller's, with `stream` made to wait for the copy -- or (view, grad_image, grad_alpha, grads_ready) with a
        CUDA event that marks the gradients' arrival and is waited for only before the backward pass.

        Streams: view k of the shard runs on stream k mod n_streams and adds its appearance sum into that
        stream's row of a partial buffer (the row's first view stores instead of adding: nothing is zero-filled).
        When a stream has enqueued its last view its row is all-reduced right there, on that stream, under the
        views the other streams still have in flight; every rank issues exactly n_streams such all-reduces, in
        stream order.  One fused sum over the rows and the (small) MAX all-reduce of the leaf statistics end
        the batch."""
        import torch.distributed as dist
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.buffers.leaf.reset()
        out = None
        mine = partition_views(len(views), rank, world_size)

        def view_inputs(vi, stream):
            if inputs is not None:
                got = inputs(vi, stream)
                return got if len(got) == 4 else (*got, None)
            gi, ga = grads if isinstance(grads[0], torch.Tensor) else grads[vi]
            return views[vi], gi, ga, None

        if self.n_streams == 1:
            main = torch.cuda.current_stream()
            if not mine:
                self.buffers.appearance.zero_()
            for k, vi in enumerate(mine):
                view, gi, ga, ready = view_inputs(vi, main)
                out = self.run_view(view, gi, ga, view_index=vi, appearance=self.buffers.appearance, overwrite=k == 0, grads_ready=ready)
            if distributed:
                dist.all_reduce(self.buffers.appearance, op=dist.ReduceOp.SUM, group=group)
        else:
            streams, parts = self._pipeline()
            main = torch.cuda.current_stream()
            for s in streams:
                s.wait_stream(main)
            for k, vi in enumerate(mine):
                slot = k % self.n_streams
                with torch.cuda.stream(streams[slot]):
                    view, gi, ga, ready = view_inputs(vi, streams[slot])
                    out = self.run_view(view, gi, ga, view_index=vi, appearance=parts[slot], overwrite=k < self.n_streams, grads_ready=ready)
            for slot, s in enumerate(streams):
                with torch.cuda.stream(s):
                    if slot >= len(mine):
                        parts[slot].zero_()          # a stream without a view this batch
                    if distributed:
                        dist.all_reduce(parts[slot], op=dist.ReduceOp.SUM, group=group)
            for s in streams:
                main.wait_stream(s)
            torch.sum(parts, dim=0, out=self.buffers.appearance)
        self.buffers.leaf.all_reduce(group)
        return out
