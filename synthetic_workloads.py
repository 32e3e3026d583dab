"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark
configurations.  They stand in for the Mip-NeRF360 / Tanks-and-Temples scenes the reference trains on
(no dataset is available offline).  Everything is generated on the CPU with `torch.Generator`, so
the same seed gives the same tensors on every machine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from inpc_b200.views import View, look_at_view

INITIAL_SIZE = 2.0   # root cube [-1,1]^3: a leaf of level l has edge 2 / 2**l


@dataclass
class Octree:
    centers: torch.Tensor   # (L,3) float32
    levels: torch.Tensor    # (L,) int32
    weights: torch.Tensor   # (L,) float32
    initial_size: float = INITIAL_SIZE

    def to(self, device) -> "Octree":
        return Octree(self.centers.to(device), self.levels.to(device), self.weights.to(device), self.initial_size)


def uniform_octree(level: int, seed: int, log_std: float = 1.0) -> Octree:
    """Every cell of one level; weights = softmax(N(0, log_std))."""
    g = torch.Generator().manual_seed(seed)
    r = 2 ** level
    edge = INITIAL_SIZE / r
    ax = (torch.arange(r, dtype=torch.float32) + 0.5) * edge - 1.0
    centers = torch.stack(torch.meshgrid(ax, ax, ax, indexing="ij"), dim=-1).reshape(-1, 3).contiguous()
    levels = torch.full((r ** 3,), level, dtype=torch.int32)
    weights = torch.softmax(torch.randn(r ** 3, generator=g) * log_std, dim=0)
    return Octree(centers, levels, weights.contiguous())


def adaptive_octree(n_leaves: int, seed: int, min_level: int = 6, max_level: int = 10, log_std: float = 2.0) -> Octree:
    """Carved adaptive octree: a random set of `min_level` cells of the root cube, of which a random
    half is split at every level up to `max_level`; trimmed to exactly `n_leaves` leaves.
    weights = softmax(N(0, log_std))."""
    g = torch.Generator().manual_seed(seed)
    depth = max_level - min_level
    # expected leaves per start cell when half the cells split at each of `depth` levels
    per_cell = sum(0.5 * 4 ** k for k in range(depth)) + 4 ** depth
    n_start = int(math.ceil(n_leaves / per_cell * 1.01)) + 2
    r = 2 ** min_level
    n_start = min(n_start, r ** 3)
    start = torch.randperm(r ** 3, generator=g)[:n_start]
    ijk = torch.stack([start // (r * r), (start // r) % r, start % r], dim=1)   # integer cell coordinates
    lv = torch.full((n_start,), min_level, dtype=torch.int32)
    done_ijk, done_lv = [], []
    offs = torch.tensor([[a, b, c] for a in (0, 1) for b in (0, 1) for c in (0, 1)], dtype=torch.int64)
    for level in range(min_level, max_level):
        split = torch.zeros(ijk.shape[0], dtype=torch.bool)
        split[torch.randperm(ijk.shape[0], generator=g)[:(ijk.shape[0] + 1) // 2]] = True
        done_ijk.append(ijk[~split])
        done_lv.append(lv[~split])
        parents = ijk[split]
        ijk = (parents[:, None, :] * 2 + offs[None, :, :]).reshape(-1, 3)
        lv = torch.full((ijk.shape[0],), level + 1, dtype=torch.int32)
    done_ijk.append(ijk)
    done_lv.append(lv)
    ijk = torch.cat(done_ijk)
    lv = torch.cat(done_lv)
    if ijk.shape[0] < n_leaves:
        raise RuntimeError(f"adaptive_octree produced {ijk.shape[0]} < {n_leaves} leaves; raise the start count")
    keep = torch.randperm(ijk.shape[0], generator=g)[:n_leaves].sort().values
    ijk, lv = ijk[keep], lv[keep]
    edge = INITIAL_SIZE / torch.pow(2.0, lv.to(torch.float32))
    centers = ((ijk.to(torch.float32) + 0.5) * edge[:, None] - 1.0).contiguous()
    weights = torch.softmax(torch.randn(n_leaves, generator=g) * log_std, dim=0)
    return Octree(centers, lv.contiguous(), weights.contiguous())


def orbit_view(azimuth: float, elevation: float, radius: float, width: int, height: int, focal: float,
               near_plane: float = 0.01, far_plane: float = 100.0) -> View:
    eye = (radius * math.cos(elevation) * math.sin(azimuth), radius * math.sin(elevation),
           radius * math.cos(elevation) * math.cos(azimuth))
    return look_at_view(eye, (0.0, 0.0, 0.0), width, height, focal, focal, near_plane=near_plane,
                        far_plane=far_plane)


def orbit_views(n: int, seed: int, radius: float = 3.0, width: int = 1237, height: int = 822,
                focal: float = 960.0) -> list[View]:
    """`n` cameras on a sphere of `radius` around the origin, random azimuth/elevation."""
    g = torch.Generator().manual_seed(seed)
    az = torch.rand(n, generator=g) * (2 * math.pi)
    el = (torch.rand(n, generator=g) - 0.5) * (math.pi / 3)
    return [orbit_view(float(a), float(e), radius, width, height, focal) for a, e in zip(az, el)]


def sh_features(n: int, seed: int, dist: str = "normal", scale: float = 0.5) -> torch.Tensor:
    """(n,36) float16 SH coefficients; 'normal' ~ N(0, scale), 'uniform' ~ U(0,1)."""
    g = torch.Generator().manual_seed(seed)
    if dist == "normal":
        return (torch.randn((n, 36), generator=g) * scale).to(torch.float16)
    return torch.rand((n, 36), generator=g).to(torch.float16)


def opacities_sigmoid(n: int, seed: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.sigmoid(torch.randn((n, 1), generator=g) * std + mean)


def gaussian_mixture_points(n: int, seed: int, n_components: int = 64, sigma: float = 0.1) -> torch.Tensor:
    """Positions from a mixture of isotropic Gaussians with centres inside [-1,1]^3."""
    g = torch.Generator().manual_seed(seed)
    mu = torch.rand((n_components, 3), generator=g) * 2 - 1
    comp = torch.randint(0, n_components, (n,), generator=g)
    return (mu[comp] + torch.randn((n, 3), generator=g) * sigma).contiguous()


def skewed_points(n: int, seed: int, hot_center=(0.0, 0.0, 2.0), hot_sigma: float = 0.02,
                  hot_fraction: float = 0.9) -> torch.Tensor:
    """`hot_fraction` of the points in one tight Gaussian (near the camera of `skew_view`), the rest
    uniform in [-1,1]^3: extreme per-tile imbalance and deep per-pixel lists."""
    g = torch.Generator().manual_seed(seed)
    n_hot = int(n * hot_fraction)
    hot = torch.tensor(hot_center, dtype=torch.float32) + torch.randn((n_hot, 3), generator=g) * hot_sigma
    rest = torch.rand((n - n_hot, 3), generator=g) * 2 - 1
    pts = torch.cat([hot, rest])
    return pts[torch.randperm(n, generator=g)].contiguous()


# ---- the five benchmark configurations ------------------------------------------------------------

def config0():
    """Tiny plumbing check: 4096 leaves at level 4, 2^16 draws, 256x256, f=300, eye (0,0,3)."""
    tree = uniform_octree(4, seed=0, log_std=1.0)
    view = look_at_view((0.0, 0.0, 3.0), (0.0, 0.0, 0.0), 256, 256, 300.0, 300.0)
    n = 1 << 16
    return dict(tree=tree, view=view, n_samples=n, features=sh_features(n, 10, "uniform"),
                opacities=opacities_sigmoid(n, 11))


def config1(n_samples: int = 1 << 23, n_leaves: int = 1 << 18):
    """Single-view training step: 2^18 adaptive leaves, 2^23 samples, 1237x822, f=960, radius-3 orbit."""
    tree = adaptive_octree(n_leaves, seed=1)
    view = orbit_view(0.6, 0.25, 3.0, 1237, 822, 960.0)
    return dict(tree=tree, view=view, n_samples=n_samples, features=sh_features(n_samples, 12, "normal", 0.5),
                opacities=opacities_sigmoid(n_samples, 13))


def config2(n_points: int = 1 << 25):
    """Pre-extracted inference: Gaussian-mixture cloud, 1920x1080, f=1400, eye (0,0.5,3)."""
    view = look_at_view((0.0, 0.5, 3.0), (0.0, 0.0, 0.0), 1920, 1080, 1400.0, 1400.0)
    g = torch.Generator().manual_seed(21)
    return dict(view=view, positions=gaussian_mixture_points(n_points, 20), features=sh_features(n_points, 22, "uniform"),
                opacities=(torch.rand((n_points, 1), generator=g) * 0.9 + 0.05))


def config3_views(n_views: int = 64):
    """The 64 orbit cameras of the view-sharded batch (octree and attributes are config 1's)."""
    return orbit_views(n_views, seed=2)


def config4(n_points: int = 1 << 24):
    """Skewed stress case: 90 % of the points in one sigma=0.02 Gaussian near the camera; 3840x2160."""
    view = look_at_view((0.0, 0.0, 3.0), (0.0, 0.0, 0.0), 3840, 2160, 2800.0, 2800.0)
    return dict(view=view, positions=skewed_points(n_points, 40), features=sh_features(n_points, 42, "normal", 0.5),
                opacities=opacities_sigmoid(n_points, 43, mean=2.0))
