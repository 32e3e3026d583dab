"""Shared helpers of the test-suite: view conversion for the oracle, tolerances, tie handling."""
from __future__ import annotations

import numpy as np
import torch

import oracle as O

# tolerances for fp32 images / weights / opacity gradients: 1e-5 relative, 1e-6 absolute
RTOL, ATOL = 1e-5, 1e-6
# grad_features is rounded to fp16 per coefficient (sh_utils.cuh:53-61): half-precision tolerance
RTOL_H, ATOL_H = 2e-3, 1e-7


def oracle_camera(view) -> O.Camera:
    c = view.camera
    return O.Camera(view.w2c.detach().cpu().numpy(), view.position.detach().cpu().numpy(), c.width, c.height,
                    c.focal_x, c.focal_y, c.center_x, c.center_y, c.near_plane, c.far_plane)


def n_bad(a, b, rtol=RTOL, atol=ATOL) -> int:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return int((np.abs(a - b) > atol + rtol * np.abs(b)).sum())


def assert_close(a, b, rtol=RTOL, atol=ATOL, max_bad=0, what=""):
    bad = n_bad(a, b, rtol, atol)
    if bad > max_bad:
        a64, b64 = np.asarray(a, np.float64), np.asarray(b, np.float64)
        raise AssertionError(f"{what}: {bad} of {a64.size} elements outside rtol={rtol} atol={atol} "
                             f"(max abs diff {np.abs(a64 - b64).max():.3e})")


def silence_depth_ties(depth: np.ndarray, visible: np.ndarray, opacities: torch.Tensor) -> torch.Tensor:
    """The reference orders points of bit-identical depth by the outcome of an atomic race
    (bilinear/kernels.cu:79-82), so two such points on one pixel blend in either order.  Giving all
    but the first point of every depth tie zero opacity removes the ambiguity without changing any
    sort key: a zero-opacity point contributes nothing and leaves the transmittance untouched.
    `depth` are the per-point depths of a first forward pass, `visible` marks the unculled points."""
    bits = depth.view(np.uint32).astype(np.int64)
    bits = np.where(visible, bits, -1 - np.arange(len(bits)))   # culled points never tie
    order = np.argsort(bits, kind="stable")
    ks = bits[order]
    dup = np.zeros(len(ks), bool)
    dup[1:] = ks[1:] == ks[:-1]
    out = opacities.clone()
    out.reshape(-1)[torch.from_numpy(order[dup]).to(out.device)] = 0.0
    return out


def small_scene(n=20000, width=160, height=120, seed=3, focal=140.0, eye=(0.7, 0.4, 2.6), near=0.01, far=100.0):
    """A rotated camera over uniformly scattered points, with culled points on every side."""
    from inpc_b200.views import look_at_view
    g = torch.Generator().manual_seed(seed)
    view = look_at_view(eye, (0.05, -0.02, 0.0), width, height, focal, focal * 1.07, center_x=width / 2 + 1.25,
                        center_y=height / 2 - 0.75, near_plane=near, far_plane=far)
    pos = (torch.rand((n, 3), generator=g) * 2 - 1) * 1.4
    feats = (torch.randn((n, 36), generator=g) * 0.5).to(torch.float16)
    opac = torch.sigmoid(torch.randn((n, 1), generator=g))
    return view, pos.contiguous(), feats.contiguous(), opac.contiguous()
