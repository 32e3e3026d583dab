"""Minimal stand-ins for the NeRFICG `View` / `PerspectiveCamera` objects.

The bindings read only `view.w2c`, `view.position` and `view.camera.{width, height, focal_x, focal_y,
center_x, center_y, near_plane, far_plane, distortion}` (reference:
INPCCudaBackend/INPCCudaBackend/torch_bindings/rasterization.py:116-128, sampling.py:16-33), so any
object with those attributes works — NeRFICG's own classes included.  Camera space is +z forward,
+x right, +y down; `center_x/center_y` are absolute pixel coordinates.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PerspectiveCamera:
    width: int
    height: int
    focal_x: float
    focal_y: float
    center_x: float
    center_y: float
    near_plane: float = 0.01
    far_plane: float = 100.0
    distortion: object = None


@dataclass
class View:
    camera: PerspectiveCamera
    w2c: torch.Tensor        # (4,4) float32, world -> camera
    position: torch.Tensor   # (3,) float32, camera centre in world space

    def to(self, device) -> "View":
        return View(self.camera, self.w2c.to(device), self.position.to(device))


def look_at_view(eye, target, width, height, focal_x, focal_y, center_x=None, center_y=None, near_plane=0.01,
                 far_plane=100.0, up=(0.0, 1.0, 0.0), device="cpu") -> View:
    """View looking from `eye` at `target` (world up = +y, image y pointing down)."""
    eye_t = torch.tensor(eye, dtype=torch.float64)
    fwd = torch.tensor(target, dtype=torch.float64) - eye_t
    fwd = fwd / fwd.norm()
    up_t = torch.tensor(up, dtype=torch.float64)
    right = torch.linalg.cross(fwd, up_t)
    if right.norm() < 1e-9:
        right = torch.linalg.cross(fwd, torch.tensor((0.0, 0.0, 1.0), dtype=torch.float64))
    right = right / right.norm()
    down = torch.linalg.cross(fwd, right)
    rot = torch.stack([right, down, fwd])            # rows: camera axes in world coordinates
    w2c = torch.eye(4, dtype=torch.float64)
    w2c[:3, :3] = rot
    w2c[:3, 3] = -rot @ eye_t
    cam = PerspectiveCamera(int(width), int(height), float(focal_x), float(focal_y),
                            float(width) / 2 if center_x is None else float(center_x),
                            float(height) / 2 if center_y is None else float(center_y), float(near_plane),
                            float(far_plane))
    return View(cam, w2c.to(torch.float32).to(device).contiguous(), eye_t.to(torch.float32).to(device).contiguous())
