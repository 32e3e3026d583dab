"""Randomised small scenes against the CPU oracle, through the Python mirror and hence the C ABI: odd
image sizes, off-centre principal points, tight near / far planes, points snapped to pixel centres, pixel
borders and tile corners (the places where floor / ceil / `< 1` decisions flip), both tile sizes, training
forward + backward and inference."""
import numpy as np
import pytest
import torch

import oracle as O
from helpers import ATOL_H, RTOL_H, assert_close, oracle_camera

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _scene(seed):
    from inpc_b200.views import look_at_view
    g = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: float(torch.rand((), generator=g) * (hi - lo) + lo)
    width, height = int(r(9, 150)), int(r(9, 110))
    focal = r(20, 160)
    eye = (r(-0.6, 0.6), r(-0.6, 0.6), r(1.8, 3.2))
    view = look_at_view(eye, (r(-0.1, 0.1), r(-0.1, 0.1), 0.0), width, height, focal, focal * r(0.9, 1.1),
                        center_x=width / 2 + r(-3, 3), center_y=height / 2 + r(-3, 3), near_plane=r(0.01, 1.9), far_plane=r(2.6, 50.0))
    n = int(r(1, 2500))
    pos = (torch.rand((n, 3), generator=g) * 2 - 1) * 1.2
    # a third of the points on an axis-aligned plane in front of an (almost) axis-aligned camera would not hit
    # exact pixel coordinates; snap them in screen space instead: move the point along its camera ray's
    # perpendicular so that it projects onto a multiple of 0.5 px
    w2c = view.w2c.double()
    c = view.camera
    k = max(1, n // 3)
    p = torch.cat([pos[:k].double(), torch.ones((k, 1), dtype=torch.float64)], dim=1) @ w2c.T
    z = p[:, 2:3].clamp_min(0.5)
    sx = p[:, 0:1] / z * c.focal_x + c.center_x
    sy = p[:, 1:2] / z * c.focal_y + c.center_y
    sx, sy = torch.round(sx * 2) / 2, torch.round(sy * 2) / 2
    cam = torch.cat([(sx - c.center_x) / c.focal_x * z, (sy - c.center_y) / c.focal_y * z, z, torch.ones_like(z)], dim=1)
    pos[:k] = (cam @ torch.linalg.inv(w2c).T)[:, :3].float()
    feats = (torch.randn((n, 36), generator=g) * 0.5).to(torch.float16)
    opac = torch.rand((n, 1), generator=g) ** 0.5
    opac[torch.rand((n, 1), generator=g) < 0.1] = 1.0
    opac[torch.rand((n, 1), generator=g) < 0.05] = 0.0
    return view, pos.contiguous(), feats.contiguous(), opac.contiguous(), g


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_scene_matches_oracle(seed):
    import inpc_b200
    view, pos, feats, opac, g = _scene(seed)
    cam = oracle_camera(view)
    v = view.to(DEV)
    H, W = view.camera.height, view.camera.width
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    for tile in (8, 16):
        rast = inpc_b200.INPCRasterizer(tile_size=tile)
        f = feats.to(DEV).requires_grad_(True)
        o = opac.to(DEV).requires_grad_(True)
        image, alpha, bw = rast(v, 0, pos.to(DEV), f, o)
        st = O.rasterize_forward(O.BILINEAR, cam, pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
        assert_close(image.detach().cpu().numpy(), st.image, what=f"seed {seed} tile {tile} image")
        assert_close(alpha.detach().cpu().numpy(), st.alpha, what=f"seed {seed} tile {tile} alpha")
        assert_close(bw.detach().cpu().numpy(), st.blending_weights, what=f"seed {seed} tile {tile} blending weights")
        torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
        gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
        assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-4, atol=1e-8, max_bad=2, what=f"seed {seed} tile {tile} grad_opacities")
        assert_close(f.grad.float().detach().cpu().numpy(), gf.astype(np.float32), rtol=RTOL_H, atol=ATOL_H, max_bad=36,
                     what=f"seed {seed} tile {tile} grad_features")
        img, dep, alp = rast.render_preextracted(v, 0, pos.to(DEV), feats.to(DEV), opac.to(DEV), None)
        oi, od, oa, _ = O.render_preextracted(0, cam, pos.numpy(), feats.numpy(), opac.numpy(), None, 0.05 / view.camera.focal_y, 3.0, tile=tile)
        assert_close(img.cpu().numpy(), oi, what=f"seed {seed} tile {tile} inference image")
        assert_close(dep.cpu().numpy(), od, rtol=1e-5, atol=1e-5, what=f"seed {seed} tile {tile} inference depth")
        assert_close(alp.cpu().numpy(), oa, what=f"seed {seed} tile {tile} inference alpha")


@pytest.mark.parametrize("seed", [100, 101, 102, 103])
def test_random_scene_gaussian_mode_matches_oracle(seed):
    """Gaussian splats (fast exponentials on the device, libm in the oracle: looser tolerances)."""
    import inpc_b200
    view, pos, feats, opac, g = _scene(seed)
    pos, feats, opac = pos[:600], feats[:600], opac[:600]
    cam = oracle_camera(view)
    v = view.to(DEV)
    H, W = view.camera.height, view.camera.width
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    for tile in (8, 16):
        f = feats.to(DEV).requires_grad_(True)
        o = opac.to(DEV).requires_grad_(True)
        image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=tile)(v, 1, pos.to(DEV), f, o)
        st = O.rasterize_forward(O.GAUSSIAN, cam, pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
        assert_close(image.detach().cpu().numpy(), st.image, rtol=1e-4, atol=1e-5, max_bad=4, what=f"seed {seed} tile {tile} gaussian image")
        assert_close(alpha.detach().cpu().numpy(), st.alpha, rtol=1e-4, atol=1e-5, max_bad=4, what=f"seed {seed} tile {tile} gaussian alpha")
        torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
        gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
        assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-3, atol=1e-8, max_bad=8, what=f"seed {seed} tile {tile} gaussian grad_opacities")
        assert_close(f.grad.float().detach().cpu().numpy(), gf.astype(np.float32), rtol=4e-3, atol=2e-7, max_bad=36 * 8,
                     what=f"seed {seed} tile {tile} gaussian grad_features")
