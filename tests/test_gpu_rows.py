"""GPU parity tests of the feature-row layout ((N,C) fp32 features blended as they are, C = 4, 8, 16, 32)
through the Python mirror and hence the C ABI: against the CPU oracle run as C/4 four-channel passes
and, where oracle/_ref is built, against C/4 runs of the reference's own CUDA backend on DC-only
spherical-harmonics coefficients.

Bar: images, alpha, blending weights and opacity gradients within rtol 1e-5 / atol 1e-6 of the
oracle; feature gradients of the reference are fp16, compared at half precision."""
import numpy as np
import pytest
import torch

import oracle as O
import ref_backend as RB
from helpers import ATOL_H, RTOL_H, assert_close, oracle_camera, silence_depth_ties, small_scene

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SH_DC = 0.28209479177387814


def _rows(n, channels, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn((n, channels), generator=g) * 0.5).contiguous()


def _silenced(view, pos, opac):
    """Opacities with all but the first point of every depth tie zeroed (see helpers.silence_depth_ties)."""
    from inpc_b200 import rasterization as R
    settings = R.INPCRasterizer.extract_settings(view, 0)
    n = pos.shape[0]
    feats = torch.zeros((n, 36), dtype=torch.float16, device=DEV)
    _, _, _, state, blobs, _ = R.forward_with_state(pos.to(DEV), feats, opac.to(DEV), settings, 8)
    dbg = R.debug_arrays(state, settings, blobs.point, blobs.instance)
    return silence_depth_ties(dbg["depth"].cpu().numpy(), dbg["n_touched"].cpu().numpy() > 0, opac.to(DEV))


@pytest.mark.parametrize("tile", [8, 16])
@pytest.mark.parametrize("channels", [4, 8, 16, 32])
def test_rows_forward_backward_match_oracle(channels, tile):
    import inpc_b200
    view, pos, _, opac = small_scene(n=12000, width=136, height=104, focal=120.0)
    v = view.to(DEV)
    feats = _rows(pos.shape[0], channels, 40 + channels)
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=tile).forward_rows(v, pos.to(DEV), f, o)
    st = O.rasterize_rows_forward(oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
    assert image.shape == (channels, view.camera.height, view.camera.width)
    assert_close(image.detach().cpu().numpy(), st.image, what="rows image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, what="rows alpha")
    assert_close(bw.detach().cpu().numpy(), st.blending_weights, what="rows blending weights")
    g = torch.Generator().manual_seed(41)
    gi = torch.randn(image.shape, generator=g) * 1e-3
    ga = torch.randn(alpha.shape, generator=g) * 1e-3
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    gf, go = O.rasterize_rows_backward(st, gi.numpy(), ga.numpy())
    assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-4, atol=1e-8, what="rows grad_opacities")
    assert_close(f.grad.detach().cpu().numpy(), gf, rtol=1e-5, atol=1e-9, what="rows grad_features")


@pytest.mark.parametrize("tile", [8, 16])
def test_rows_deep_tiles_training_and_inference(tile):
    """Lists cut into many segments, pixels that saturate in the middle: 16 channels."""
    import inpc_b200
    from inpc_b200.views import look_at_view
    view = look_at_view((0.0, 0.0, 3.0), (0.0, 0.0, 0.0), 64, 48, 60.0, 60.0)
    g = torch.Generator().manual_seed(42)
    n = 40000
    pos = torch.cat([torch.randn((n, 2), generator=g) * 0.15, torch.rand((n, 1), generator=g) - 0.5], dim=1).contiguous()
    opac = torch.rand((n, 1), generator=g) * 0.3 + 0.05
    feats = _rows(n, 16, 43)
    v = view.to(DEV)
    opac_d = _silenced(v, pos, opac)
    cam = oracle_camera(view)
    rast = inpc_b200.INPCRasterizer(tile_size=tile)
    f = feats.to(DEV).requires_grad_(True)
    o = opac_d.clone().requires_grad_(True)
    image, alpha, bw = rast.forward_rows(v, pos.to(DEV), f, o)
    st = O.rasterize_rows_forward(cam, pos.numpy(), feats.numpy(), opac_d.cpu().numpy(), tile=tile)
    assert (st.alpha == 1.0).sum() > 50
    assert_close(image.detach().cpu().numpy(), st.image, what="deep rows image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, what="deep rows alpha")
    assert_close(bw.detach().cpu().numpy(), st.blending_weights, what="deep rows blending weights")
    gi = torch.randn(image.shape, generator=g) * 1e-3
    ga = torch.randn(alpha.shape, generator=g) * 1e-3
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    gf, go = O.rasterize_rows_backward(st, gi.numpy(), ga.numpy())
    assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-4, atol=1e-8, max_bad=4, what="deep rows grad_opacities")
    assert_close(f.grad.detach().cpu().numpy(), gf, rtol=1e-5, atol=1e-9, what="deep rows grad_features")
    img, dep, alp = rast.render_rows(v, pos.to(DEV), feats.to(DEV), opac_d)
    oi, od, oa, _ = O.render_rows(cam, pos.numpy(), feats.numpy(), opac_d.cpu().numpy(), tile=tile)
    assert_close(img.cpu().numpy(), oi, what="deep rows inference image")
    assert_close(dep.cpu().numpy(), od, what="deep rows inference depth")
    assert_close(alp.cpu().numpy(), oa, what="deep rows inference alpha")


def test_rows_with_four_channels_equal_the_sh_path_on_its_view_features():
    """The four-channel row blend on the view-space features of the SH path gives the SH path's image."""
    import inpc_b200
    from inpc_b200 import rasterization as R
    view, pos, feats, opac = small_scene(n=15000, width=120, height=96, focal=110.0)
    v = view.to(DEV)
    settings = R.INPCRasterizer.extract_settings(v, 0)
    image, alpha, bw, state, blobs, _ = R.forward_with_state(pos.to(DEV), feats.to(DEV), opac.to(DEV), settings, 8)
    fv = R.debug_arrays(state, settings, blobs.point, blobs.instance)["feat_view"]
    img2, alpha2, bw2 = inpc_b200.INPCRasterizer(tile_size=8).forward_rows(v, pos.to(DEV), fv.contiguous(), opac.to(DEV))
    assert torch.equal(alpha, alpha2)
    # a point on a tile border gets one atomic per tile, in either order
    assert_close(bw2.cpu().numpy(), bw.cpu().numpy(), what="rows blending weights vs SH path")
    assert_close(img2.cpu().numpy(), image.cpu().numpy(), what="rows image vs SH path")


@pytest.mark.skipif(not RB.available(), reason="oracle/_ref/libinpc_ref.so not built")
def test_rows_match_reference_backend_run_per_channel_group():
    """16 channels against four runs of the reference on DC-only SH coefficients (features exactly
    representable: row value = fp32(0.2820948 * half))."""
    import inpc_b200
    view, pos, _, opac = small_scene(n=40000, width=240, height=160, focal=200.0)
    v = view.to(DEV)
    n, channels = pos.shape[0], 16
    g = torch.Generator().manual_seed(44)
    dc = (torch.randn((n, channels), generator=g) * 0.5).to(torch.float16)
    rows = (torch.tensor(SH_DC, dtype=torch.float32) * dc.float()).contiguous()
    pos_d = pos.to(DEV)
    opac_d = _silenced(v, pos, opac)
    H, W = view.camera.height, view.camera.width
    gi = (torch.randn((channels, H, W), generator=g) * 1e-3).to(DEV)
    ga = (torch.randn((1, H, W), generator=g) * 1e-3).to(DEV)
    f = rows.to(DEV).requires_grad_(True)
    o = opac_d.clone().requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=8).forward_rows(v, pos_d, f, o)
    torch.autograd.backward([image, alpha], [gi, ga])
    go_ref = torch.zeros((n,), dtype=torch.float64, device=DEV)
    for grp in range(channels // 4):
        sh = torch.zeros((n, 36), dtype=torch.float16)
        sh[:, :4] = dc[:, 4 * grp:4 * grp + 4]
        sh_d = sh.to(DEV)
        rimg, ralpha, rbw = RB.forward(v, 0, pos_d, sh_d, opac_d.reshape(-1))
        assert_close(image[4 * grp:4 * grp + 4].detach().cpu().numpy(), rimg.cpu().numpy(), what=f"rows image group {grp} vs reference")
        assert_close(alpha.detach().cpu().numpy(), ralpha.cpu().numpy(), what="rows alpha vs reference")
        assert_close(bw.detach().cpu().numpy(), rbw.cpu().numpy(), what="rows blending weights vs reference")
        rgf, rgo, _ = RB.backward(v, 0, gi[4 * grp:4 * grp + 4].contiguous(), ga if grp == 0 else torch.zeros_like(ga), rimg, ralpha,
                                  pos_d, opac_d.reshape(-1))
        go_ref += rgo.reshape(-1).double()
        # d/d(row) = d/d(coefficient) / 0.2820948; the reference rounds its coefficient gradient to fp16
        assert_close((f.grad[:, 4 * grp:4 * grp + 4] * SH_DC).cpu().numpy(), rgf[:, :4].float().cpu().numpy(), rtol=RTOL_H, atol=ATOL_H,
                     max_bad=3, what=f"rows grad_features group {grp} vs reference")
    assert_close(o.grad.reshape(-1).cpu().numpy(), go_ref.cpu().numpy(), rtol=1e-4, atol=1e-9, max_bad=3, what="rows grad_opacities vs reference")


def test_rows_empty_culled_and_bad_arguments():
    import inpc_b200
    view, pos, _, opac = small_scene(n=64, width=40, height=24, focal=30.0)
    v = view.to(DEV)
    rast = inpc_b200.INPCRasterizer()
    e = lambda *s: torch.empty(s, dtype=torch.float32, device=DEV)
    image, alpha, bw = rast.forward_rows(v, e(0, 3), e(0, 16), e(0, 1))
    assert image.shape == (16, 24, 40) and torch.all(image == 0) and torch.all(alpha == 0) and bw.numel() == 0
    behind = pos.clone()
    behind[:, 2] = 50.0
    f = _rows(64, 16, 45).to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = rast.forward_rows(v, behind.to(DEV), f, o)
    assert torch.all(image == 0) and torch.all(alpha == 0) and torch.all(bw == 0)
    (image.sum() + alpha.sum()).backward()
    assert torch.all(f.grad == 0) and torch.all(o.grad == 0)
    with pytest.raises(ValueError):
        rast.forward_rows(v, pos.to(DEV), e(64, 5), opac.to(DEV))
    with pytest.raises(TypeError):
        rast.forward_rows(v, pos.to(DEV), e(64, 16).half(), opac.to(DEV))
