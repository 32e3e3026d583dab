"""GPU parity tests of the rasterizer, through the Python mirror of the reference bindings and hence
through the C ABI: against the CPU oracle (both tile sizes) and, where oracle/_ref is built, against
the reference's own CUDA backend on the same device.

Bar: integer results (tile bounds, depth keys, point order, per-tile lists, ranges) bit-exact; fp32
images / weights / opacity gradients within rtol 1e-5, atol 1e-6; fp16 feature gradients within
half precision."""
import numpy as np
import pytest
import torch

import oracle as O
import ref_backend as RB
from helpers import (ATOL, ATOL_H, RTOL, RTOL_H, assert_close, oracle_camera, silence_depth_ties, small_scene)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _fwd(view, mode, pos, feats, opac, tile):
    from inpc_b200 import rasterization as R
    settings = R.INPCRasterizer.extract_settings(view, mode)
    image, alpha, bw, state, blobs, _ = R.forward_with_state(pos, feats, opac, settings, tile)
    dbg = R.debug_arrays(state, settings, blobs.point, blobs.instance)
    torch.cuda.synchronize()
    return image, alpha, bw, state, {k: v.detach().cpu().numpy() for k, v in dbg.items()}


def _u32(a):
    return np.ascontiguousarray(a).view(np.uint32) if a.dtype != np.uint32 else a


@pytest.mark.parametrize("tile", [8, 16])
def test_bilinear_forward_matches_oracle(tile):
    view, pos, feats, opac = small_scene()
    v = view.to(DEV)
    image, alpha, bw, state, dbg = _fwd(v, 0, pos.to(DEV), feats.to(DEV), opac.to(DEV), tile)
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
    assert 0 < state.n_visible < pos.shape[0]                 # the scene has culled points on purpose
    # integer stages: bit-exact
    assert np.array_equal(dbg["n_touched"].astype(np.uint32), st.n_touched)
    assert np.array_equal(dbg["bounds"].view(np.uint16), st.bounds)
    assert np.array_equal(_u32(dbg["depth"]), _u32(st.depth))
    assert np.array_equal(_u32(dbg["screen"]), _u32(st.screen))
    assert np.array_equal(dbg["sorted_points"].astype(np.uint32), st.sorted_points)
    assert np.array_equal(dbg["inst_point"].astype(np.uint32), st.inst_point)
    assert np.array_equal(dbg["ranges"].astype(np.uint32), st.ranges)
    # floating point
    assert_close(dbg["feat_view"], st.feat_view, what="view-space features")
    assert_close(image.detach().cpu().numpy(), st.image, what="image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, what="alpha")
    assert_close(bw.detach().cpu().numpy(), st.blending_weights, what="blending weights")


@pytest.mark.parametrize("tile", [8, 16])
def test_bilinear_backward_matches_oracle(tile):
    import inpc_b200
    view, pos, feats, opac = small_scene()
    v = view.to(DEV)
    g = torch.Generator().manual_seed(11)
    H, W = view.camera.height, view.camera.width
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    p = pos.to(DEV).requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=tile)(v, 0, p, f, o)
    assert not bw.requires_grad
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    assert p.grad is None                                       # positions get no gradient (rasterization.py:96-101)
    assert f.grad.dtype == torch.float16 and f.grad.shape == (pos.shape[0], 36)
    assert o.grad.dtype == torch.float32 and o.grad.shape == (pos.shape[0], 1)
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
    gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
    assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-4, atol=1e-9, what="grad_opacities")
    assert_close(f.grad.float().detach().cpu().numpy(), gf.astype(np.float32), rtol=RTOL_H, atol=ATOL_H, what="grad_features")
    culled = st.n_touched == 0
    assert torch.all(f.grad[torch.from_numpy(culled).to(DEV)] == 0) and torch.all(o.grad[torch.from_numpy(culled).to(DEV)] == 0)


@pytest.mark.parametrize("tile", [8, 16])
def test_gaussian_forward_backward_match_oracle(tile):
    import inpc_b200
    view, pos, feats, opac = small_scene(n=6000, width=96, height=80, focal=90.0)
    v = view.to(DEV)
    g = torch.Generator().manual_seed(12)
    H, W = view.camera.height, view.camera.width
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=tile)(v, 1, pos.to(DEV), f, o)
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    st = O.rasterize_forward(O.GAUSSIAN, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
    gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
    # exp / sqrt differ in the last bits between libm and the device: a point whose footprint ends within
    # rounding of a tile edge or of the cut-off may be in or out, hence a small allowance
    assert_close(image.detach().cpu().numpy(), st.image, rtol=1e-4, atol=1e-5, max_bad=8, what="gaussian image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, rtol=1e-4, atol=1e-5, max_bad=4, what="gaussian alpha")
    assert_close(bw.detach().cpu().numpy(), st.blending_weights, rtol=1e-4, atol=1e-6, max_bad=8, what="gaussian blending weights")
    assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-3, atol=1e-8, max_bad=8, what="gaussian grad_opacities")
    assert_close(f.grad.float().detach().cpu().numpy(), gf.astype(np.float32), rtol=4e-3, atol=2e-7, max_bad=36 * 8, what="gaussian grad_features")


@pytest.mark.parametrize("mode", [0, 1])
def test_render_variants_match_oracle(mode):
    import inpc_b200
    view, pos, feats, opac = small_scene(n=6000, width=96, height=80, focal=90.0)
    v = view.to(DEV)
    g = torch.Generator().manual_seed(13)
    raw = torch.cat([torch.randn((pos.shape[0], 1), generator=g).to(torch.float16), feats], dim=1).contiguous()
    scales = (torch.rand((pos.shape[0],), generator=g) * 0.01 + 0.002)
    rast = inpc_b200.INPCRasterizer(tile_size=16)
    cam = oracle_camera(view)
    sw = 1.5 * 0.05 / view.camera.focal_y
    tol = dict(rtol=2e-4, atol=2e-5, max_bad=12 if mode == 1 else 0)
    # raw 37-half layout: opacity = 1 - exp(-exp(raw)) with the device's fast exponential
    img, dep, alp = rast.render(v, mode, pos.to(DEV), raw.to(DEV), sigma_world_scale=1.5, sigma_cutoff=2.5)
    oi, od, oa, _ = O.render(mode, cam, pos.numpy(), raw.numpy(), sw, 2.5, tile=16)
    assert_close(img.detach().cpu().numpy(), oi, what="render image", **tol)
    assert_close(dep.detach().cpu().numpy(), od, what="render depth", **tol)
    assert_close(alp.detach().cpu().numpy(), oa, what="render alpha", **tol)
    # pre-extracted, without and with per-point scales
    for sc in (None, scales):
        img, dep, alp = rast.render_preextracted(v, mode, pos.to(DEV), feats.to(DEV), opac.to(DEV), None if sc is None else sc.to(DEV),
                                                 sigma_world_scale=1.5, sigma_cutoff=2.5)
        oi, od, oa, _ = O.render_preextracted(mode, cam, pos.numpy(), feats.numpy(), opac.numpy(), None if sc is None else sc.numpy(), sw, 2.5, tile=16)
        assert_close(img.detach().cpu().numpy(), oi, what="preextracted image", **tol)
        assert_close(dep.detach().cpu().numpy(), od, what="preextracted depth", **tol)
        assert_close(alp.detach().cpu().numpy(), oa, what="preextracted alpha", **tol)


# ---------------------------------------------------------------------------- against the reference backend

needs_ref = pytest.mark.skipif(not RB.available(), reason="oracle/_ref/libinpc_ref.so not built")


@needs_ref
def test_bilinear_matches_reference_backend():
    """Tile ranges, per-tile lists and depth keys bit-exact at the reference's 8x8 tiling; images,
    weights and gradients within rtol 1e-5 / atol 1e-6.  Depth ties are silenced first."""
    import inpc_b200
    view, pos, feats, opac = small_scene(n=60000, width=320, height=200, focal=260.0)
    v = view.to(DEV)
    pos_d, feats_d = pos.to(DEV), feats.to(DEV)
    _, _, _, _, dbg0 = _fwd(v, 0, pos_d, feats_d, opac.to(DEV), 8)
    opac_d = silence_depth_ties(dbg0["depth"], dbg0["n_touched"] > 0, opac.to(DEV))
    image, alpha, bw, state, dbg = _fwd(v, 0, pos_d, feats_d, opac_d, 8)
    rimg, ralpha, rbw = RB.forward(v, 0, pos_d, feats_d, opac_d.reshape(-1))
    ref = RB.intermediates(v, pos.shape[0])
    assert ref["n_visible"] == state.n_visible and ref["n_instances"] == state.n_instances
    vis = ref["n_touched"] > 0
    assert np.array_equal(ref["n_touched"], dbg["n_touched"].astype(np.uint32))
    assert np.array_equal(ref["bounds"][vis], dbg["bounds"].view(np.uint16)[vis])
    assert np.array_equal(_u32(ref["depth"])[vis], _u32(dbg["depth"])[vis])
    assert np.array_equal(_u32(ref["screen"])[vis], _u32(dbg["screen"])[vis])
    assert np.array_equal(ref["sorted_depth_keys"], dbg["sorted_depth_keys"].astype(np.uint32))
    assert np.array_equal(ref["ranges"], dbg["ranges"].astype(np.uint32))
    # order: identical after ordering depth ties by point id (the reference's tie order is a race)
    bits = _u32(dbg["depth"])

    def canon(ids, tiles=None):
        ids = ids.astype(np.int64)
        key = (bits[ids].astype(np.int64) << 32) | ids
        if tiles is not None:
            return ids[np.lexsort((key, tiles))]
        return ids[np.argsort(key, kind="stable")]
    assert np.array_equal(canon(ref["sorted_points"]), dbg["sorted_points"].astype(np.int64))
    tiles = np.repeat(np.arange(ref["ranges"].shape[0]), (ref["ranges"][:, 1] - ref["ranges"][:, 0]).astype(np.int64))
    assert np.array_equal(canon(ref["inst_point"], tiles), dbg["inst_point"].astype(np.int64))
    assert_close(dbg["feat_view"][vis], ref["feat_view"][vis], what="view-space features vs reference")
    assert_close(image.detach().cpu().numpy(), rimg.detach().cpu().numpy(), what="image vs reference")
    assert_close(alpha.detach().cpu().numpy(), ralpha.detach().cpu().numpy(), what="alpha vs reference")
    assert_close(bw.detach().cpu().numpy(), rbw.detach().cpu().numpy(), what="blending weights vs reference")
    # backward, both tile sizes against the reference's gradients
    g = torch.Generator().manual_seed(14)
    H, W = view.camera.height, view.camera.width
    gi = (torch.randn((4, H, W), generator=g) * 1e-3).to(DEV)
    ga = (torch.randn((1, H, W), generator=g) * 1e-3).to(DEV)
    rgf, rgo, _ = RB.backward(v, 0, gi, ga, rimg, ralpha, pos_d, opac_d.reshape(-1))
    for tile in (8, 16):
        f = feats_d.clone().requires_grad_(True)
        o = opac_d.clone().requires_grad_(True)
        im, al, _ = inpc_b200.INPCRasterizer(tile_size=tile)(v, 0, pos_d, f, o)
        torch.autograd.backward([im, al], [gi, ga])
        assert_close(im.detach().cpu().numpy(), rimg.detach().cpu().numpy(), what=f"image (tile {tile}) vs reference")
        # The reference sums per-fragment terms with float atomics in a race-dependent order; for a
        # near-opaque fragment the terms carry 1/max(1-alpha, 1e-8) and cancel, so an element or two of
        # its own result moves between runs by more than the tolerance.
        assert_close(o.grad.detach().cpu().numpy(), rgo.detach().cpu().numpy(), rtol=1e-4, atol=1e-9, max_bad=3, what="grad_opacities vs reference")
        assert_close(f.grad.float().detach().cpu().numpy(), rgf.float().detach().cpu().numpy(), rtol=RTOL_H, atol=ATOL_H, max_bad=3, what="grad_features vs reference")


@needs_ref
@pytest.mark.parametrize("mode", [0, 1])
def test_inference_matches_reference_backend(mode):
    import inpc_b200
    view, pos, feats, opac = small_scene(n=30000, width=200, height=160, focal=180.0)
    v = view.to(DEV)
    g = torch.Generator().manual_seed(15)
    raw = torch.cat([torch.randn((pos.shape[0], 1), generator=g).to(torch.float16), feats], dim=1).contiguous().to(DEV)
    pos_d, feats_d = pos.to(DEV), feats.to(DEV)
    _, _, _, _, dbg0 = _fwd(v, 0, pos_d, feats_d, opac.to(DEV), 8)
    dead = silence_depth_ties(dbg0["depth"], dbg0["n_touched"] > 0, torch.ones_like(opac).to(DEV)).reshape(-1) == 0
    opac_d = opac.to(DEV).clone()
    opac_d[dead] = 0.0
    raw[dead, 0] = -30000.0                                      # exp(-inf-ish) -> opacity exactly 0
    rast = inpc_b200.INPCRasterizer(tile_size=16)
    sw = 2.0 * 0.05 / view.camera.focal_y
    tol = dict(rtol=RTOL, atol=ATOL) if mode == 0 else dict(rtol=1e-4, atol=1e-5, max_bad=16)
    img, dep, alp = rast.render(v, mode, pos_d, raw, sigma_world_scale=2.0, sigma_cutoff=3.0)
    rimg, rdep, ralp = RB.render(v, mode, pos_d, raw, sw, 3.0)
    assert_close(img.detach().cpu().numpy(), rimg.detach().cpu().numpy(), what="render image vs reference", **tol)
    assert_close(dep.detach().cpu().numpy(), rdep.detach().cpu().numpy(), what="render depth vs reference", **tol)
    assert_close(alp.detach().cpu().numpy(), ralp.detach().cpu().numpy(), what="render alpha vs reference", **tol)
    img, dep, alp = rast.render_preextracted(v, mode, pos_d, feats_d, opac_d, None, sigma_world_scale=2.0, sigma_cutoff=3.0)
    rimg, rdep, ralp = RB.render_preextracted(v, mode, pos_d, feats_d, opac_d.reshape(-1), None, sw, 3.0)
    assert_close(img.detach().cpu().numpy(), rimg.detach().cpu().numpy(), what="preextracted image vs reference", **tol)
    assert_close(dep.detach().cpu().numpy(), rdep.detach().cpu().numpy(), what="preextracted depth vs reference", **tol)
    assert_close(alp.detach().cpu().numpy(), ralp.detach().cpu().numpy(), what="preextracted alpha vs reference", **tol)


@needs_ref
def test_gaussian_training_matches_reference_backend():
    import inpc_b200
    view, pos, feats, opac = small_scene(n=30000, width=200, height=160, focal=180.0)
    v = view.to(DEV)
    pos_d, feats_d = pos.to(DEV), feats.to(DEV)
    _, _, _, _, dbg0 = _fwd(v, 0, pos_d, feats_d, opac.to(DEV), 8)
    opac_d = silence_depth_ties(dbg0["depth"], dbg0["n_touched"] > 0, opac.to(DEV))
    g = torch.Generator().manual_seed(16)
    H, W = view.camera.height, view.camera.width
    gi = (torch.randn((4, H, W), generator=g) * 1e-3).to(DEV)
    ga = (torch.randn((1, H, W), generator=g) * 1e-3).to(DEV)
    rimg, ralpha, rbw = RB.forward(v, 1, pos_d, feats_d, opac_d.reshape(-1))
    rgf, rgo, _ = RB.backward(v, 1, gi, ga, rimg, ralpha, pos_d, opac_d.reshape(-1))
    f = feats_d.clone().requires_grad_(True)
    o = opac_d.clone().requires_grad_(True)
    im, al, bw = inpc_b200.INPCRasterizer(tile_size=8)(v, 1, pos_d, f, o)
    torch.autograd.backward([im, al], [gi, ga])
    assert_close(im.detach().cpu().numpy(), rimg.detach().cpu().numpy(), what="gaussian image vs reference")
    assert_close(al.detach().cpu().numpy(), ralpha.detach().cpu().numpy(), what="gaussian alpha vs reference")
    assert_close(bw.detach().cpu().numpy(), rbw.detach().cpu().numpy(), rtol=1e-4, atol=1e-6, what="gaussian blending weights vs reference")
    assert_close(o.grad.detach().cpu().numpy(), rgo.detach().cpu().numpy(), rtol=1e-3, atol=1e-8, what="gaussian grad_opacities vs reference")
    assert_close(f.grad.float().detach().cpu().numpy(), rgf.float().detach().cpu().numpy(), rtol=4e-3, atol=2e-7, what="gaussian grad_features vs reference")


# ---------------------------------------------------------------------------- edge cases and properties

def test_empty_and_fully_culled_inputs():
    import inpc_b200
    view, pos, feats, opac = small_scene(n=64, width=40, height=24, focal=30.0)
    v = view.to(DEV)
    rast = inpc_b200.INPCRasterizer()
    e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=DEV)
    image, alpha, bw = rast(v, 0, e(0, 3), e(0, 36, dt=torch.float16), e(0, 1))
    assert image.shape == (4, 24, 40) and torch.all(image == 0) and torch.all(alpha == 0) and bw.numel() == 0
    behind = pos.clone()
    behind[:, 2] = 50.0                                           # behind the camera: everything culled
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = rast(v, 0, behind.to(DEV), f, o)
    assert torch.all(image == 0) and torch.all(alpha == 0) and torch.all(bw == 0)
    (image.sum() + alpha.sum()).backward()
    assert torch.all(f.grad == 0) and torch.all(o.grad == 0)
    img, dep, alp = rast.render_preextracted(v, 0, behind.to(DEV), feats.to(DEV), opac.to(DEV))
    assert torch.all(img == 0) and torch.all(dep == 0) and torch.all(alp == 0)


def test_single_hot_tile_and_deep_pixel_lists():
    """All points inside one tile: ragged final batch, early termination, alpha clamped to 1."""
    import inpc_b200
    from inpc_b200.views import look_at_view
    view = look_at_view((0.0, 0.0, 3.0), (0.0, 0.0, 0.0), 64, 48, 60.0, 60.0)
    g = torch.Generator().manual_seed(17)
    n = 5000
    pos = torch.cat([torch.randn((n, 2), generator=g) * 0.02, torch.rand((n, 1), generator=g) - 0.5], dim=1).contiguous()
    feats = (torch.randn((n, 36), generator=g) * 0.5).to(torch.float16)
    opac = torch.sigmoid(torch.randn((n, 1), generator=g) + 2)
    for tile in (8, 16):
        image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=tile)(view.to(DEV), 0, pos.to(DEV), feats.to(DEV), opac.to(DEV))
        st = O.rasterize_forward(O.BILINEAR, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
        assert (st.alpha == 1.0).sum() > 0
        assert_close(image.detach().cpu().numpy(), st.image, what="hot-tile image")
        assert_close(alpha.detach().cpu().numpy(), st.alpha, what="hot-tile alpha")
        assert_close(bw.detach().cpu().numpy(), st.blending_weights, what="hot-tile blending weights")


def test_inference_on_deep_tiles_stops_where_the_reference_stops():
    """Tiles whose lists are cut into many segments: pixels that saturate in the middle of the list
    must report the transmittance of the fragment that stopped them (expected depth = Z / (1 - T))."""
    import inpc_b200
    from inpc_b200.views import look_at_view
    view = look_at_view((0.0, 0.0, 3.0), (0.0, 0.0, 0.0), 64, 48, 60.0, 60.0)
    g = torch.Generator().manual_seed(18)
    n = 40000
    pos = torch.cat([torch.randn((n, 2), generator=g) * 0.15, torch.rand((n, 1), generator=g) - 0.5], dim=1).contiguous()
    feats = (torch.randn((n, 36), generator=g) * 0.5).to(torch.float16)
    opac = torch.rand((n, 1), generator=g) * 0.3 + 0.05
    v = view.to(DEV)
    _, _, _, _, dbg0 = _fwd(v, 0, pos.to(DEV), feats.to(DEV), opac.to(DEV), 8)
    opac_d = silence_depth_ties(dbg0["depth"], dbg0["n_touched"] > 0, opac.to(DEV))
    for tile in (8, 16):
        img, dep, alp = inpc_b200.INPCRasterizer(tile_size=tile).render_preextracted(
            v, 0, pos.to(DEV), feats.to(DEV), opac_d, None, sigma_world_scale=1.0, sigma_cutoff=3.0)
        oi, od, oa, _ = O.render_preextracted(0, oracle_camera(view), pos.numpy(), feats.numpy(), opac_d.cpu().numpy(), None,
                                              1.0 * 0.05 / view.camera.focal_y, 3.0, tile=tile)
        assert (oa == 1.0).sum() > 50 and ((oa > 0) & (oa < 1)).sum() > 50
        assert_close(img.detach().cpu().numpy(), oi, what="deep-tile image")
        assert_close(dep.detach().cpu().numpy(), od, what="deep-tile depth")
        assert_close(alp.detach().cpu().numpy(), oa, what="deep-tile alpha")


def test_argument_errors_raise():
    import inpc_b200
    from inpc_b200 import _cabi
    view, pos, feats, opac = small_scene(n=32, width=40, height=24, focal=30.0)
    v = view.to(DEV)
    rast = inpc_b200.INPCRasterizer()
    with pytest.raises(TypeError):
        rast(v, 0, pos.to(DEV), feats.float().to(DEV), opac.to(DEV))          # features must be fp16
    with pytest.raises(ValueError):
        rast(v, 0, pos, feats.to(DEV), opac.to(DEV))                           # positions on the CPU
    with pytest.raises(ValueError):
        rast(v, 0, pos.to(DEV), feats[:, :30].contiguous().to(DEV), opac.to(DEV))
    with pytest.raises(ValueError):
        inpc_b200.INPCRasterizer(tile_size=12)
    # non-contiguous inputs are accepted, as the reference's .contiguous() calls do
    wide = torch.zeros((32, 6), device=DEV)
    wide[:, ::2] = pos.to(DEV)
    a = rast(v, 0, wide[:, ::2], feats.to(DEV), opac.to(DEV))[0]
    b = rast(v, 0, pos.to(DEV), feats.to(DEV), opac.to(DEV))[0]
    assert torch.equal(a, b)
    # an invalid mode falls back to bilinear with a warning (rasterization.py:109-113)
    with pytest.warns(UserWarning):
        c = rast(v, 7, pos.to(DEV), feats.to(DEV), opac.to(DEV))[0]
    assert torch.equal(c, b)
    # the C ABI itself rejects a bad tile size with a message
    import ctypes as C
    st = _cabi.RasterState()
    rc = _cabi.lib().inpc_rasterize_forward(0, 5, None, 0, None, None, None, None, None, None, _cabi.ALLOC_FN(lambda u, n: 0),
                                            _cabi.ALLOC_FN(lambda u, n: 0), None, C.byref(st), None)
    assert rc == -1 and b"view" in _cabi.lib().inpc_last_error()


def test_full_size_properties():
    """Full benchmark sizes (2^23 points, 1237x822): properties that need no oracle — sorted keys, ranges
    partition the instance list, tile-size independence of the image, run-to-run determinism."""
    from inpc_b200 import rasterization as R
    import synthetic_workloads as syn
    n = 1 << 23
    view = syn.orbit_view(0.6, 0.25, 3.0, 1237, 822, 960.0).to(DEV)
    g = torch.Generator(device=DEV).manual_seed(18)
    pos = (torch.rand((n, 3), generator=g, device=DEV) * 2 - 1)
    feats = (torch.randn((n, 36), generator=g, device=DEV) * 0.5).to(torch.float16)
    opac = torch.sigmoid(torch.randn((n, 1), generator=g, device=DEV))
    settings = R.INPCRasterizer.extract_settings(view, 0)
    out = {}
    for tile in (8, 16):
        image, alpha, bw, state, blobs, _ = R.forward_with_state(pos, feats, opac, settings, tile)
        dbg = R.debug_arrays(state, settings, blobs.point, blobs.instance)
        keys = dbg["sorted_depth_keys"].to(torch.int64) & 0xFFFFFFFF
        assert bool((keys[1:] >= keys[:-1]).all())
        r = dbg["ranges"].to(torch.int64) & 0xFFFFFFFF
        lens = r[:, 1] - r[:, 0]
        assert int(lens.sum()) == state.n_instances and bool((lens >= 0).all())
        nonempty = r[lens > 0]
        assert bool((nonempty[1:, 0] == nonempty[:-1, 1]).all()) and int(nonempty[0, 0]) == 0
        assert int(dbg["n_touched"].to(torch.int64).sum()) == state.n_instances
        # per-tile lists are depth-sorted
        d = dbg["depth"][dbg["inst_point"].to(torch.int64)]
        tile_of = torch.repeat_interleave(torch.arange(r.shape[0], device=DEV), lens)
        same = tile_of[1:] == tile_of[:-1]
        assert bool((d[1:][same] >= d[:-1][same]).all())
        out[tile] = (image, alpha, bw)
        again = R.forward_with_state(pos, feats, opac, settings, tile)
        assert torch.equal(again[0], image) and torch.equal(again[1], alpha)
    # the image does not depend on the tiling, up to the summation order of per-segment partial colours
    assert torch.allclose(out[8][0], out[16][0], rtol=1e-5, atol=1e-6) and torch.allclose(out[8][1], out[16][1], rtol=1e-5, atol=1e-6)
    assert torch.allclose(out[8][2], out[16][2], rtol=1e-5, atol=1e-6)
    covered = out[8][1] > 0
    assert 0.2 < covered.float().mean().item() <= 1.0


@needs_ref
def test_full_size_training_step_matches_reference_backend():
    """The bench workload itself (2^23 samples of the 2^18-leaf octree, 1237x822, forward and backward)
    against the reference's CUDA backend on the same points, both tilings.  Depth ties (about a third of
    the clustered samples share their depth's bit pattern with another one) are silenced first."""
    import inpc_b200
    from inpc_b200 import rasterization as R, sampling as S
    import synthetic_workloads as syn
    cfg = syn.config1()
    view, tree = cfg["view"].to(DEV), cfg["tree"].to(DEV)
    feats, opac = cfg["features"].to(DEV), cfg["opacities"].to(DEV)
    n = cfg["n_samples"]
    pos, _ = S.ProbabilityFieldSampler(0).generate_training_samples(tree.centers, tree.levels, tree.weights, view, n, tree.initial_size)
    settings = R.INPCRasterizer.extract_settings(view, 0)
    _, _, _, state, blobs, _ = R.forward_with_state(pos, feats, opac, settings, 8)
    dbg = R.debug_arrays(state, settings, blobs.point, blobs.instance)
    opac_s = silence_depth_ties(dbg["depth"].cpu().numpy(), dbg["n_touched"].cpu().numpy() > 0, opac)
    del dbg, blobs
    H, W = view.camera.height, view.camera.width
    g = torch.Generator().manual_seed(5)
    gi = (torch.randn((4, H, W), generator=g) * 1e-3).to(DEV)
    ga = (torch.randn((1, H, W), generator=g) * 1e-3).to(DEV)
    rimg, ralpha, rbw = RB.forward(view, 0, pos, feats, opac_s.reshape(-1))
    rgf, rgo, _ = RB.backward(view, 0, gi, ga, rimg, ralpha, pos, opac_s.reshape(-1))
    for tile in (8, 16):
        f = feats.clone().requires_grad_(True)
        o = opac_s.clone().requires_grad_(True)
        im, al, bw = inpc_b200.INPCRasterizer(tile_size=tile)(view, 0, pos, f, o)
        torch.autograd.backward([im, al], [gi, ga])
        assert_close(im.detach().cpu().numpy(), rimg.cpu().numpy(), what=f"full-size image (tile {tile})")
        assert_close(al.detach().cpu().numpy(), ralpha.cpu().numpy(), what=f"full-size alpha (tile {tile})")
        assert_close(bw.detach().cpu().numpy(), rbw.cpu().numpy(), what=f"full-size blending weights (tile {tile})")
        assert_close(f.grad.float().cpu().numpy(), rgf.float().cpu().numpy(), rtol=RTOL_H, atol=ATOL_H, max_bad=36,
                     what=f"full-size grad_features (tile {tile})")
        # the reference sums the per-fragment terms with float atomics in arbitrary order; near-opaque
        # fragments carry 1/max(1-alpha, 1e-8) and cancel, so a few of its own 8.4 M values move between runs
        assert_close(o.grad.reshape(-1).cpu().numpy(), rgo.reshape(-1).cpu().numpy(), rtol=1e-4, atol=1e-9, max_bad=800,
                     what=f"full-size grad_opacities (tile {tile})")
        del f, o, im, al, bw


@pytest.mark.parametrize("tile", [8, 16])
def test_gaussian_deep_tiles_training_and_inference(tile):
    """Gaussian splats on tiles whose lists are cut into several segments: forward, backward and inference
    against the oracle (fast exponentials on the device: looser tolerances)."""
    import inpc_b200
    from inpc_b200.views import look_at_view
    view = look_at_view((0.0, 0.0, 3.0), (0.0, 0.0, 0.0), 64, 48, 60.0, 60.0)
    g = torch.Generator().manual_seed(19)
    n = 30000
    pos = torch.cat([torch.randn((n, 2), generator=g) * 0.15, torch.rand((n, 1), generator=g) - 0.5], dim=1).contiguous()
    feats = (torch.randn((n, 36), generator=g) * 0.5).to(torch.float16)
    opac = torch.rand((n, 1), generator=g) * 0.1 + 0.01
    v = view.to(DEV)
    cam = oracle_camera(view)
    H, W = view.camera.height, view.camera.width
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    rast = inpc_b200.INPCRasterizer(tile_size=tile)
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = rast(v, 1, pos.to(DEV), f, o)
    st = O.rasterize_forward(O.GAUSSIAN, cam, pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
    assert (st.alpha == 1.0).sum() > 20 and (st.ranges[:, 1] - st.ranges[:, 0]).max() > 16 * tile * tile
    assert_close(image.detach().cpu().numpy(), st.image, rtol=1e-4, atol=1e-5, max_bad=4, what="gaussian deep image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, rtol=1e-4, atol=1e-5, max_bad=4, what="gaussian deep alpha")
    assert_close(bw.detach().cpu().numpy(), st.blending_weights, rtol=1e-4, atol=1e-6, max_bad=8, what="gaussian deep blending weights")
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
    assert_close(o.grad.detach().cpu().numpy(), go, rtol=1e-3, atol=1e-8, max_bad=16, what="gaussian deep grad_opacities")
    assert_close(f.grad.float().detach().cpu().numpy(), gf.astype(np.float32), rtol=4e-3, atol=2e-7, max_bad=36 * 16, what="gaussian deep grad_features")
    img, dep, alp = rast.render_preextracted(v, 1, pos.to(DEV), feats.to(DEV), opac.to(DEV), None, sigma_world_scale=1.0, sigma_cutoff=3.0)
    oi, od, oa, _ = O.render_preextracted(1, cam, pos.numpy(), feats.numpy(), opac.numpy(), None, 0.05 / view.camera.focal_y, 3.0, tile=tile)
    assert_close(img.cpu().numpy(), oi, rtol=2e-4, atol=2e-5, max_bad=12, what="gaussian deep inference image")
    assert_close(dep.cpu().numpy(), od, rtol=2e-4, atol=2e-5, max_bad=12, what="gaussian deep inference depth")
    assert_close(alp.cpu().numpy(), oa, rtol=2e-4, atol=2e-5, max_bad=12, what="gaussian deep inference alpha")
