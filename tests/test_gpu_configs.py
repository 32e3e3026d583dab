"""The tiny plumbing configuration end to end on the GPU (4096 leaves at level 4, 2^16 draws with seed 0,
256x256, f = 300, 16x16 tiles, forward blend; compare feature image and alpha): sampling bit-exact
against the CPU oracle, then both feature layouts rasterised from the sampled points."""
import numpy as np
import pytest
import torch

import oracle as O
from helpers import assert_close, oracle_camera

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_config0_sample_then_blend_matches_oracle():
    import inpc_b200
    import synthetic_workloads as syn
    cfg = syn.config0()
    tree, view, n = cfg["tree"], cfg["view"], cfg["n_samples"]
    cam = oracle_camera(view)
    sampler = inpc_b200.ProbabilityFieldSampler(0)
    t = tree.to(DEV)
    pos, idx = sampler.generate_training_samples(t.centers, t.levels, t.weights, view.to(DEV), n, t.initial_size)
    vw = O.viewpoint_weights(cam, tree.centers.numpy(), tree.levels.numpy(), tree.weights.numpy(), tree.initial_size)
    cdf, _ = O.build_cdf(vw)
    opos, oidx, _ = O.training_samples(cam, 0, 0, cdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, n)
    assert np.array_equal(pos.cpu().numpy(), opos) and np.array_equal(idx.cpu().numpy(), oidx)
    rast = inpc_b200.INPCRasterizer(tile_size=16)
    # reference layout: 36 SH halves -> 4 channels
    image, alpha, bw = rast(view.to(DEV), 0, pos, cfg["features"].to(DEV), cfg["opacities"].to(DEV))
    st = O.rasterize_forward(O.BILINEAR, cam, opos, cfg["features"].numpy(), cfg["opacities"].numpy(), tile=16)
    assert_close(image.cpu().numpy(), st.image, what="config 0 image")
    assert_close(alpha.cpu().numpy(), st.alpha, what="config 0 alpha")
    # the configuration's own layout: 16 fp32 channels ~ U(0,1)
    rows = torch.rand((n, 16), generator=torch.Generator().manual_seed(10))
    image, alpha, bw = rast.forward_rows(view.to(DEV), pos, rows.to(DEV), cfg["opacities"].to(DEV))
    st = O.rasterize_rows_forward(cam, opos, rows.numpy(), cfg["opacities"].numpy(), tile=16)
    assert image.shape == (16, 256, 256)
    assert_close(image.cpu().numpy(), st.image, what="config 0 image, 16 channels")
    assert_close(alpha.cpu().numpy(), st.alpha, what="config 0 alpha, 16 channels")
    assert_close(bw.cpu().numpy(), st.blending_weights, what="config 0 blending weights, 16 channels")


def _integer_stages_match(R, state, blobs, settings, st):
    """Sorted point order, per-tile lists and tile ranges of a forward against the oracle's, bit for bit."""
    dbg = R.debug_arrays(state, settings, blobs.point, blobs.instance)
    assert int(state.n_visible) == len(st.sorted_points) and int(state.n_instances) == len(st.inst_point)
    assert np.array_equal(dbg["sorted_points"].cpu().numpy().view(np.uint32), st.sorted_points)
    assert np.array_equal(dbg["inst_point"].cpu().numpy().view(np.uint32), st.inst_point)
    assert np.array_equal(dbg["ranges"].cpu().numpy().view(np.uint32), st.ranges)
    assert np.array_equal(dbg["bounds"].cpu().numpy().view(np.uint16), st.bounds)
    assert np.array_equal(dbg["depth"].cpu().numpy().view(np.uint32), st.depth.view(np.uint32))


def test_config2_resolution_inference_matches_oracle_and_reference():
    """Configuration 2 at its own resolution (1920x1080, f = 1400, eye (0, 0.5, 3), Gaussian-mixture cloud,
    render_preextracted) with the point count cut to what the CPU restatement does in seconds: integer stages
    bit-exact, image / depth / alpha within 1e-5 relative + 1e-6 absolute of the oracle, and the same against
    the reference's own backend when it has been built."""
    import inpc_b200
    from inpc_b200 import rasterization as R
    import synthetic_workloads as syn
    c = syn.config2(n_points=400_000)
    view, pos, feats, opac = c["view"], c["positions"], c["features"], c["opacities"]
    assert (view.camera.width, view.camera.height) == (1920, 1080)
    cam = oracle_camera(view)
    v = view.to(DEV)
    settings = R.INPCRasterizer.extract_settings(v, 0)
    _, _, _, state, blobs, _ = R.forward_with_state(pos.to(DEV), feats.to(DEV), opac.to(DEV), settings, 8)
    st = O.preprocess_and_order(O.BILINEAR, O.TRAIN, cam, pos.numpy(), feats.numpy(), opac.numpy(), tile=8)
    _integer_stages_match(R, state, blobs, settings, st)
    rast = inpc_b200.INPCRasterizer(tile_size=8)
    img, dep, alp = rast.render_preextracted(v, 0, pos.to(DEV), feats.to(DEV), opac.to(DEV))
    oi, od, oa, _ = O.render_preextracted(0, cam, pos.numpy(), feats.numpy(), opac.numpy(), None, 0.05 / view.camera.focal_y, 3.0, tile=8)
    assert_close(img.cpu().numpy(), oi, what="config 2 image")
    assert_close(alp.cpu().numpy(), oa, what="config 2 alpha")
    assert_close(dep.cpu().numpy(), od, rtol=1e-5, atol=1e-5, what="config 2 depth")
    try:
        import ref_backend as RB
        have_ref = RB.available()
    except Exception:
        have_ref = False
    if have_ref:
        # the reference orders equal depths by an atomic race: silence all but the first point of every tie
        dbg = R.debug_arrays(state, settings, blobs.point, blobs.instance)
        from helpers import silence_depth_ties
        opac_s = silence_depth_ties(dbg["depth"].cpu().numpy(), dbg["n_touched"].cpu().numpy() > 0, opac.to(DEV))
        ri, rd, ra = RB.render_preextracted(v, 0, pos.to(DEV), feats.to(DEV), opac_s.reshape(-1).contiguous(), None, 1.0, 3.0)
        img, dep, alp = rast.render_preextracted(v, 0, pos.to(DEV), feats.to(DEV), opac_s)
        assert_close(img.cpu().numpy(), ri.cpu().numpy(), what="config 2 image vs reference")
        assert_close(alp.cpu().numpy(), ra.cpu().numpy(), what="config 2 alpha vs reference")
        assert_close(dep.cpu().numpy(), rd.cpu().numpy(), rtol=1e-5, atol=1e-5, what="config 2 depth vs reference")


def test_config4_resolution_both_layouts_match_oracle():
    """Configuration 4 at its own resolution: 3840x2160, f = 2800, i.e. 129,600 tiles of 8x8 pixels and 17 tile
    bits -- the case in which the reference's 16-bit tile key overflows (bilinear/kernels.cu:214), so the oracle is
    the only yardstick.  Skewed cloud (90 % in one tight cluster: deep per-pixel lists, lists of many segments), point
    count cut to what the CPU restatement does in seconds.  Forward and backward in the reference's layout (36 SH
    halves -> 4 channels) and in the configuration's own (32 fp32 channels): integer stages bit-exact, floats
    within 1e-5 relative + 1e-6 absolute (fp16 feature gradients: half precision)."""
    import inpc_b200
    from inpc_b200 import rasterization as R
    import synthetic_workloads as syn
    from helpers import RTOL_H, ATOL_H
    c = syn.config4(n_points=1_500_000)
    view, pos, feats, opac = c["view"], c["positions"], c["features"], c["opacities"]
    H, W = view.camera.height, view.camera.width
    assert (W, H) == (3840, 2160) and (-(-W // 8)) * (-(-H // 8)) == 129_600
    cam = oracle_camera(view)
    v = view.to(DEV)
    settings = R.INPCRasterizer.extract_settings(v, 0)
    g = torch.Generator().manual_seed(44)
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    _, _, _, state, blobs, _ = R.forward_with_state(pos.to(DEV), feats.to(DEV), opac.to(DEV), settings, 8)
    st = O.rasterize_forward(O.BILINEAR, cam, pos.numpy(), feats.numpy(), opac.numpy(), tile=8)
    lens = st.ranges[:, 1].astype(np.int64) - st.ranges[:, 0]
    assert lens.max() > 4096 and int(np.nonzero(lens)[0].max()) >= 1 << 16   # several segments; tiles beyond 16 bits in use
    _integer_stages_match(R, state, blobs, settings, st)
    del blobs
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=8)(v, 0, pos.to(DEV), f, o)
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    assert_close(image.detach().cpu().numpy(), st.image, what="config 4 image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, what="config 4 alpha")
    assert_close(bw.cpu().numpy(), st.blending_weights, what="config 4 blending weights")
    gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
    assert_close(o.grad.cpu().numpy(), go, rtol=1e-4, atol=1e-9, max_bad=8, what="config 4 grad_opacities")
    assert_close(f.grad.float().cpu().numpy(), gf.astype(np.float32), rtol=RTOL_H, atol=ATOL_H, max_bad=36, what="config 4 grad_features")
    del f, o, image, alpha, bw
    # the configuration's own layout: 32 fp32 channels ~ N(0, 0.5)
    rows = torch.randn((pos.shape[0], 32), generator=g) * 0.5
    gi32 = torch.randn((32, H, W), generator=g) * 1e-3
    f = rows.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=8).forward_rows(v, pos.to(DEV), f, o)
    torch.autograd.backward([image, alpha], [gi32.to(DEV), ga.to(DEV)])
    sr = O.rasterize_rows_forward(cam, pos.numpy(), rows.numpy(), opac.numpy(), tile=8)
    assert_close(image.detach().cpu().numpy(), sr.image, what="config 4 image, 32 channels")
    assert_close(alpha.detach().cpu().numpy(), sr.alpha, what="config 4 alpha, 32 channels")
    assert_close(bw.cpu().numpy(), sr.blending_weights, what="config 4 blending weights, 32 channels")
    grows, go = O.rasterize_rows_backward(sr, gi32.numpy(), ga.numpy())
    # opacities ~ sigmoid(N(2,1)) make 1 / (1 - alpha) large; the row kernels sum <g, C_run - C_final> over the 32
    # channels first and scale once, the restatement scales per group of four channels and adds the groups: two
    # roundings of the same cancelling sum, hence an absolute floor of 1e-7 (values are ~1e-4) instead of 1e-9
    assert_close(o.grad.cpu().numpy(), go, rtol=1e-4, atol=1e-7, max_bad=8, what="config 4 grad_opacities, 32 channels")
    assert_close(f.grad.cpu().numpy(), grows, rtol=1e-4, atol=1e-9, max_bad=32, what="config 4 grad_features, 32 channels")


def test_bench_workload_unsilenced_matches_oracle():
    """The scene the benchmark times -- 2^23 samples of the 2^18-leaf octree, 1237x822, a third of the samples sharing
    their depth's bit pattern with another one, nothing silenced -- forward and backward against the CPU restatement
    (which breaks depth ties by point id exactly like the library): the heavy blend that is timed is the one checked."""
    import inpc_b200
    from inpc_b200 import sampling as S
    import synthetic_workloads as syn
    from helpers import RTOL_H, ATOL_H
    cfg = syn.config1()
    view, tree = cfg["view"], cfg["tree"].to(DEV)
    feats, opac = cfg["features"], cfg["opacities"]
    n = cfg["n_samples"]
    v = view.to(DEV)
    pos, _ = S.ProbabilityFieldSampler(0).generate_training_samples(tree.centers, tree.levels, tree.weights, v, n, tree.initial_size)
    H, W = view.camera.height, view.camera.width
    g = torch.Generator().manual_seed(5)
    gi = torch.randn((4, H, W), generator=g) * 1e-3
    ga = torch.randn((1, H, W), generator=g) * 1e-3
    f = feats.to(DEV).requires_grad_(True)
    o = opac.to(DEV).requires_grad_(True)
    image, alpha, bw = inpc_b200.INPCRasterizer(tile_size=8)(v, 0, pos, f, o)
    torch.autograd.backward([image, alpha], [gi.to(DEV), ga.to(DEV)])
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(view), pos.cpu().numpy(), feats.numpy(), opac.numpy(), tile=8)
    depth_bits = st.depth.view(np.uint32)[st.n_touched > 0]
    assert len(np.unique(depth_bits)) < 0.9 * len(depth_bits)          # the ties are there
    assert (st.alpha == 1.0).sum() > 10_000                            # and so are the saturated pixels
    assert_close(image.detach().cpu().numpy(), st.image, what="bench scene image")
    assert_close(alpha.detach().cpu().numpy(), st.alpha, what="bench scene alpha")
    assert_close(bw.cpu().numpy(), st.blending_weights, what="bench scene blending weights")
    gf, go, _ = O.rasterize_backward(st, gi.numpy(), ga.numpy())
    # near-opaque fragments carry 1/max(1-alpha, 1e-8) and cancel: a handful of the 8.4 M values differ by summation order
    assert_close(o.grad.reshape(-1).cpu().numpy(), go.reshape(-1), rtol=1e-4, atol=1e-9, max_bad=100, what="bench scene grad_opacities")
    assert_close(f.grad.float().cpu().numpy(), gf.astype(np.float32), rtol=RTOL_H, atol=ATOL_H, max_bad=36, what="bench scene grad_features")
