"""CPU-only checks of the oracle itself: hand-computed cases for the projection, tile coverage and
blend rules, the draw rule, both random generators against their published known-answer vectors,
and the analytic backward against torch autograd of an independent float64 transcription."""
import math

import numpy as np
import pytest
import torch

import oracle as O
from helpers import oracle_camera, small_scene
from inpc_b200.views import look_at_view


def axis_camera(w=32, h=32, f=16.0):
    # eye at (0,0,-4) looking down +z, so world x/y map straight to image x/y
    return look_at_view((0.0, 0.0, -4.0), (0.0, 0.0, 0.0), w, h, f, f, up=(0.0, -1.0, 0.0))


def dc_features(n, value=1.0):
    f = np.zeros((n, 36), np.float16)
    f[:, 0:4] = np.float16(value / 0.28209479177387814)
    return f


def world_at_pixel(view, sx, sy, depth=4.0):
    c = view.camera
    return [(sx - c.center_x) / c.focal_x * depth, (sy - c.center_y) / c.focal_y * depth, depth - 4.0]


def test_axis_camera_convention():
    v = axis_camera()
    st = O.preprocess_and_order(O.BILINEAR, O.TRAIN, oracle_camera(v), np.array([world_at_pixel(v, 10.5, 7.5)], np.float32),
                                dc_features(1), np.ones(1, np.float32))
    assert st.n_touched[0] == 1
    assert np.allclose(st.screen[0], [10.5, 7.5], atol=1e-5)
    assert np.isclose(st.depth[0], 4.0)


def test_point_on_pixel_centre_has_unit_weight():
    v = axis_camera()
    pos = np.array([world_at_pixel(v, 10.5, 7.5)], np.float32)
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(v), pos, dc_features(1, 0.8), np.array([0.5], np.float32))
    img, alpha = st.image, st.alpha[0]
    assert np.isclose(alpha[7, 10], 0.5)
    assert np.isclose(img[0, 7, 10], 0.5 * 0.8, rtol=1e-3)
    assert alpha.sum() == pytest.approx(0.5, rel=1e-6)          # no other pixel is touched (distance >= 1 is skipped)
    assert np.isclose(st.blending_weights[0], 0.5)               # bw * w with w = 1


def test_point_on_tile_corner_touches_four_tiles_and_four_pixels():
    v = axis_camera()
    pos = np.array([world_at_pixel(v, 16.0, 8.0)], np.float32)    # corner shared by 4 tiles of 8x8
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(v), pos, dc_features(1), np.array([1.0], np.float32), tile=8)
    assert st.n_touched[0] == 4
    assert list(st.bounds[0]) == [1, 3, 0, 2]
    a = st.alpha[0]
    assert np.allclose([a[7, 15], a[7, 16], a[8, 15], a[8, 16]], 0.25)
    assert a.sum() == pytest.approx(1.0)
    # blending weight carries the bilinear weight twice: 4 * (0.25 * 0.25)
    assert np.isclose(st.blending_weights[0], 0.25)
    # at 16x16 the same point touches two tiles only; the image does not change
    st16 = O.rasterize_forward(O.BILINEAR, oracle_camera(v), pos, dc_features(1), np.array([1.0], np.float32), tile=16)
    assert st16.n_touched[0] == 2
    assert np.array_equal(st16.alpha, st.alpha)


def test_half_integer_offset_excludes_one_side():
    v = axis_camera()
    pos = np.array([world_at_pixel(v, 11.5, 7.5)], np.float32)    # exactly on the centre of pixel 11
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(v), pos, dc_features(1), np.array([1.0], np.float32))
    a = st.alpha[0]
    assert a[7, 11] == pytest.approx(1.0) and a[7, 10] == 0.0 and a[7, 12] == 0.0


def test_culls_near_far_and_offscreen():
    v = axis_camera()
    v.camera.near_plane, v.camera.far_plane = 1.0, 6.0
    pos = np.array([world_at_pixel(v, 10.5, 7.5, 0.5), world_at_pixel(v, 10.5, 7.5, 7.0), world_at_pixel(v, -3.0, 7.5),
                    world_at_pixel(v, 10.5, 40.0), world_at_pixel(v, 10.5, 7.5, 1.0), world_at_pixel(v, 10.5, 7.5, 6.0),
                    world_at_pixel(v, -0.4, 7.5)], np.float32)
    st = O.preprocess_and_order(O.BILINEAR, O.TRAIN, oracle_camera(v), pos, dc_features(len(pos)), np.ones(len(pos), np.float32))
    assert list(st.n_touched[:4]) == [0, 0, 0, 0]
    assert st.n_touched[4] > 0 and st.n_touched[5] > 0             # both depth bounds are inclusive
    assert st.n_touched[6] == 1                                    # still reaches pixel column 0


def test_opaque_stack_terminates_and_saturates_alpha():
    v = axis_camera()
    n = 40
    pos = np.array([world_at_pixel(v, 10.5, 7.5, 2.0 + 0.01 * k) for k in range(n)], np.float32)
    opac = np.full(n, 0.9, np.float32)
    st = O.rasterize_forward(O.BILINEAR, oracle_camera(v), pos, dc_features(n), opac)
    assert st.alpha[0, 7, 10] == 1.0                               # T < 1e-4 clamps alpha to exactly 1
    # T after k points is 0.1^k, so the walk stops after the 4th or 5th point (0.1^4 against 1e-4 in
    # fp32); later points can only leak a rounding-sized weight into a neighbouring pixel
    contributing = int((st.blending_weights > 1e-5).sum())
    assert contributing in (4, 5)
    assert np.all(st.blending_weights[contributing:] < 1e-5)
    # front-to-back order is by depth, not by input order
    st2 = O.rasterize_forward(O.BILINEAR, oracle_camera(v), pos[::-1].copy(), dc_features(n), opac)
    assert np.array_equal(st2.image, st.image)
    assert np.allclose(st2.blending_weights[::-1], st.blending_weights, rtol=1e-6, atol=1e-12)


def test_ordering_is_tile_then_depth_then_index():
    view, pos, feats, opac = small_scene(n=5000)
    for tile in (8, 16):
        st = O.preprocess_and_order(O.BILINEAR, O.TRAIN, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=tile)
        gw = -(-view.camera.width // tile)
        bits = st.depth.view(np.uint32)
        vis = np.flatnonzero(st.n_touched)
        expect = vis[np.lexsort((vis, bits[vis]))]
        assert np.array_equal(st.sorted_points, expect.astype(np.uint32))
        key = st.inst_tile.astype(np.int64) << 32 | bits[st.inst_point]
        assert np.all(np.diff(key) >= 0)
        for t in range(st.ranges.shape[0]):
            r0, r1 = st.ranges[t]
            assert np.all(st.inst_tile[r0:r1] == t)
        assert st.ranges[:, 1].max() == len(st.inst_point)
        # every instance lies inside its point's bounds
        b = st.bounds[st.inst_point].astype(np.int64)
        tx, ty = st.inst_tile % gw, st.inst_tile // gw
        assert np.all((tx >= b[:, 0]) & (tx < b[:, 1]) & (ty >= b[:, 2]) & (ty < b[:, 3]))
        assert st.n_touched.sum() == len(st.inst_point)


def test_image_is_independent_of_tile_size():
    view, pos, feats, opac = small_scene(n=8000)
    a = O.rasterize_forward(O.BILINEAR, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=8)
    b = O.rasterize_forward(O.BILINEAR, oracle_camera(view), pos.numpy(), feats.numpy(), opac.numpy(), tile=16)
    assert np.array_equal(a.image, b.image) and np.array_equal(a.alpha, b.alpha)
    assert np.allclose(a.blending_weights, b.blending_weights, rtol=1e-6, atol=0)


def test_end_bit():
    L = O.lib()
    assert [L.orc_end_bit(x) for x in (0, 1, 2, 3, 255, 256, 15964, 65535, 65536)] == [0, 1, 2, 2, 8, 9, 14, 16, 17]


# ---------------------------------------------------------------------------- draw rule

def test_lower_bound_edge_cases():
    cdf = np.array([0.0, 0.0, 0.25, 0.25, 0.25, 0.75, 1.0], np.float32)
    u = np.array([0.0, 1e-9, 0.25, np.nextafter(np.float32(0.25), np.float32(1)), 0.5, 0.75, 0.9, 1.0], np.float32)
    assert list(O.draw_leaves(cdf, u)) == [0, 2, 2, 5, 5, 5, 6, 6]
    # u above the last entry clamps to the last leaf (a CDF that rounds below 1)
    assert list(O.draw_leaves(np.array([0.2, 0.5, 0.9999], np.float32), np.array([0.99995], np.float32))) == [2]


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    assert O.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert O.philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert O.philox4x32([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_pcg32_known_answers():
    # pcg32 reference demo: seed(42, 54) -> first six outputs
    import ctypes as C
    g = O._Pcg()
    O.lib().orc_pcg_seed(C.byref(g), C.c_uint64(42), C.c_uint64(54))
    out = [int(O.lib().orc_pcg_next_uint(C.byref(g))) for _ in range(6)]
    assert out == [0xa15c02b7, 0x7b47f409, 0xba1d3330, 0x83d2f293, 0xbfa4784b, 0xcbed606e]
    # advance(k) equals k single steps
    a, b = O._Pcg(), O._Pcg()
    for s in (a, b):
        O.lib().orc_pcg_seed(C.byref(s), C.c_uint64(7), C.c_uint64(1))
    for _ in range(1000):
        O.lib().orc_pcg_next_uint(C.byref(a))
    O.lib().orc_pcg_advance(C.byref(b), C.c_uint64(1000))
    assert (a.state, a.inc) == (b.state, b.inc)


def test_training_samples_inside_leaf_and_frustum():
    import synthetic_workloads as syn
    cfg = syn.config0()
    tree, view = cfg["tree"], cfg["view"]
    cam = oracle_camera(view)
    vw = O.viewpoint_weights(cam, tree.centers.numpy(), tree.levels.numpy(), tree.weights.numpy(), tree.initial_size)
    cdf, total = O.build_cdf(vw)
    assert total > 0 and abs(cdf[-1] - 1.0) < 1e-3 and np.all(np.diff(cdf) >= 0)
    pos, idx, exhausted = O.training_samples(cam, 0, 0, cdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, 20000)
    assert exhausted == 0
    half = tree.initial_size / 2.0 ** tree.levels.numpy()[idx] / 2
    assert np.all(np.abs(pos - tree.centers.numpy()[idx]) <= half[:, None] * (1 + 1e-6))
    # every accepted sample projects inside the image and depth range
    w2c = view.w2c.numpy().astype(np.float64)
    pc = pos.astype(np.float64) @ w2c[:3, :3].T + w2c[:3, 3]
    sx = pc[:, 0] / pc[:, 2] * view.camera.focal_x + view.camera.center_x
    sy = pc[:, 1] / pc[:, 2] * view.camera.focal_y + view.camera.center_y
    assert np.all((pc[:, 2] >= view.camera.near_plane) & (sx > -1e-3) & (sx < view.camera.width + 1e-3) & (sy > -1e-3) &
                  (sy < view.camera.height + 1e-3))
    # same stream -> same samples; next call -> different samples
    pos2, idx2, _ = O.training_samples(cam, 0, 0, cdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, 20000)
    pos3, _, _ = O.training_samples(cam, 0, 1, cdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, 20000)
    assert np.array_equal(pos, pos2) and np.array_equal(idx, idx2) and not np.array_equal(pos, pos3)


def test_training_sample_histogram_matches_weights():
    import synthetic_workloads as syn
    tree = syn.uniform_octree(2, seed=4)      # 64 leaves, all well inside the frustum below
    view = look_at_view((0.0, 0.0, 6.0), (0.0, 0.0, 0.0), 256, 256, 500.0, 500.0)
    cam = oracle_camera(view)
    vw = O.viewpoint_weights(cam, tree.centers.numpy(), tree.levels.numpy(), tree.weights.numpy(), tree.initial_size)
    cdf, total = O.build_cdf(vw)
    n = 200000
    _, idx, _ = O.training_samples(cam, 3, 0, cdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, n)
    counts = np.bincount(idx, minlength=64).astype(np.float64)
    expect = vw.astype(np.float64) / vw.astype(np.float64).sum() * n
    chi2 = ((counts - expect) ** 2 / expect).sum()
    assert chi2 < 63 + 6 * math.sqrt(2 * 63)          # 63 dof: mean 63, sd ~11.2


def test_expected_counts_rule():
    vw = np.array([0.0, 1.0, 3.0, 1e-9, 0.0], np.float32)
    counts, total = O.expected_counts(vw, float(vw.sum()), 100)
    assert list(counts) == [0, 25, 75, 1, 0] and total == 101


# ---------------------------------------------------------------------------- backward vs autograd

def _torch_blend(screen, feat, opac, order_per_pixel, W, H):
    """float64 transcription of the blend rule, differentiable; lists are precomputed per pixel."""
    img = torch.zeros((4, H, W), dtype=torch.float64)
    alpha = torch.zeros((H, W), dtype=torch.float64)
    rows_i, rows_a = [], []
    for (px, py), ids in order_per_pixel.items():
        C = torch.zeros(4, dtype=torch.float64)
        T = torch.ones((), dtype=torch.float64)
        for i in ids:
            dx = (screen[i, 0] - (px + 0.5)).abs()
            dy = (screen[i, 1] - (py + 0.5)).abs()
            w = (1 - dx).clamp(0, 1) * (1 - dy).clamp(0, 1)
            a = opac[i] * w
            C = C + T * a * feat[i]
            T = T * (1 - a)
            if T.item() < 1e-4:
                break
        rows_i.append(((px, py), C))
        rows_a.append(((px, py), 1 - T if T.item() >= 1e-4 else torch.ones((), dtype=torch.float64) + 0 * T))
    return rows_i, rows_a


def test_backward_matches_autograd_of_float64_transcription():
    view, pos, feats, opac = small_scene(n=600, width=24, height=20, focal=20.0)
    cam = oracle_camera(view)
    st = O.rasterize_forward(O.BILINEAR, cam, pos.numpy(), feats.numpy(), opac.numpy(), tile=8)
    g = torch.Generator().manual_seed(9)
    H, W = view.camera.height, view.camera.width
    gi = torch.randn((4, H, W), generator=g, dtype=torch.float64)
    ga = torch.randn((1, H, W), generator=g, dtype=torch.float64)
    _, go, gfv = O.rasterize_backward(st, gi.numpy().astype(np.float32), ga.numpy().astype(np.float32))
    # per-pixel lists from the oracle's own ordering
    gw = -(-W // 8)
    lists = {}
    for py in range(H):
        for px in range(W):
            t = (py // 8) * gw + px // 8
            r0, r1 = st.ranges[t]
            ids = [int(i) for i in st.inst_point[r0:r1]
                   if abs(st.screen[i, 0] - (px + 0.5)) < 1 and abs(st.screen[i, 1] - (py + 0.5)) < 1]
            if ids:
                lists[(px, py)] = ids
    screen = torch.tensor(st.screen, dtype=torch.float64)
    feat = torch.tensor(st.feat_view, dtype=torch.float64, requires_grad=True)
    op = torch.tensor(st.opacity, dtype=torch.float64, requires_grad=True)
    rows_i, rows_a = _torch_blend(screen, feat, op, lists, W, H)
    loss = sum((C * gi[:, py, px]).sum() for (px, py), C in rows_i) + sum(A * ga[0, py, px] for (px, py), A in rows_a)
    loss.backward()
    assert np.allclose(gfv, feat.grad.numpy(), rtol=2e-4, atol=2e-5)
    assert np.allclose(go[:, 0], op.grad.numpy(), rtol=2e-4, atol=2e-5)


def test_sh_backward_is_transpose_of_forward():
    view, pos, feats, opac = small_scene(n=50, width=24, height=20, focal=20.0)
    cam = oracle_camera(view)
    st = O.rasterize_forward(O.BILINEAR, cam, pos.numpy(), feats.numpy(), opac.numpy())
    gfv = np.random.default_rng(0).standard_normal((50, 4)).astype(np.float32)
    import ctypes as C
    out = np.zeros((50, 36), np.float16)
    cc = cam.c()
    O.lib().orc_preprocess_backward(C.byref(cc), C.c_int64(50), O._p(st.positions), O._p(st.n_touched), O._p(gfv), O._p(out))
    vis = st.n_touched > 0
    # <SH(f), g> == <f, SH^T(g)> for visible points; zero rows for culled ones
    lhs = (st.feat_view[vis].astype(np.float64) * gfv[vis]).sum()
    rhs = (feats.numpy()[vis].astype(np.float64) * out[vis].astype(np.float64)).sum()
    assert lhs == pytest.approx(rhs, rel=5e-3)
    assert np.all(out[~vis] == 0)


# ---------------------------------------------------------------------------- misc

def test_misc_against_torch_formulas():
    rng = np.random.default_rng(1)
    p = (rng.standard_normal((1000, 3)) * 2).astype(np.float32)
    n2 = np.maximum((p.astype(np.float64) ** 2).sum(1, keepdims=True), 1.0)
    ref = np.clip(p * ((2 * np.sqrt(n2) - 1) / n2 * 0.25) + 0.5, 0, 1)
    assert np.allclose(O.spherical_contraction(p), ref, atol=1e-6)
    a, b = rng.standard_normal(5000).astype(np.float32), rng.standard_normal(5000).astype(np.float32)
    ta = torch.tensor(a, dtype=torch.float64, requires_grad=True)
    loss = torch.log1p(12.5 * (ta - torch.tensor(b, dtype=torch.float64)) ** 2).mean()
    loss.backward()
    assert O.cauchy_loss(a, b) == pytest.approx(loss.item(), rel=1e-5)
    assert np.allclose(O.cauchy_loss_backward(1.0, a, b), ta.grad.numpy(), rtol=1e-4, atol=1e-9)
    # weight decay: ten level bands, zero below 6144
    assert O.weight_decay_factor(0) == 0 and O.weight_decay_factor(6143) == 0
    assert O.weight_decay_factor(6144) == pytest.approx(0.2 / (22528 - 6144))
    assert O.weight_decay_factor(22528) == pytest.approx(0.2 / (153600 - 22528))
    assert O.weight_decay_factor(177362944) == pytest.approx(0.2 / (210917376 - 177362944))
    w = rng.standard_normal(30000).astype(np.float32)
    g0 = rng.standard_normal(30000).astype(np.float32)
    fac = np.array([O.weight_decay_factor(i) for i in range(0, 30000, 997)])
    assert np.allclose(O.weight_decay(w)[::997], fac * w[::997], rtol=1e-6)
    assert np.allclose(O.weight_decay(w, g0)[::997], g0[::997] + fac * w[::997], rtol=1e-5, atol=1e-7)


def test_feature_rows_equal_sh_path_with_dc_only_coefficients():
    """The C/4-pass restatement of the feature-row layout against the four-channel SH restatement:
    rows = 0.2820948 * DC coefficient, every other coefficient zero -> same image, alpha, weights and
    opacity gradient; feature gradient = coefficient gradient / 0.2820948 (the latter rounded to fp16)."""
    rng = np.random.default_rng(11)
    cam = O.Camera(np.eye(4, dtype=np.float32), np.zeros(3, np.float32), 48, 40, 50.0, 50.0, 24.0, 20.0)
    n = 3000
    pos = np.stack([rng.uniform(-1, 1, n), rng.uniform(-1, 1, n), rng.uniform(1.5, 3.0, n)], axis=1).astype(np.float32)
    opac = rng.uniform(0.05, 0.9, (n, 1)).astype(np.float32)
    dc = rng.normal(0, 0.5, (n, 8)).astype(np.float16)
    rows = (np.float32(0.28209479177387814) * dc.astype(np.float32)).astype(np.float32)
    st = O.rasterize_rows_forward(cam, pos, rows, opac, tile=8)
    gi = rng.normal(0, 1e-3, (8, 40, 48)).astype(np.float32)
    ga = rng.normal(0, 1e-3, (1, 40, 48)).astype(np.float32)
    gf, go = O.rasterize_rows_backward(st, gi, ga)
    go_sh = np.zeros((n, 1), np.float64)
    for g in range(2):
        sh = np.zeros((n, 36), np.float16)
        sh[:, :4] = dc[:, 4 * g:4 * g + 4]
        s4 = O.rasterize_forward(O.BILINEAR, cam, pos, sh, opac, tile=8)
        np.testing.assert_allclose(st.image[4 * g:4 * g + 4], s4.image, rtol=1e-6, atol=1e-7)
        np.testing.assert_array_equal(st.alpha, s4.alpha)
        np.testing.assert_array_equal(st.blending_weights, s4.blending_weights)
        gsh, gop, gfv = O.rasterize_backward(s4, gi[4 * g:4 * g + 4], ga if g == 0 else np.zeros_like(ga))
        np.testing.assert_allclose(gf[:, 4 * g:4 * g + 4], gfv, rtol=1e-6, atol=1e-12)
        go_sh += gop
    np.testing.assert_allclose(go, go_sh, rtol=1e-5, atol=1e-10)
