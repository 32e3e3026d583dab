"""GPU tests of the image-composition kernels (background compose, multisample accumulate / resolve)
through the Python mirror and hence the C ABI: bit-exact against outputs of the reference renderer's own
code (tests/golden/renderer_vectors.npz) and against its numpy restatement at a full-size image."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _golden():
    return np.load(Path(__file__).resolve().parent / "golden" / "renderer_vectors.npz")


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def test_multisample_resolve_reproduces_the_reference_renderer():
    from inpc_b200.compose import MultisampleAccumulator
    g = _golden()
    for n in (1, 3, 4):
        for premult in (True, False):
            tag = f"n{n}_{'premultiplied' if premult else 'straight'}"
            acc = MultisampleAccumulator(n, premult)
            for i in range(n):
                acc.add(_t(g[f"sample{i}_image"]), _t(g[f"sample{i}_depth"]), _t(g[f"sample{i}_alpha"]))
            f, d, a, s = acc.resolve(_t(g["background"]))
            np.testing.assert_array_equal(f.cpu().numpy(), g[f"{tag}_feature_image"])
            np.testing.assert_array_equal(d.cpu().numpy(), g[f"{tag}_depth"])
            np.testing.assert_array_equal(a.cpu().numpy(), g[f"{tag}_alpha"])
            np.testing.assert_array_equal(s.cpu().numpy(), g[f"{tag}_alpha_sum"])


def test_compose_background_forward_and_backward():
    from inpc_b200.compose import compose_background
    g = _golden()
    img = _t(g["sample0_image"]).requires_grad_(True)
    alpha = _t(g["sample0_alpha"]).requires_grad_(True)
    bg = _t(g["background"]).requires_grad_(True)
    out = compose_background(img, alpha, bg)
    np.testing.assert_array_equal(out.detach().cpu().numpy(), g["train_feature_image"])
    go = torch.randn(out.shape, generator=torch.Generator().manual_seed(3)).to(DEV)
    out.backward(go)
    i2, a2, b2 = (x.detach().clone().requires_grad_(True) for x in (img, alpha, bg))
    (i2 + (1.0 - a2) * b2).backward(go)
    assert torch.equal(img.grad, i2.grad)
    torch.testing.assert_close(alpha.grad, a2.grad, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(bg.grad, b2.grad, rtol=0, atol=0)


def test_full_size_images_match_restatement():
    from inpc_b200.compose import MultisampleAccumulator, compose_background
    gen = torch.Generator().manual_seed(9)
    C, H, W, n = 4, 822, 1237, 4
    samples = []
    for _ in range(n):
        a = torch.rand((1, H, W), generator=gen)
        a[a < 0.2] = 0.0
        samples.append(((torch.randn((C, H, W), generator=gen) * a).numpy(), (torch.rand((1, H, W), generator=gen) * (a > 0)).numpy(), a.numpy()))
    bg = torch.randn((C, H, W), generator=gen).numpy()
    for premult in (True, False):
        acc = MultisampleAccumulator(n, premult)
        for f, d, a in samples:
            acc.add(_t(f), _t(d), _t(a))
        out = acc.resolve(_t(bg))
        ref = O.multisample_resolve(samples, bg, premult)
        for x, y in zip(out, ref):
            np.testing.assert_array_equal(x.cpu().numpy(), y)
    np.testing.assert_array_equal(compose_background(_t(samples[0][0]), _t(samples[0][2]), _t(bg)).cpu().numpy(),
                                  O.compose_background(samples[0][0], samples[0][2], bg))


def test_compose_argument_errors():
    from inpc_b200.compose import MultisampleAccumulator, compose_background
    img = torch.zeros((4, 8, 8), device=DEV)
    with pytest.raises(ValueError):
        compose_background(img, torch.zeros((1, 4, 4), device=DEV), img)
    with pytest.raises(TypeError):
        compose_background(img.half(), torch.zeros((1, 8, 8), device=DEV), img)
    acc = MultisampleAccumulator(2)
    acc.add(img, torch.zeros((1, 8, 8), device=DEV), torch.zeros((1, 8, 8), device=DEV))
    with pytest.raises(RuntimeError):
        acc.resolve()


def test_ring_buffer_and_multisampled_render():
    """The ring buffer hands out the same sets as the reference class would (start-up rule included), and a
    multisampled render equals rasterising every set and composing with the restatement."""
    import inpc_b200
    from helpers import small_scene
    from inpc_b200.compose import MultisamplingRingBuffer, render_multisampled
    view, pos, feats, _ = small_scene(n=8000, width=96, height=72, focal=90.0)
    v = view.to(DEV)
    gen = torch.Generator().manual_seed(12)
    sets = []
    for k in range(3):
        p = (pos + torch.randn(pos.shape, generator=gen) * 0.01).to(DEV)
        raw = torch.cat([torch.randn((pos.shape[0], 1), generator=gen).to(torch.float16), feats], dim=1).contiguous().to(DEV)
        sets.append((p, raw))
    ring = MultisamplingRingBuffer()
    ring.append(*sets[0], 3)
    got = [ring.get_next() for _ in range(3)]
    assert got[0][0] is sets[0][0] and got[1][0] is sets[0][0] and got[2][0] is sets[0][0]      # unfilled slots yield set 0
    ring.append(*sets[1], 3)
    ring.append(*sets[2], 3)
    assert [ring.get_next()[0] is s[0] for s in sets] == [True, True, True]
    ring.append(*sets[0], 3)                                                                      # wraps around
    rast = inpc_b200.INPCRasterizer()
    bg = torch.randn((4, 72, 96), generator=gen).to(DEV)
    for premult in (True, False):
        ring.read_idx = 0
        f, d, a, s = render_multisampled(rast, v, 0, ring, bg, 1.0, 3.0, premult)
        singles = [tuple(x.cpu().numpy() for x in rast.render(v, 0, p, raw, 1.0, 3.0)) for p, raw in sets]
        rf, rd, ra, rs = O.multisample_resolve(singles, bg.cpu().numpy(), premult)
        np.testing.assert_array_equal(f.cpu().numpy(), rf)
        np.testing.assert_array_equal(d.cpu().numpy(), rd)
        np.testing.assert_array_equal(a.cpu().numpy(), ra)
        np.testing.assert_array_equal(s.cpu().numpy(), rs)
        # rasterising the sets concurrently on several streams changes nothing
        ring.read_idx = 0
        f2, d2, a2, s2 = render_multisampled(rast, v, 0, ring, bg, 1.0, 3.0, premult, n_streams=3)
        assert torch.equal(f2, f) and torch.equal(d2, d) and torch.equal(a2, a) and torch.equal(s2, s)
        # ... and neither does rendering all sets with ONE batched call (one cull / sort / blend sequence for all of them)
        ring.read_idx = 0
        f3, d3, a3, s3 = render_multisampled(rast, v, 0, ring, bg, 1.0, 3.0, premult, batched=True)
        assert torch.equal(f3, f) and torch.equal(d3, d) and torch.equal(a3, a) and torch.equal(s3, s)


def test_batched_multi_set_render_equals_per_set_render():
    """inpc_render_multi against inpc_render, set by set and bit for bit: sets of different sizes (none a multiple of
    the internal alignment, one empty), clustered points whose tile lists span several segments, an image whose
    height is not a multiple of the tile edge, so that the rows of one set's tile grid end inside a tile."""
    import inpc_b200
    from inpc_b200.views import look_at_view
    view = look_at_view((0.3, 0.2, 2.8), (0.0, 0.0, 0.0), 333, 205, 260.0, 250.0).to(DEV)
    gen = torch.Generator().manual_seed(21)
    sizes = [70_001, 0, 33_333, 120_777, 1]
    sets = []
    for n in sizes:
        cluster = torch.randn((n, 3), generator=gen) * torch.tensor([0.05, 0.05, 0.4])
        spread = (torch.rand((n, 3), generator=gen) * 2 - 1) * 1.3
        pos = torch.where(torch.rand((n, 1), generator=gen) < 0.7, cluster, spread).contiguous()
        raw = torch.cat([torch.randn((n, 1), generator=gen) * 2 - 2, torch.randn((n, 36), generator=gen) * 0.5], dim=1).to(torch.float16)
        sets.append((pos.to(DEV), raw.contiguous().to(DEV)))
    rast = inpc_b200.INPCRasterizer(tile_size=8)
    images, depths, alphas = rast.render_multi(view, sets)
    assert images.shape == (len(sizes), 4, 205, 333)
    for j, (pos, raw) in enumerate(sets):
        img, dep, alp = rast.render(view, 0, pos, raw, 1.0, 3.0)
        assert torch.equal(images[j], img) and torch.equal(depths[j], dep) and torch.equal(alphas[j], alp), f"set {j}"
    assert float(alphas[0].max()) == 1.0 and float(alphas[1].abs().max()) == 0.0      # saturated pixels; the empty set is blank
    with pytest.raises(ValueError):
        rast.render_multi(view, sets * 2)                                              # more than 8 sets
    # the composed frame: per set, batched, and batched in two groups on two streams
    from inpc_b200.compose import render_multisampled
    bg = torch.randn((4, 205, 333), generator=gen).to(DEV)
    one_by_one = render_multisampled(rast, view, 0, sets, bg)
    for kw in (dict(batched=True), dict(batched=True, n_streams=2)):
        frame = render_multisampled(rast, view, 0, sets, bg, **kw)
        assert all(torch.equal(x, y) for x, y in zip(frame, one_by_one)), kw
