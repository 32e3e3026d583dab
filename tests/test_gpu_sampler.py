"""GPU parity tests of the probability-field sampler through the Python mirror / C ABI.

Against the CPU oracle the whole chain is bit-exact by construction (explicit fused arithmetic,
integer CDF, counter-based Philox): viewpoint weights, CDF, drawn leaves and positions.  Against the
reference backend the comparison is what its design allows: weights within rounding, the draw rule
bit-exact on the reference's own CDF and uniform stream, and the same distribution."""
import math

import numpy as np
import pytest
import torch

import oracle as O
import ref_backend as RB
from helpers import assert_close, oracle_camera

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
needs_ref = pytest.mark.skipif(not RB.available(), reason="oracle/_ref/libinpc_ref.so not built")


def _scene(adaptive=True):
    import synthetic_workloads as syn
    tree = syn.adaptive_octree(20000, seed=7, min_level=3, max_level=7) if adaptive else syn.uniform_octree(4, seed=0)
    view = syn.orbit_view(0.8, -0.3, 2.2, 200, 150, 170.0)      # close enough that part of the tree is outside
    return tree, view


def _np(tree):
    return tree.centers.numpy(), tree.levels.numpy(), tree.weights.numpy()


def test_viewpoint_weights_and_cdf_bit_exact_vs_oracle():
    import inpc_b200
    from inpc_b200 import sampling as S
    tree, view = _scene()
    t, v = tree.to(DEV), view.to(DEV)
    vw = inpc_b200.compute_viewpoint_weights(t.centers, t.levels, t.weights, v, tree.initial_size)
    ovw = O.viewpoint_weights(oracle_camera(view), *_np(tree), tree.initial_size)
    assert 0 < (ovw == 0).sum() < len(ovw)                       # some leaves are outside the frustum
    assert np.array_equal(vw.detach().cpu().numpy().view(np.uint32), ovw.view(np.uint32))
    cdf, total = S.build_cdf(vw)
    ocdf, ototal = O.build_cdf(ovw)
    assert np.array_equal(cdf.detach().cpu().numpy().view(np.uint32), ocdf.view(np.uint32))
    assert total.item() == ototal
    assert np.all(np.diff(ocdf) >= 0) and ocdf[-1] == 1.0
    assert total.item() == pytest.approx(float(ovw.astype(np.float64).sum()), rel=1e-6)


def test_training_samples_bit_exact_vs_oracle_and_resumable():
    import inpc_b200
    tree, view = _scene()
    t, v = tree.to(DEV), view.to(DEV)
    cam = oracle_camera(view)
    ovw = O.viewpoint_weights(cam, *_np(tree), tree.initial_size)
    ocdf, _ = O.build_cdf(ovw)
    n = 50000
    s = inpc_b200.ProbabilityFieldSampler(1234)
    for call in range(2):
        pos, idx = s.generate_training_samples(t.centers, t.levels, t.weights, v, n, tree.initial_size)
        opos, oidx, exhausted = O.training_samples(cam, 1234, call, ocdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, n)
        assert exhausted == 0
        assert idx.dtype == torch.int64 and pos.shape == (n, 3)
        assert np.array_equal(idx.detach().cpu().numpy(), oidx)
        assert np.array_equal(pos.detach().cpu().numpy().view(np.uint32), opos.view(np.uint32))
    # checkpoint / resume: restoring the counter replays the same call
    assert s.get_rng_state() == 2
    state = s.state_dict()
    s2 = inpc_b200.ProbabilityFieldSampler(1234)
    s2.load_state_dict(state)
    a = s.generate_training_samples(t.centers, t.levels, t.weights, v, 1000, tree.initial_size)
    b = s2.generate_training_samples(t.centers, t.levels, t.weights, v, 1000, tree.initial_size)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_generate_samples_and_expected_samples_vs_oracle():
    import inpc_b200
    tree, view = _scene()
    t, v = tree.to(DEV), view.to(DEV)
    cam = oracle_camera(view)
    ovw = O.viewpoint_weights(cam, *_np(tree), tree.initial_size)
    ocdf, ototal = O.build_cdf(ovw)
    s = inpc_b200.ProbabilityFieldSampler(99)
    pos = s.generate_samples(t.centers, t.levels, t.weights, v, 30000, tree.initial_size)
    opos, _ = O.samples(99, 0, ocdf, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, 30000)
    assert np.array_equal(pos.detach().cpu().numpy().view(np.uint32), opos.view(np.uint32))
    exp = s.generate_expected_samples(t.centers, t.levels, t.weights, v, 40000, 3, tree.initial_size)
    counts, n_created = O.expected_counts(ovw, ototal, 40000)
    assert exp.shape == (n_created * 3, 3)
    oexp = O.expected_samples(99, 1, counts, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, 3)
    assert np.array_equal(exp.detach().cpu().numpy().view(np.uint32), oexp.view(np.uint32))


def test_zero_weight_sum_behaviour():
    import inpc_b200
    tree, view = _scene(adaptive=False)
    t, v = tree.to(DEV), view.to(DEV)
    zero = torch.zeros_like(t.weights)
    s = inpc_b200.ProbabilityFieldSampler(0)
    pos, idx = s.generate_training_samples(t.centers, t.levels, zero, v, 1000, tree.initial_size)
    assert torch.all(pos == 0) and torch.all(idx == -1)          # sampling.cu:107-111
    assert s.generate_samples(t.centers, t.levels, zero, v, 1000, tree.initial_size).shape == (0, 3)
    assert s.generate_expected_samples(t.centers, t.levels, zero, v, 1000, 2, tree.initial_size).shape == (0, 3)
    with pytest.raises(TypeError):
        s.generate_samples(t.centers, t.levels.long(), t.weights, v, 10, tree.initial_size)
    with pytest.raises(NotImplementedError):
        v.camera.distortion = object()
        s.generate_samples(t.centers, t.levels, t.weights, v, 10, tree.initial_size)


def test_draw_leaves_edge_cases_on_device():
    from inpc_b200 import sampling as S
    cdf = torch.tensor([0.0, 0.0, 0.25, 0.25, 0.25, 0.75, 1.0], device=DEV)
    u = torch.tensor([0.0, 1e-9, 0.25, float(np.nextafter(np.float32(0.25), np.float32(1))), 0.5, 0.75, 0.9, 1.0], device=DEV)
    assert S.draw_leaves(cdf, u).tolist() == [0, 2, 2, 5, 5, 5, 6, 6]
    g = torch.Generator().manual_seed(2)
    big = torch.cumsum(torch.rand(100_000, generator=g), 0)
    big = (big / big[-1]).float()
    uu = torch.rand(200_000, generator=g)
    assert np.array_equal(S.draw_leaves(big.to(DEV), uu.to(DEV)).detach().cpu().numpy(), O.draw_leaves(big.numpy(), uu.numpy()))


@needs_ref
def test_viewpoint_weights_vs_reference_backend():
    import inpc_b200
    tree, view = _scene()
    t, v = tree.to(DEV), view.to(DEV)
    vw = inpc_b200.compute_viewpoint_weights(t.centers, t.levels, t.weights, v, tree.initial_size)
    rvw = RB.viewpoint_weights(v, t.centers, t.levels, t.weights, tree.initial_size)
    # a leaf whose only visible corner lies within rounding of the frustum may flip; none should here
    assert_close(vw.detach().cpu().numpy(), rvw.detach().cpu().numpy(), rtol=2e-6, atol=0, max_bad=2, what="viewpoint weights vs reference")


@needs_ref
def test_draw_rule_bit_exact_on_reference_cdf_and_stream():
    """Feeds the reference's own CDF and its PCG32 uniform stream to the device look-up: the drawn
    leaves reproduce the reference's sample positions exactly (sampling_kernels.cu:128-150)."""
    from inpc_b200 import sampling as S
    tree, view = _scene()
    t, v = tree.to(DEV), view.to(DEV)
    n = 40000
    RB.sampler_seed(2024)
    rpos, rcdf = RB.samples(v, t.centers, t.levels, t.weights, n, tree.initial_size)
    assert rpos.shape == (n, 3)
    pcg = O.RefPcg(2024)
    cdf_host = rcdf.detach().cpu().numpy()
    for fused in (True, False):
        opos, u, oleaf = O.RefPcg(2024).create_samples(cdf_host, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, n, fused)
        if np.array_equal(opos.view(np.uint32), rpos.detach().cpu().numpy().view(np.uint32)):
            break
    else:
        raise AssertionError("oracle restatement of create_samples_cu does not reproduce the reference positions")
    leaves = S.draw_leaves(rcdf, torch.from_numpy(u).to(DEV))
    assert np.array_equal(leaves.detach().cpu().numpy(), oleaf)
    # the host generator advanced by 4n: a second call continues the stream
    rpos2, _ = RB.samples(v, t.centers, t.levels, t.weights, 1000, tree.initial_size)
    pcg2 = O.RefPcg(2024)
    pcg2.create_samples(cdf_host, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, n, fused)
    opos2, _, _ = pcg2.create_samples(cdf_host, tree.centers.numpy(), tree.levels.numpy(), tree.initial_size, 1000, fused)
    assert np.array_equal(opos2.view(np.uint32), rpos2.detach().cpu().numpy().view(np.uint32))


@needs_ref
def test_training_sample_distribution_matches_reference():
    """The reference's rejection sampler is race-ordered (atomic ticket), so only distributions can be
    compared: per-leaf histograms of both samplers against the expected conditional probabilities."""
    import inpc_b200
    import synthetic_workloads as syn
    tree = syn.uniform_octree(2, seed=4)
    view = syn.orbit_view(0.3, 0.2, 3.0, 256, 256, 300.0)
    t, v = tree.to(DEV), view.to(DEV)
    n = 400000
    pos, idx = inpc_b200.ProbabilityFieldSampler(5).generate_training_samples(t.centers, t.levels, t.weights, v, n, tree.initial_size)
    RB.sampler_seed(5)
    rpos, ridx, _ = RB.training_samples(v, t.centers, t.levels, t.weights, n, tree.initial_size)
    mine = np.bincount(idx.detach().cpu().numpy(), minlength=64).astype(np.float64)
    ref = np.bincount(ridx.detach().cpu().numpy(), minlength=64).astype(np.float64)
    # two-sample chi-square over the 64 leaves
    chi2 = ((mine - ref) ** 2 / np.maximum(mine + ref, 1)).sum()
    assert chi2 < 63 + 6 * math.sqrt(2 * 63)
    for p, i in ((pos, idx), (rpos, ridx)):
        half = tree.initial_size / 2.0 ** tree.levels.numpy()[i.detach().cpu().numpy()] / 2
        assert np.all(np.abs(p.detach().cpu().numpy() - tree.centers.numpy()[i.detach().cpu().numpy()]) <= half[:, None] * (1 + 1e-6))


def test_full_size_sampler_properties():
    """2^18 leaves, 2^23 samples: every sample inside its leaf and inside the frustum, deterministic."""
    import inpc_b200
    import synthetic_workloads as syn
    cfg = syn.config1(n_samples=8)                                # attributes are not needed here
    t, v = cfg["tree"].to(DEV), cfg["view"].to(DEV)
    n = 1 << 23
    s = inpc_b200.ProbabilityFieldSampler(0)
    pos, idx = s.generate_training_samples(t.centers, t.levels, t.weights, v, n, t.initial_size)
    assert int(idx.min()) >= 0 and int(idx.max()) < t.centers.shape[0]
    half = (t.initial_size / torch.pow(2.0, t.levels[idx].float()) / 2)[:, None]
    assert bool(((pos - t.centers[idx]).abs() <= half * (1 + 1e-6)).all())
    pc = pos @ v.w2c[:3, :3].T + v.w2c[:3, 3]
    c = v.camera
    sx = pc[:, 0] / pc[:, 2] * c.focal_x + c.center_x
    sy = pc[:, 1] / pc[:, 2] * c.focal_y + c.center_y
    ok = (pc[:, 2] >= c.near_plane) & (sx > -1e-2) & (sx < c.width + 1e-2) & (sy > -1e-2) & (sy < c.height + 1e-2)
    assert bool(ok.all())
    s.set_rng_state(0)
    pos2, idx2 = s.generate_training_samples(t.centers, t.levels, t.weights, v, n, t.initial_size)
    assert torch.equal(pos, pos2) and torch.equal(idx, idx2)
