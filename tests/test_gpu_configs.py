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
    from inpc_b200 import synthetic as syn
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
