"""GPU test of the view-sharded batch driver: pipelining a shard's views over several CUDA streams
changes nothing but the order in which the appearance partial sums are added."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_stream_pipelined_batch_equals_sequential_batch():
    import synthetic_workloads as syn
    from inpc_b200.batch import ViewShardedTrainer
    tree = syn.adaptive_octree(4096, seed=1, min_level=3, max_level=6).to(DEV)
    n = 1 << 17
    feats = syn.sh_features(n, 12, "normal", 0.5).to(DEV)
    opac = syn.opacities_sigmoid(n, 13).to(DEV)
    views = [v.to(DEV) for v in syn.orbit_views(7, seed=2, width=320, height=208, focal=250.0)]
    g = torch.Generator().manual_seed(5)
    gi = (torch.randn((4, 208, 320), generator=g) * 1e-3).to(DEV)
    ga = (torch.randn((1, 208, 320), generator=g) * 1e-3).to(DEV)
    results = {}
    for n_streams in (1, 3):
        tr = ViewShardedTrainer(tree, feats, opac, n, seed=0, n_appearance=1 << 12, n_streams=n_streams)
        for _ in range(2):                                        # twice: the second batch reuses streams and partial buffers
            out = tr.run_batch(views, (gi, ga))
        torch.cuda.synchronize()
        results[n_streams] = ((tr.buffers.leaf.max_sampled.clone(), tr.buffers.leaf.min_sampled.clone()), tr.buffers.appearance.clone(),
                              [o.clone() for o in out])
    # A point's blending weight is summed with one atomic per tile it touches, in either order, so the
    # statistics (maxima / minima of those weights) agree to rounding, not bit for bit - between two
    # sequential runs just as between a sequential and a pipelined one.
    torch.testing.assert_close(results[1][0][0], results[3][0][0], rtol=1e-5, atol=1e-8)
    torch.testing.assert_close(results[1][0][1], results[3][0][1], rtol=1e-5, atol=1e-8)
    torch.testing.assert_close(results[1][1], results[3][1], rtol=1e-4, atol=1e-8)
    for a, b in zip(results[1][2][:2], results[3][2][:2]):        # last view's image and alpha
        assert torch.equal(a, b)
