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
    # gradients are accumulated without floating-point atomics (every (point, part) slot has one writer, the slots are
    # added in fixed order): bit-identical whatever the scheduling
    assert torch.equal(results[1][2][3], results[3][2][3]) and torch.equal(results[1][2][4], results[3][2][4])


def test_gradients_are_bit_identical_from_run_to_run():
    """Two backward passes over the same forward inputs give the same bits: grad_features and grad_opacities of the
    bilinear 8x8 path are sums over per-point slots in fixed order, not over atomics in arrival order (the reference
    adds five float atomics per fragment, bilinear/kernels.cu:392-415, and is not reproducible)."""
    import inpc_b200
    import synthetic_workloads as syn
    cfg = syn.config1(n_samples=1 << 21, n_leaves=1 << 16)
    view, tree = cfg["view"].to(DEV), cfg["tree"].to(DEV)
    feats, opac = cfg["features"].to(DEV), cfg["opacities"].to(DEV)
    pos, _ = inpc_b200.ProbabilityFieldSampler(0).generate_training_samples(tree.centers, tree.levels, tree.weights, view, 1 << 21,
                                                                             tree.initial_size)
    H, W = view.camera.height, view.camera.width
    g = torch.Generator().manual_seed(5)
    gi = (torch.randn((4, H, W), generator=g) * 1e-3).to(DEV)
    ga = (torch.randn((1, H, W), generator=g) * 1e-3).to(DEV)
    grads = []
    for _ in range(3):
        f = feats.detach().requires_grad_(True)
        o = opac.detach().requires_grad_(True)
        im, al, _ = inpc_b200.INPCRasterizer(tile_size=8)(view, 0, pos, f, o)
        torch.autograd.backward([im, al], [gi, ga])
        grads.append((f.grad.clone(), o.grad.clone()))
    assert float(grads[0][1].abs().sum()) > 0
    for gf, go in grads[1:]:
        assert torch.equal(gf, grads[0][0]) and torch.equal(go, grads[0][1])


def test_inputs_from_host_memory_give_the_same_batch():
    """run_batch with an `inputs` callback that copies every view's camera and upstream gradients from pinned host
    memory on a stream of its own -- the forward waiting for the camera, only the backward for the gradients -- gives
    what the device-resident call gives."""
    import synthetic_workloads as syn
    from inpc_b200.batch import ViewShardedTrainer
    from inpc_b200.views import View
    tree = syn.adaptive_octree(4096, seed=1, min_level=3, max_level=6).to(DEV)
    n = 1 << 16
    feats = syn.sh_features(n, 12, "normal", 0.5).to(DEV)
    opac = syn.opacities_sigmoid(n, 13).to(DEV)
    host_views = syn.orbit_views(5, seed=2, width=256, height=160, focal=200.0)
    views = [v.to(DEV) for v in host_views]
    g = torch.Generator().manual_seed(5)
    gi_host = (torch.randn((4, 160, 256), generator=g) * 1e-3).pin_memory()
    ga_host = (torch.randn((1, 160, 256), generator=g) * 1e-3).pin_memory()
    pinned = [(v.w2c.pin_memory(), v.position.pin_memory()) for v in host_views]
    copy_stream = torch.cuda.Stream(device=DEV)

    def inputs(vi, stream):
        with torch.cuda.stream(copy_stream):
            w2c, cpos = (t.to(DEV, non_blocking=True) for t in pinned[vi])
            camera_copied = torch.cuda.Event()
            camera_copied.record(copy_stream)
            gi, ga = gi_host.to(DEV, non_blocking=True), ga_host.to(DEV, non_blocking=True)
            grads_copied = torch.cuda.Event()
            grads_copied.record(copy_stream)
        stream.wait_event(camera_copied)
        for t in (w2c, cpos, gi, ga):
            t.record_stream(stream)
        return View(host_views[vi].camera, w2c, cpos), gi, ga, grads_copied

    results = []
    for use_callback in (False, True):
        tr = ViewShardedTrainer(tree, feats, opac, n, seed=0, n_appearance=1 << 12, n_streams=2)
        if use_callback:
            copy_stream.wait_stream(torch.cuda.current_stream())
            out = tr.run_batch(views, None, inputs=inputs)
        else:
            out = tr.run_batch(views, (gi_host.to(DEV), ga_host.to(DEV)))
        torch.cuda.synchronize()
        results.append((tr.buffers.appearance.clone(), tr.buffers.leaf.max_sampled.clone(), [o.clone() for o in out]))
    assert torch.equal(results[0][0], results[1][0]) and float(results[0][0].abs().sum()) > 0
    torch.testing.assert_close(results[0][1], results[1][1], rtol=1e-5, atol=1e-8)
    image_a, alpha_a, weights_a, gf_a, go_a = results[0][2]
    image_b, alpha_b, weights_b, gf_b, go_b = results[1][2]
    assert torch.equal(image_a, image_b) and torch.equal(alpha_a, alpha_b)
    assert torch.equal(gf_a, gf_b) and torch.equal(go_a, go_b)
    torch.testing.assert_close(weights_a, weights_b, rtol=1e-5, atol=1e-8)
