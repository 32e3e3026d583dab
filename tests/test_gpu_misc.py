"""GPU parity tests of the fused misc ops (weight decay, contraction, Cauchy loss) against the CPU
oracle and, where built, the reference backend."""
import numpy as np
import pytest
import torch

import oracle as O
import ref_backend as RB
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
needs_ref = pytest.mark.skipif(not RB.available(), reason="oracle/_ref/libinpc_ref.so not built")


def test_spherical_contraction():
    import inpc_b200
    g = torch.Generator().manual_seed(1)
    p = torch.randn((100_003, 3), generator=g) * 2
    out = inpc_b200.spherical_contraction(p.to(DEV))
    assert_close(out.detach().cpu().numpy(), O.spherical_contraction(p.numpy()), rtol=1e-6, atol=1e-7, what="contraction vs oracle")
    assert inpc_b200.spherical_contraction(torch.empty((0, 3), device=DEV)).shape == (0, 3)
    if RB.available():
        assert torch.equal(out, RB.contraction(p.to(DEV)))


def test_cauchy_loss_forward_backward():
    import inpc_b200
    g = torch.Generator().manual_seed(2)
    a = torch.randn((3, 301, 211), generator=g)
    b = torch.randn((3, 301, 211), generator=g)
    x = a.to(DEV).requires_grad_(True)
    loss = inpc_b200.fused_cauchy_loss(x, b.to(DEV))
    (loss * 3.0).backward()
    assert loss.shape == () and loss.item() == pytest.approx(O.cauchy_loss(a.numpy(), b.numpy()), rel=2e-6)
    assert_close(x.grad.detach().cpu().numpy(), O.cauchy_loss_backward(3.0, a.numpy(), b.numpy()), rtol=1e-5, atol=1e-12, what="cauchy grad")
    with pytest.raises(ValueError):
        inpc_b200.fused_cauchy_loss(x, b[:2].to(DEV))
    if RB.available():
        assert loss.item() == pytest.approx(RB.cauchy(a.to(DEV), b.to(DEV)).item(), rel=2e-6)
        rg = RB.cauchy_backward(torch.tensor([3.0], device=DEV), a.to(DEV), b.to(DEV))
        assert torch.equal(x.grad, rg)


def test_weight_decay_grads():
    import inpc_b200
    g = torch.Generator().manual_seed(3)
    n = 1_300_001                                                  # crosses five level boundaries, ragged tail
    w = torch.randn(n, generator=g)
    g0 = torch.randn(n, generator=g)
    out = inpc_b200.compute_normalized_weight_decay_grads(w.to(DEV))
    assert_close(out.detach().cpu().numpy(), O.weight_decay(w.numpy()), rtol=1e-6, atol=0, what="weight decay")
    assert torch.all(out[:6144] == 0)
    p = torch.nn.Parameter(w.to(DEV))
    p.grad = g0.to(DEV).clone()
    inpc_b200.add_normalized_weight_decay_grads(p)
    assert_close(p.grad.detach().cpu().numpy(), O.weight_decay(w.numpy(), g0.numpy()), rtol=1e-5, atol=1e-7, what="weight decay (add)")
    # an unaligned view takes the scalar path and gives the same numbers
    out2 = inpc_b200.compute_normalized_weight_decay_grads(torch.cat([torch.zeros(1), w]).to(DEV)[1:])
    assert torch.equal(out2, out)
    if RB.available():
        assert torch.equal(out, RB.weight_decay(w.to(DEV)))


def test_probability_field_update_matches_reference_formula():
    """`ProbabilityField.update` (Modules/ProbabilityField.py:146-157) as fused kernels, against the
    reference's own torch formulation, including leaves without samples and slots without a leaf."""
    from inpc_b200 import probability_field as PF
    g = torch.Generator().manual_seed(4)
    n_leaves, n = 5000, 200_000
    leaf_w = torch.rand(n_leaves, generator=g)
    scores = torch.rand(n_leaves, generator=g) * 0.1
    idx = torch.randint(0, n_leaves // 2, (n,), generator=g)           # the upper half of the leaves gets no sample
    idx[::97] = -1
    w = torch.rand(n, generator=g) ** 4
    # the reference, on the CPU
    rw, rs = leaf_w.clone(), scores.clone()
    valid = idx >= 0
    rw.mul_(0.9968)
    rs.mul_(0.9968)
    mx, mn = torch.zeros_like(rw), torch.zeros_like(rw)
    mx.scatter_reduce_(0, idx[valid], w[valid], reduce="amax", include_self=False)
    mn.scatter_reduce_(0, idx[valid], w[valid], reduce="amin", include_self=False)
    torch.maximum(rw, mx, out=rw)
    torch.maximum(rs, (mx - mn).clamp_(0.0, 1.0), out=rs)
    # the kernels, in two accumulation steps as a multi-view batch does
    lw, sc = leaf_w.to(DEV), scores.to(DEV)
    stats = PF.LeafStatistics(n_leaves, DEV)
    half = n // 2
    stats.accumulate(idx[:half].to(DEV), w[:half].to(DEV))
    stats.accumulate(idx[half:].to(DEV), w[half:].to(DEV))
    PF.update(lw, sc, stats)
    assert torch.equal(lw.cpu(), rw) and torch.equal(sc.cpu(), rs)
    # one-call form
    lw2, sc2 = leaf_w.to(DEV), scores.to(DEV)
    PF.update_from_samples(lw2, sc2, idx.to(DEV), w.to(DEV))
    assert torch.equal(lw2, lw) and torch.equal(sc2, sc)
    with pytest.raises(TypeError):
        stats.accumulate(idx.int().to(DEV), w.to(DEV))
