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
