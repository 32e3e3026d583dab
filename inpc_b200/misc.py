"""Host-side mirror of the reference misc bindings
(INPCCudaBackend/INPCCudaBackend/torch_bindings/misc.py) on top of libinpc_b200."""
from __future__ import annotations

import torch
from torch.autograd.function import once_differentiable

from . import _cabi
from .rasterization import _cuda_f32, _ptr, _stream


def compute_normalized_weight_decay_grads(weights: torch.Tensor) -> torch.Tensor:
    weights = _cuda_f32(weights, "weights").reshape(-1)
    with torch.cuda.device(weights.device):
        grads = torch.empty_like(weights)
        _cabi.check(_cabi.lib().inpc_weight_decay_grads(_ptr(weights), _ptr(grads), weights.numel(), 0, _stream()))
    return grads


def add_normalized_weight_decay_grads(param: torch.nn.Parameter) -> None:
    if param.grad is None:
        raise ValueError("parameter has no gradient to add to")
    weights, grads = param.data, param.grad
    if not weights.is_cuda or not grads.is_cuda or weights.dtype != torch.float32 or grads.dtype != torch.float32:
        raise TypeError("weights and gradients must be CUDA float32 tensors")
    if not weights.is_contiguous() or not grads.is_contiguous():
        raise ValueError("weights and gradients must be contiguous (the update is in place)")
    with torch.cuda.device(weights.device):
        _cabi.check(_cabi.lib().inpc_weight_decay_grads(_ptr(weights), _ptr(grads), weights.numel(), 1, _stream()))


def spherical_contraction(positions: torch.Tensor) -> torch.Tensor:
    positions = _cuda_f32(positions, "positions")
    n = positions.shape[0]
    with torch.cuda.device(positions.device):
        out = torch.empty((n, 3), dtype=torch.float32, device=positions.device)
        _cabi.check(_cabi.lib().inpc_spherical_contraction(_ptr(positions), _ptr(out), n, _stream()))
    return out


class _FusedCauchy(torch.autograd.Function):
    """Mean Cauchy loss: forward = two kernels (partial sums, final sum), backward = one."""

    @staticmethod
    def forward(ctx, prediction, target):
        input = _cuda_f32(prediction, "input")
        target = _cuda_f32(target, "target")
        n, dev = input.numel(), input.device
        with torch.cuda.device(dev):
            loss = torch.empty((), dtype=torch.float32, device=dev)
            ws = torch.empty(int(_cabi.lib().inpc_cauchy_workspace_bytes(n)), dtype=torch.uint8, device=dev)
            _cabi.check(_cabi.lib().inpc_cauchy_loss(_ptr(input), _ptr(target), n, _ptr(loss), _ptr(ws), _stream()))
            ws.record_stream(torch.cuda.current_stream())
        ctx.set_materialize_grads(False)     # an unused loss arrives as None in backward
        ctx.save_for_backward(input, target)
        return loss

    @staticmethod
    @once_differentiable
    def backward(ctx, upstream):
        if upstream is None:
            return None, None
        input, target = ctx.saved_tensors
        grad = upstream
        grad = _cuda_f32(grad, "grad").reshape(1)
        with torch.cuda.device(input.device):
            grad_input = torch.empty_like(input)
            _cabi.check(_cabi.lib().inpc_cauchy_loss_backward(_ptr(grad), _ptr(input), _ptr(target), input.numel(),
                                                              _ptr(grad_input), _stream()))
        return grad_input, None


def fused_cauchy_loss(input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Cauchy loss between input and target with mean reduction."""
    if input.shape != target.shape:
        raise ValueError(f"input and target shapes must match ({input.shape} vs. {target.shape})")
    return _FusedCauchy.apply(input, target)
