"""inpc_b200 — B200-native (sm_100a) replacement for the INPCCudaBackend extension of
nerficg-project/INPC.  Exports the same names as the reference package
(INPCCudaBackend/__init__.py:14-21); underneath, every operation is a kernel of the C-ABI library
`libinpc_b200.so` (declared in include/inpc_b200.h)."""
from .rasterization import INPCRasterizer, RasterizerSettings, RasterizerMode
from .sampling import ProbabilityFieldSampler, compute_viewpoint_weights
from .misc import (compute_normalized_weight_decay_grads, add_normalized_weight_decay_grads, spherical_contraction,
                   fused_cauchy_loss)

__all__ = [
    'INPCRasterizer', 'RasterizerSettings', 'RasterizerMode',
    'ProbabilityFieldSampler', 'compute_viewpoint_weights',
    'compute_normalized_weight_decay_grads', 'add_normalized_weight_decay_grads', 'spherical_contraction',
    'fused_cauchy_loss',
]
