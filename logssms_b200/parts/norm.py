"""RMSNorm, in the fused residual form the blocks use."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import NORMS
from .base import VECTOR, ParamSpec, Part, ones_init


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    """`forward(x, residual, other=..., in_scales=..., out_scales=...)`:
    residual <- (x [scaled, + other scaled]) + residual ; outputs = rmsnorm(residual) * out_scale_k.
    (python/logssms/layers/norm.py:56-97, python/logssms/kernel/norm.py:8-52.)"""
    kernels = ("norm",)

    def __init__(self, spec, perturb_init: bool = False):
        self.size, self.eps = spec.size, spec.eps
        self._jitter = 0.1 if perturb_init else 0.0
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), VECTOR, ones_init(self._jitter))}

    def forward(self, x, residual=None, *, other=None, in_scales=(1.0, 1.0), out_scales=(1.0,), want_residual=True):
        return K.add_rmsnorm(x, self.weight, self.eps, residual, other=other, in_scales=in_scales,
                             out_scales=out_scales, want_residual=want_residual)
