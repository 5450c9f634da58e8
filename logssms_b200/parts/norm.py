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
    kernels = ("norm", "linear_skinny")
    can_defer = True          # forward() takes `defer=`: see there
    takes_summed_rows = True  # forward() takes `K.SummedRows` as x: the product before has joined the residual already
    takes_scaled_rows = True  # forward() takes `K.ScaledRows` as x: it applies the pending multiplier while it loads x

    def __init__(self, spec, perturb_init: bool = False):
        self.size, self.eps = spec.size, spec.eps
        self._jitter = 0.1 if perturb_init else 0.0
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), VECTOR, ones_init(self._jitter))}

    def forward(self, x, residual=None, *, other=None, in_scales=(1.0, 1.0), out_scales=(1.0,), want_residual=True,
                defer=False):
        """With `defer` (the caller's consumers all take `NormedRows`: their first step is a product), and
        few enough rows, nothing is launched here: the outputs are `NormedRows` that the consumers' products
        normalise in their prologue, and the new residual is a fresh tensor that the first of them writes."""
        if isinstance(x, K.ScaledRows):
            # the multiplier of the product that made x rides in this norm's load of x (as in_scales[0])
            if other is None and in_scales[0] == 1.0:
                x, in_scales = x.rows, (x.scale, in_scales[1])
            else:
                x = x.tensor()
        if isinstance(x, K.SummedRows):
            # x is already the residual sum (float32), with its rounded copy and the rows' sums of squares
            if residual is not None or other is not None:
                raise ValueError("summed rows have joined their residual already")
            if defer and K.deferred_norm_ok(x):
                shared = {"residual_out": None, "written": True}
                return tuple(K.NormedRows(x, None, None, self.weight, self.eps, (1.0, 1.0), s, shared) for s in out_scales), x.residual
            return K.summed_rmsnorm(x, self.weight, self.eps, out_scales), x.residual
        if defer and K.deferred_norm_ok(x):
            shared = {"residual_out": torch.empty_like(x) if want_residual else None, "written": False}
            outs = tuple(K.NormedRows(x, other, residual, self.weight, self.eps, in_scales, s, shared) for s in out_scales)
            return outs, shared["residual_out"]
        return K.add_rmsnorm(x, self.weight, self.eps, residual, other=other, in_scales=in_scales,
                             out_scales=out_scales, want_residual=want_residual)
