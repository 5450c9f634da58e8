"""Gated (SwiGLU) feed-forward."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import FEED_FORWARDS
from .base import MATRIX, ParamSpec, Part


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(Part):
    """down(silu(gate * s0) * up) * s1.  `gate_proj` and `up_proj` are concatenated at bind time
    (python/logssms/models/weight.py:32-33); flow python/logssms/layers/mlp.py:50-61."""
    takes_normed_rows = True      # forward() passes its input straight into a product
    joins_residual = True         # forward() takes `join=`: its last product may add the residual in its epilogue
    kernels = ("norm", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self.gate_up = self.down = None

    def param_specs(self):
        s = self.spec
        return {
            "gate_proj.weight": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX),
            "up_proj.weight": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX),
            "down_proj.weight": ParamSpec((s.hidden_size, s.intermediate_size), MATRIX),
        }

    def bind(self, t):
        self.gate_up = torch.cat([t["gate_proj.weight"], t["up_proj.weight"]], 0).contiguous()
        self.down = t["down_proj.weight"]

    def setup(self, rt) -> None:
        pass

    can_lazy_scale = True     # forward() takes `lazy_scale=`: see there

    def forward(self, x: torch.Tensor, join=None, lazy_scale: bool = False):
        """With `join` (a `K.ResidualJoin`) and few rows the down projection adds the residual in its epilogue and
        `K.SummedRows` come back instead of a tensor.  With `lazy_scale` (the norm that reads the output next takes
        `K.ScaledRows`) the output multiplier may be left to that norm."""
        s = self.spec
        h = K.linear_swiglu(x, self.gate_up, s.activation_scale)
        if K.linear_join_ok(h, self.down, None, join):
            return K.linear_join(h, self.down, None, join, out_scale=s.output_scale)
        return K.linear(h, self.down, out_scale=s.output_scale, lazy_scale=lazy_scale)
