"""Dense projection: y = x W^T (+ b)."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init


class Linear(Part):
    kernels = ("linear_skinny", "gemm_tcgen05",)

    def __init__(self, in_features: int, out_features: int, bias: bool = False, bias_init=None):
        self.in_features, self.out_features, self.has_bias = in_features, out_features, bias
        self._bias_init = bias_init or (lambda gen, shape: torch.zeros(shape))
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def param_specs(self):
        specs = {"weight": ParamSpec((self.out_features, self.in_features), MATRIX)}
        if self.has_bias:
            specs["bias"] = ParamSpec((self.out_features,), VECTOR, self._bias_init)
        return specs

    def bind(self, tensors):
        self.weight = tensors["weight"]
        self.bias = tensors.get("bias")
        if self.bias is not None and self.weight.dtype != torch.float32:
            self.bias = self.bias.to(self.weight.dtype)      # the library product adds it in the activation dtype

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.linear(x, self.weight, self.bias)
