"""Token embedding and output head."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import EMBEDDINGS, HEADS
from .base import MATRIX, ParamSpec, Part


@EMBEDDINGS.register("embedding")
class Embedding(Part):
    """out = round(table[id] * multiplier), one kernel (python/logssms/models/falcon_h1.py:213)."""
    kernels = ("embed",)

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float = 1.0):
        self.vocab_size, self.hidden_size, self.multiplier = vocab_size, hidden_size, multiplier
        self.weight: torch.Tensor | None = None
        self.bad_ids: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def bind(self, t):
        self.weight = t["weight"]
        self.bad_ids = torch.zeros(1, dtype=torch.int32, device=self.weight.device)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return K.embed_gather(self.weight, ids, self.multiplier, self.bad_ids)


@HEADS.register("lm_head")
class LMHead(Part):
    """logits = float32((h W^T) * multiplier); W is the embedding table when the model ties them
    (python/logssms/layers/embedding.py:94-106, python/logssms/models/falcon_h1.py:237)."""
    kernels = ("norm", "linear_skinny", "gemm_tcgen05")

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float, tied_to: Embedding | None):
        self.vocab_size, self.hidden_size, self.multiplier, self.tied_to = vocab_size, hidden_size, multiplier, tied_to
        self._weight = None

    def param_specs(self):
        if self.tied_to is not None:
            return {}
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def bind(self, t):
        self._weight = t.get("weight")

    @property
    def weight(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self._weight

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return K.linear(h, self.weight, out_scale=self.multiplier, out_f32=True)
