"""What every part of a model is: a thing that may own tensors and children.

A `Part` declares the tensors it needs (`param_specs`: checkpoint name relative
to the part's prefix -> `ParamSpec`) and its child parts.  The weight loader
walks this tree to know every expected name and shape, checks the checkpoint
against it, and hands each part its tensors through `bind`.  The same
declaration drives the random-weights writer (`ParamSpec.init`).

This plays the role of the reference's attribute-walking `BaseOP.state_dict /
load_state_dict` (python/logssms/layers/base.py:14-59), with explicit
declarations instead of attribute introspection.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterator

import torch

# how a loaded tensor is held on the device
MATRIX = "matrix"   # matrix-product / gather operand: kept in the dtype it is stored in (bfloat16 stays
                    # bfloat16, a tensor stored in 32-bit stays 32-bit); everything becomes float32 only
                    # when the engine itself runs in float32
VECTOR = "vector"   # per-channel constants (norm weights, biases, A_log, D, conv taps): a few KB, read by
                    # kernels whose maths is 32-bit, so held as float32 (bfloat16 -> float32 is exact)
TABLE = "table"     # integer table: int32


def normal_init(std: float = 0.02):
    def init(gen: torch.Generator, shape):
        return torch.randn(shape, generator=gen, dtype=torch.float32) * std
    return init


def ones_init(jitter: float = 0.0):
    def init(gen: torch.Generator, shape):
        t = torch.ones(shape, dtype=torch.float32)
        if jitter:
            t = t + jitter * torch.randn(shape, generator=gen, dtype=torch.float32)
        return t
    return init


@dataclass(frozen=True)
class ParamSpec:
    shape: tuple[int, ...]
    role: str = MATRIX
    init: Callable[[torch.Generator, tuple[int, ...]], torch.Tensor] = normal_init()
    store_dtype: torch.dtype | None = None    # dtype the random-weights writer stores (None: the folder's dtype)


class Part:
    """Base of mixers, feed-forwards, norms, embeddings, blocks and models."""

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def children(self) -> dict[str, "Part"]:
        """prefix -> child part (prefix is prepended to the child's names)."""
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive this part's own tensors (keys as in `param_specs`), already on
        the device and in their held dtype.  Build merged layouts here."""
        for name, t in tensors.items():
            setattr(self, name.replace(".", "_"), t)

    # ---- tree walks used by the loader and the random-weights writer
    def named_param_specs(self, prefix: str = "") -> Iterator[tuple[str, ParamSpec]]:
        for name, spec in self.param_specs().items():
            yield prefix + name, spec
        for child_prefix, child in self.children().items():
            yield from child.named_param_specs(prefix + child_prefix)

    def bind_tree(self, tensors: dict[str, torch.Tensor], prefix: str = "") -> None:
        own = {name: tensors[prefix + name] for name in self.param_specs()}
        for child_prefix, child in self.children().items():
            child.bind_tree(tensors, prefix + child_prefix)
        self.bind(own)
