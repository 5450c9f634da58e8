"""Plain data that describes a model as parts, layer by layer.

An architecture's typed config (e.g. `FalconH1Config`) turns its config.json
keys into one `ModelSpec`.  Everything below the architecture file works from
these specs only, so no part knows which model it is in, and every size and
constant a part needs arrives as a field.

`kind` names an entry of the matching registry in `logssms_b200.registry`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding (neox / half-split pairing).

    Mirrors the reference's `RotaryConfig` (python/logssms/models/config.py:33-37).
    `scaling` is the config.json `rope_scaling` mapping as sorted items, or None.
    """
    head_dim: int
    rotary_dim: int
    theta: float
    max_position: int
    scaling: tuple[tuple[str, Any], ...] | None = None
    kind: str = "rope"


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: RopeSpec | None
    key_scale: float = 1.0
    softmax_scale: float | None = None      # None -> head_dim ** -0.5
    window: int | None = None               # None -> all earlier keys
    kind: str = "attention"


@dataclass(frozen=True)
class Mamba2Spec:
    """Mamba2 (SSD) mixer with a depthwise causal conv in front."""
    hidden_size: int
    num_heads: int
    head_dim: int
    state_dim: int
    num_groups: int
    conv_kernel: int
    conv_bias: bool
    proj_bias: bool
    out_bias: bool
    gated_norm: bool
    norm_before_gate: bool
    norm_eps: float
    multipliers: tuple[float, float, float, float, float]   # gate z, x, B, C, dt
    chunk_size: int
    kind: str = "mamba2"

    @property
    def inner_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def conv_dim(self) -> int:
        return self.inner_size + 2 * self.num_groups * self.state_dim

    @property
    def proj_size(self) -> int:
        return self.inner_size + self.conv_dim + self.num_heads


@dataclass(frozen=True)
class GatedMLPSpec:
    hidden_size: int
    intermediate_size: int
    activation_scale: float = 1.0
    output_scale: float = 1.0
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class MixerSlot:
    """One mixer of a block: its spec, the checkpoint prefix of its tensors
    (relative to the block's prefix), and the scales applied to the normed
    input it reads and to the output it adds to the residual stream."""
    spec: Any
    name: str
    in_scale: float = 1.0
    out_scale: float = 1.0


@dataclass(frozen=True)
class BlockSpec:
    """Pre-norm block: norm -> mixers side by side on the same normed input ->
    their scaled sum joins the residual -> norm -> feed-forward."""
    prefix: str
    mixers: tuple[MixerSlot, ...]
    mixer_norm: NormSpec
    mixer_norm_name: str
    feed_forward: Any
    feed_forward_name: str
    feed_forward_norm: NormSpec
    feed_forward_norm_name: str
    kind: str = "prenorm_parallel"


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  `layer` indexes `ModelSpec.layers` (a layer
    may appear in several entries: its weights then run more than once).
    `cache` names the cache layer this execution uses; by default every entry
    owns one.  An entry whose `cache` equals an earlier entry's and which has
    `writes_cache=False` reads that entry's keys/values instead of storing its own."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding_name: str
    embedding_multiplier: float
    lm_head_name: str
    lm_head_multiplier: float
    tie_word_embeddings: bool
    final_norm: NormSpec
    final_norm_name: str
    layers: tuple[BlockSpec, ...]
    schedule: tuple[ScheduleEntry, ...] = field(default=())
    embedding_kind: str = "embedding"       # registry.EMBEDDINGS: built as cls(vocab_size, hidden_size, multiplier)
    lm_head_kind: str = "lm_head"           # registry.HEADS: built as cls(vocab_size, hidden_size, multiplier, tied_to)

    def resolved_schedule(self) -> tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i, i) for i in range(len(self.layers)))
