"""Rotary position encoding: inverse frequencies on the host, cos/sin table on the device."""
from __future__ import annotations

import math

import torch

from ..ops import kernels as K
from ..registry import POSITION_ENCODINGS
from .base import Part


def inverse_frequencies(spec) -> torch.Tensor:
    """float32 inverse frequencies with the `llama3` / `yarn` post-processing of config.json's
    rope_scaling (python/logssms/layers/rotary.py:24-26, 63-122)."""
    d = spec.rotary_dim
    inv = 1.0 / (spec.theta ** (torch.arange(0, d, 2, dtype=torch.float) / d))
    scaling = dict(spec.scaling) if spec.scaling else None
    if not scaling or scaling.get("rope_type", "default") == "default":
        return inv
    kind = scaling["rope_type"]
    if kind == "llama3":
        factor, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
        orig = scaling["original_max_position_embeddings"]
        wave_len = 2 * math.pi / inv
        if low == high:
            return torch.where(wave_len < orig / high, inv, inv / factor)
        smooth = torch.clamp((orig / wave_len - low) / (high - low), 0, 1)
        return ((1 - smooth) / factor + smooth) * inv
    if kind == "yarn":
        factor = scaling["factor"]
        beta_fast, beta_slow = scaling.get("beta_fast", 32.0), scaling.get("beta_slow", 1.0)
        orig = scaling["original_max_position_embeddings"]

        def correction_dim(rotations: float) -> float:
            return d * math.log(orig / (rotations * 2 * math.pi)) / (2 * math.log(spec.theta))
        lo = max(math.floor(correction_dim(beta_fast)), 0)
        hi = min(math.ceil(correction_dim(beta_slow)), d // 2 - 1)
        ramp = torch.clamp((torch.arange(d // 2, dtype=torch.float32) - lo) / max(hi - lo, 1), 0, 1)
        return (inv / factor) * ramp + inv * (1 - ramp)
    raise ValueError(f"Unsupported rope_scaling {scaling!r}")


@POSITION_ENCODINGS.register("rope")
class RotaryEmbedding(Part):
    """Owns the float32 [positions, rotary_dim] cos|sin table that the fused rotate-and-store kernel reads."""
    kernels = ("rope",)

    def __init__(self, spec):
        self.spec = spec
        self.table: torch.Tensor | None = None

    def setup(self, rt) -> None:
        # one row per position the engine can ever hold: its sequence limit replaces the model's
        # max_position_embeddings when the two differ (python/logssms/engine/config.py:76-80), and the kernels
        # index the table by position without a check of their own
        rows = max(rt.max_seq_len, 1)
        if self.table is None or self.table.shape[0] != rows or self.table.device != rt.device:
            self.table = K.rope_table(inverse_frequencies(self.spec).to(rt.device), rows)


class NoPositionEncoding(Part):
    """Stand-in for attention without rotation: an empty table (rotary_dim 0)."""

    def __init__(self):
        self.table = None

    def setup(self, rt) -> None:
        self.table = torch.empty((1, 0), dtype=torch.float32, device=rt.device)
