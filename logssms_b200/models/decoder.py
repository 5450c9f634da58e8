"""The one model class: embedding -> scheduled layers -> final norm -> head, all from a ModelSpec."""
from __future__ import annotations

import torch

from ..ops import build as kernel_build
from ..ops import kernels as K
from ..ops.profiler import PROFILER, nvtx_range
from ..parts import Part
from ..registry import BLOCKS, EMBEDDINGS, HEADS, NORMS


class DecoderModel(Part):
    """Runs `spec.layers` in the order of `spec.resolved_schedule()`.

    The schedule is data: an entry names the layer to run (a layer may appear twice) and the cache
    layer it uses; an entry with `writes_cache=False` reads the keys/values another entry stored.
    The cache manager is sized from `cache_needs()`: one entry per cache layer."""

    def __init__(self, spec, perturb_init: bool = False):
        self.spec = spec
        shared: dict = {}
        self.embedding = EMBEDDINGS.get(spec.embedding_kind)(spec.vocab_size, spec.hidden_size, spec.embedding_multiplier)
        self.layers = [BLOCKS.get(b.kind)(b, perturb_init=perturb_init, shared=shared) for b in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, perturb_init)
        self.lm_head = HEADS.get(spec.lm_head_kind)(spec.vocab_size, spec.hidden_size, spec.lm_head_multiplier,
                                                    self.embedding if spec.tie_word_embeddings else None)
        self.schedule = spec.resolved_schedule()
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.layers)}")
        self.num_cache_layers = max(e.cache for e in self.schedule) + 1

    def children(self):
        kids = {self.spec.embedding_name: self.embedding, self.spec.final_norm_name: self.final_norm,
                self.spec.lm_head_name: self.lm_head}
        for block_spec, block in zip(self.spec.layers, self.layers):
            kids[block_spec.prefix] = block
        return kids

    def duplicate_names(self) -> dict[str, str]:
        """Checkpoint names that may be stored although the model shares the tensor with another name: with tied
        embeddings some writers still store the output head."""
        if not self.spec.tie_word_embeddings:
            return {}
        return {self.spec.lm_head_name + "weight": self.spec.embedding_name + "weight"}

    def cache_needs(self):
        from ..cache import CacheNeeds
        needs = [None] * self.num_cache_layers
        for e in self.schedule:
            need = self.layers[e.layer].cache_needs()
            if needs[e.cache] is None:
                if not e.writes_cache:
                    raise ValueError(f"schedule entry reads cache layer {e.cache} before anything wrote it")
                needs[e.cache] = need
            elif needs[e.cache] != need:
                raise ValueError(f"cache layer {e.cache} is shared by layers with different needs")
        return [n if n is not None else CacheNeeds() for n in needs]

    def kernel_libraries(self) -> list[str]:
        """Names of the CUDA libraries this model's parts call (compiled at first use)."""
        names: list[str] = []

        def walk(part):
            names.extend(getattr(part, "kernels", ()))
            for child in part.children().values():
                walk(child)
        walk(self)
        if K.GEMM_MODE != "tcgen05":          # the engine's own tcgen05 product is built only where it is switched on
            names = [n for n in names if n != "gemm_tcgen05"]
        return list(dict.fromkeys(names))

    def setup(self, rt) -> None:
        libs = self.kernel_libraries()
        if rt.dtype == torch.float32:
            libs.append("gemm_f32")
        kernel_build.build_many(libs)
        for block in self.layers:
            block.setup(rt)

    def forward(self, ctx):
        """Residual stream after all scheduled layers, as the pair (x, residual) whose sum it is."""
        with nvtx_range("embedding"):
            x = self.embedding.forward(ctx.token_ids)
        residual = None
        for i, e in enumerate(self.schedule):
            # a block may hand its output on already joined with the residual (`SummedRows`) where the norm that
            # comes next takes it: the next block's first norm, which a block names as `input_norm` (a block that
            # names none is handed plain tensors; the rows before the head are gathered first)
            nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
            ctx.extras["next_norm_takes_summed"] = getattr(getattr(nxt, "input_norm", None), "takes_summed_rows", False)
            # ... or with its output multiplier still to be applied (`ScaledRows`); after the last block that norm is
            # the one before the head
            ctx.extras["next_norm_takes_scaled"] = getattr(getattr(nxt, "input_norm", None) if nxt is not None else self.final_norm,
                                                           "takes_scaled_rows", False)
            if PROFILER.nvtx:                      # named ranges per layer (and per part inside it) for a timeline
                with nvtx_range(f"layer {e.layer}"):
                    x, residual = self.layers[e.layer].forward(x, residual, ctx, e.cache, e.writes_cache)
            else:
                x, residual = self.layers[e.layer].forward(x, residual, ctx, e.cache, e.writes_cache)
        ctx.extras.pop("next_norm_takes_summed", None)
        ctx.extras.pop("next_norm_takes_scaled", None)
        return x, residual

    def logits(self, x: torch.Tensor, residual, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the token rows that were asked for."""
        x = K.ScaledRows(K.gather_rows(x.rows, rows), x.scale) if isinstance(x, K.ScaledRows) else K.gather_rows(x, rows)
        if residual is not None:
            residual = K.gather_rows(residual, rows)
        # The norm runs as a kernel of its own here: in the head's prologue every one of its vocabulary / 16 CTAs would
        # redo it (measured: a decode step 14-19 us longer).
        with nvtx_range("final norm + head"):
            (h,), _ = self.final_norm.forward(x, residual, want_residual=False)
            return self.lm_head.forward(h)
