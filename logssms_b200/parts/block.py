"""How a layer's parts are arranged."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..ops.profiler import PROFILER, nvtx_range
from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .base import Part


@BLOCKS.register("prenorm_parallel")
class PreNormParallelBlock(Part):
    """norm -> one or two mixers side by side on the same normed input (each with its own input
    scale) -> their scaled sum joins the residual inside the next norm -> feed-forward.  The
    feed-forward's output joins the residual inside the NEXT block's first norm (or the final
    norm), so a block returns (x, residual) with x not yet added.

    With two mixers this is Falcon-H1's layer (python/logssms/models/falcon_h1.py:152-185);
    with one mixer and unit scales it is the plain sequential pre-norm decoder layer."""

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if not 1 <= len(spec.mixers) <= 2:
            raise ValueError("prenorm_parallel blocks take one or two mixers")
        self.spec = spec
        self.mixers = [MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared) for m in spec.mixers]
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, perturb_init)
        self.ff_norm = NORMS.get(spec.feed_forward_norm.kind)(spec.feed_forward_norm, perturb_init)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, perturb_init=perturb_init,
                                                                      shared=shared)

    @property
    def input_norm(self):
        """The norm that reads this block's input: the block before may hand it rows in the form it takes
        (`takes_summed_rows`, `takes_scaled_rows`).  A block kind that names none is handed plain tensors."""
        return self.mixer_norm

    def children(self):
        s = self.spec
        kids = {s.mixer_norm_name: self.mixer_norm, s.feed_forward_norm_name: self.ff_norm,
                s.feed_forward_name: self.feed_forward}
        for slot, mixer in zip(s.mixers, self.mixers):
            kids[slot.name] = mixer
        return kids

    def cache_needs(self):
        """Needs of all mixers of this block, merged into one cache layer."""
        from ..cache import CacheNeeds
        kv, states = None, []
        for mixer in self.mixers:
            need = mixer.cache_needs()
            if need.kv is not None:
                if kv is not None:
                    raise ValueError("a block holds at most one mixer with a key/value cache")
                kv = need.kv
            states.extend(need.states)
        names = [s.name for s in states]
        if len(set(names)) != len(names):
            raise ValueError(f"state names clash inside one block: {names}")
        return CacheNeeds(kv=kv, states=tuple(states))

    def setup(self, rt) -> None:
        for part in (*self.mixers, self.feed_forward):
            part.setup(rt)

    def forward(self, x: torch.Tensor, residual, ctx, cache_layer: int, writes_cache: bool = True):
        if PROFILER.nvtx and not getattr(self, "_ranged", False):
            # named ranges around the parts, put on once (only when ranges are switched on)
            self._ranged = True
            for part, label in [*((m, s.spec.kind) for m, s in zip(self.mixers, self.spec.mixers)),
                                (self.feed_forward, self.spec.feed_forward.kind),
                                (self.mixer_norm, "mixer norm"), (self.ff_norm, "feed-forward norm")]:
                inner = part.forward

                def ranged(*args, _inner=inner, _label=label, **kwargs):
                    with nvtx_range(_label):
                        return _inner(*args, **kwargs)
                part.forward = ranged
        slots = self.spec.mixers
        # parts whose first step is a product say so (`takes_normed_rows`): the norm in front of them can then
        # ride in that product's prologue (decode steps: fewer dependent launches)
        defer_mix = {"defer": True} if (getattr(self.mixer_norm, "can_defer", False)
                                         and all(getattr(m, "takes_normed_rows", False) for m in self.mixers)) else {}
        defer_ff = {"defer": True} if (getattr(self.ff_norm, "can_defer", False)
                                       and getattr(self.feed_forward, "takes_normed_rows", False)) else {}
        ins, residual = self.mixer_norm.forward(x, residual, out_scales=tuple(m.in_scale for m in slots), **defer_mix)
        # Where the norm in front of the feed-forward is deferred anyway, the first mixer's last product may join the
        # residual stream in its epilogue (`joins_residual`): it then returns `SummedRows`, the norm has nothing left to
        # read but those, and the feed-forward's product norms its own columns without a pass over whole rows.
        join_mix = bool(defer_ff) and getattr(self.mixers[0], "joins_residual", False) \
            and getattr(self.ff_norm, "takes_summed_rows", False) and isinstance(ins[0], K.NormedRows) \
            and (len(slots) == 2 or slots[0].out_scale == 1.0)
        in_scales = (slots[0].out_scale, slots[1].out_scale) if len(slots) == 2 else (slots[0].out_scale, 1.0)
        side = ctx.extras.get("side_stream") if len(self.mixers) == 2 else None
        if side is None:
            if join_mix:
                rest = [mixer.forward(inp, ctx, cache_layer, writes_cache) for mixer, inp in zip(self.mixers[1:], ins[1:])]
                first = self.mixers[0].forward(ins[0], ctx, cache_layer, writes_cache,
                                               join=K.ResidualJoin(residual, rest[0] if rest else None, in_scales))
                outs = [first, *rest]
            else:
                outs = [mixer.forward(inp, ctx, cache_layer, writes_cache) for mixer, inp in zip(self.mixers, ins)]
        else:
            # Inside a graph capture the two mixers go to two streams, so that the graph may run their
            # kernels side by side (each alone leaves most of the 148 SMs idle at small batch).
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                second = self.mixers[1].forward(ins[1], ctx, cache_layer, writes_cache)
                join = torch.cuda.Event()
                join.record(side)
            if join_mix:
                def other_branch():
                    main.wait_event(join)                     # called by the first mixer right before its last product
                    return second
                first = self.mixers[0].forward(ins[0], ctx, cache_layer, writes_cache,
                                               join=K.ResidualJoin(residual, other_branch, in_scales))
                if not isinstance(first, K.SummedRows):
                    main.wait_event(join)
            else:
                first = self.mixers[0].forward(ins[0], ctx, cache_layer, writes_cache)
                main.wait_event(join)
            outs = [first, second]
        next_join = bool(ctx.extras.get("next_norm_takes_summed")) and getattr(self.feed_forward, "joins_residual", False)
        if isinstance(outs[0], K.SummedRows):
            (h,), residual = self.ff_norm.forward(outs[0], None, **defer_ff)
        elif len(outs) == 2:
            (h,), residual = self.ff_norm.forward(outs[0], residual, other=outs[1],
                                                  in_scales=(slots[0].out_scale, slots[1].out_scale), **defer_ff)
        else:
            if slots[0].out_scale != 1.0:
                outs[0] = K.scale(outs[0], slots[0].out_scale)
            (h,), residual = self.ff_norm.forward(outs[0], residual, **defer_ff)
        if next_join and isinstance(h, K.NormedRows):
            # the same at the feed-forward's last product, for the norm of the next layer
            out = self.feed_forward.forward(h, join=K.ResidualJoin(residual))
            return (out, None) if isinstance(out, K.SummedRows) else (out, residual)
        if ctx.extras.get("next_norm_takes_scaled") and getattr(self.feed_forward, "can_lazy_scale", False):
            # the norm that reads the output next applies the feed-forward's output multiplier while it loads it
            return self.feed_forward.forward(h, lazy_scale=True), residual
        return self.feed_forward.forward(h), residual
