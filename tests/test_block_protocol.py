"""The optional protocols between a block's parts, with stand-in parts on the CPU: what the block passes on is
decided by what the parts declare, and a part that declares nothing is called in the plain way."""
from types import SimpleNamespace

from logssms_b200.parts.block import PreNormParallelBlock


class Norm:
    def __init__(self):
        self.seen = []

    def forward(self, x, residual=None, *, other=None, in_scales=(1.0, 1.0), out_scales=(1.0,), want_residual=True):
        self.seen.append((x, residual, other, in_scales, out_scales))
        return tuple(("normed", x, s) for s in out_scales), ("residual", x)


class Mixer:
    def forward(self, x, ctx, cache_layer, writes_cache=True):
        return ("mixed", x)


class PlainFeedForward:
    def __init__(self):
        self.calls = []

    def forward(self, x):
        self.calls.append({})
        return ("ff", x)


class LazyFeedForward:
    can_lazy_scale = True

    def __init__(self):
        self.calls = []

    def forward(self, x, join=None, lazy_scale=False):
        self.calls.append({"join": join, "lazy_scale": lazy_scale})
        return ("ff", x)


def block_of(feed_forward, n_mixers=1):
    block = object.__new__(PreNormParallelBlock)
    block.spec = SimpleNamespace(mixers=[SimpleNamespace(in_scale=1.0, out_scale=1.0) for _ in range(n_mixers)])
    block.mixers = [Mixer() for _ in range(n_mixers)]
    block.mixer_norm, block.ff_norm = Norm(), Norm()
    block.feed_forward = feed_forward
    return block


def test_the_output_multiplier_is_left_to_the_next_norm_only_when_both_sides_say_so():
    for extras, part, want in (
            ({"next_norm_takes_scaled": True}, LazyFeedForward(), [{"join": None, "lazy_scale": True}]),
            ({"next_norm_takes_scaled": False}, LazyFeedForward(), [{"join": None, "lazy_scale": False}]),
            ({}, LazyFeedForward(), [{"join": None, "lazy_scale": False}]),
            ({"next_norm_takes_scaled": True}, PlainFeedForward(), [{}])):       # a part that knows nothing of it
        block = block_of(part)
        out, residual = block.forward("x", "r", SimpleNamespace(extras=extras), cache_layer=0)
        assert part.calls == want
        assert out[0] == "ff" and residual == ("residual", ("mixed", ("normed", "x", 1.0)))


def test_a_block_of_stand_in_parts_runs_norm_mixer_norm_feed_forward_in_that_order():
    block = block_of(PlainFeedForward())
    out, residual = block.forward("x", None, SimpleNamespace(extras={}), cache_layer=3)
    # the first norm saw the block's input and no residual; the second one the mixer's output and the first's residual
    assert block.mixer_norm.seen == [("x", None, None, (1.0, 1.0), (1.0,))]
    (x2, r2, other, in_scales, out_scales), = block.ff_norm.seen
    assert x2 == ("mixed", ("normed", "x", 1.0)) and r2 == ("residual", "x") and other is None
    assert out == ("ff", ("normed", x2, 1.0)) and residual == ("residual", x2)
