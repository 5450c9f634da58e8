"""How parts hand each other work that a later kernel can do on the way: the fusion protocol of a step.

A part's `forward` normally takes and returns tensors.  Four small classes let it take or return something that is
*still to be done*, so that the kernel that consumes it does it in its prologue or epilogue (a decode step is bound
by the number of dependent launches, a prompt step by passes over the rows):

* `NormedRows`   — rows that are still to be normalised (a norm with `defer=True` returns them; a part whose first
  step is a product sets `takes_normed_rows = True` and hands them to `kernels.linear*`, which norm in the product's
  prologue where a kernel for that exists and call `.tensor()` otherwise).
* `ResidualJoin` — a request to a part (`forward(..., join=)`, the part sets `joins_residual = True`): let your
  last product add the residual (and the other mixer's output) in its epilogue.
* `SummedRows`   — what such a product leaves: the float32 residual sum, its rounded copy, and per 16 columns the
  rows' sums of squares; a norm that sets `takes_summed_rows = True` turns them into `NormedRows` without a pass.
* `ScaledRows`   — rows whose output multiplier is still to be applied (a norm with `takes_scaled_rows = True`
  applies it while it loads them).

Every class has `.tensor()` (or plain fields) that gives the ordinary tensor by the ordinary kernel, so a part that
knows nothing of the protocol still works: it never sets the `takes_*` / `joins_*` attributes and is never handed
anything but tensors.  A new norm, product or mixer that wants to join a fusion sets the attribute, accepts the
class, and either passes it on to `kernels.linear*` or asks for `.tensor()`.
"""
from __future__ import annotations

import torch


class ResidualJoin:
    """A request to a part: let your last product join the residual stream in its epilogue, i.e. leave
    v = [round(round(y * in_scales[0]) + round(other * in_scales[1])) or y] + residual instead of its output y.
    `other` may be a callable that returns the tensor (and first waits for whatever produces it)."""
    __slots__ = ("residual", "other", "in_scales")

    def __init__(self, residual, other=None, in_scales=(1.0, 1.0)):
        self.residual, self.other, self.in_scales = residual, other, in_scales

    def other_tensor(self):
        return self.other() if callable(self.other) else self.other


class SummedRows:
    """What a product with a residual join leaves (`linear_join`): the float32 sums `vsum` [M, N], their rounded
    copy `residual` (the new residual), and `partial` [N / 16, M], the sums of squares over blocks of 16 columns:
    everything the next RMSNorm needs, so that its consumers can norm their own columns where they load them."""
    __slots__ = ("vsum", "residual", "partial")

    def __init__(self, vsum, residual, partial):
        self.vsum, self.residual, self.partial = vsum, residual, partial

    @property
    def shape(self):
        return self.vsum.shape

    @property
    def dtype(self):
        return self.residual.dtype


class ScaledRows:
    """Rows whose output multiplier is still to be applied: round(rows * scale).  The product that made them ran in
    the library, which has no such epilogue; the norm that reads them next applies the multiplier while it loads
    them (`add_rmsnorm` with `in_scales[0]`: the same rounding), which saves a pass over the rows.  `tensor()` is
    the scaled tensor for any other use."""
    __slots__ = ("rows", "scale")

    def __init__(self, rows: torch.Tensor, scale: float):
        self.rows, self.scale = rows, float(scale)

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    def tensor(self) -> torch.Tensor:
        from . import kernels as K
        return K.scale(self.rows, self.scale)


class NormedRows:
    """Rows that are still to be normalised: what `add_rmsnorm` would compute, handed to the product that
    consumes them so that the few-row kernel can do the norm in its prologue (a decode step is bound by the
    number of dependent launches).  `residual_out` is shared by all consumers of one norm; the first product
    that runs writes it.  `tensor()` falls back to the norm kernel for any other use."""
    __slots__ = ("x", "other", "residual", "weight", "eps", "in_scales", "scale", "shared", "_tensor")

    def __init__(self, x, other, residual, weight, eps, in_scales, scale, shared):
        # x may be `SummedRows` (the product before has joined the residual already): other and residual are None then
        self.x, self.other, self.residual, self.weight, self.eps = x, other, residual, weight, eps
        self.in_scales, self.scale, self.shared = in_scales, scale, shared
        self._tensor = None

    @property
    def summed(self) -> bool:
        return isinstance(self.x, SummedRows)

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    def tensor(self) -> torch.Tensor:
        from . import kernels as K
        if self._tensor is None and self.summed:
            (self._tensor,) = K.summed_rmsnorm(self.x, self.weight, self.eps, (self.scale,))
        if self._tensor is None:
            write = self.shared["residual_out"] is not None and not self.shared["written"]
            (self._tensor,), res = K.add_rmsnorm(self.x, self.weight, self.eps, self.residual, other=self.other,
                                               in_scales=self.in_scales, out_scales=(self.scale,), want_residual=write,
                                               residual_out=self.shared["residual_out"] if write else None, in_place=False)
            if write:
                self.shared["written"] = True
        return self._tensor
