"""Opt-in timing of the engine's kernels by class, and NVTX ranges around the parts of a step.

The reference marks layers, sampler and graph replays with NVTX ranges (python/logssms/utils/torch_utils.py:41-64)
and keeps an opt-in profiler that times the stages of a step with CUDA events and writes JSON
(python/logssms/engine/profile.py:41).  Here: `PROFILER.enable()` makes every launch of the package's own kernels
(and every library product) record a CUDA event before and after itself; `report()` sums the device times per
kernel class (attention, mamba2, products, norms, ...) and per kernel.  Timed steps run kernel by kernel: a replayed
CUDA graph has no place for the events.  `nvtx_range` wraps a part's work in a named range when ranges are on.
"""
from __future__ import annotations

from contextlib import contextmanager

import torch

# kernel library -> class of work it is counted under
CLASSES = {
    "embed": "embedding", "norm": "norms and gates", "rope": "attention", "attention_decode": "attention",
    "attention_decode_fused": "attention", "attention_prefill": "attention", "attention_prefill_tc": "attention",
    "conv": "mamba2", "ssm": "mamba2", "ssd": "mamba2", "ssd_tc": "mamba2", "gemm_f32": "products",
    "gemm_tcgen05": "products", "linear_skinny": "products", "library": "products", "sample": "sampling",
}


class KernelProfiler:
    def __init__(self):
        self.enabled = False
        self.nvtx = False
        self._pending: list[tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = []
        self._totals: dict[tuple[str, str], list] = {}
        self.steps = 0

    def enable(self, nvtx: bool = False) -> None:
        self.enabled, self.nvtx = True, nvtx

    def disable(self) -> None:
        self.enabled = self.nvtx = False

    def timed(self, lib: str, name: str, call):
        """Run `call()` between two events on the current stream; returns its result."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = call()
        stop.record()
        self._pending.append((lib, name, start, stop))
        return out

    def collect(self) -> None:
        """Wait for the device and add the pending launches' times to the totals."""
        if not self._pending:
            return
        torch.cuda.synchronize()
        for lib, name, start, stop in self._pending:
            entry = self._totals.setdefault((lib, name), [0, 0.0])
            entry[0] += 1
            entry[1] += start.elapsed_time(stop)
        self._pending.clear()

    def report(self) -> dict:
        """{"steps", "classes": {class: {"launches", "ms"}}, "kernels": {"lib.name": {"launches", "ms"}}}; times
        are sums of the kernels' own device times (kernels that overlap on two streams count twice)."""
        self.collect()
        classes: dict[str, dict] = {}
        kernels = {}
        for (lib, name), (n, ms) in sorted(self._totals.items(), key=lambda kv: -kv[1][1]):
            c = classes.setdefault(CLASSES.get(lib, lib), {"launches": 0, "ms": 0.0})
            c["launches"] += n
            c["ms"] += ms
            kernels[f"{lib}.{name}"] = {"launches": n, "ms": ms}
        return {"steps": self.steps, "classes": classes, "kernels": kernels}

    def reset(self) -> None:
        self._pending.clear()
        self._totals.clear()
        self.steps = 0


PROFILER = KernelProfiler()


@contextmanager
def nvtx_range(name: str):
    """A named NVTX range around the body when ranges are switched on (`PROFILER.nvtx`), else nothing."""
    if not PROFILER.nvtx:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
