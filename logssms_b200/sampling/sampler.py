"""Turning logits into next tokens with the fused sampling kernel."""
from __future__ import annotations

from ctypes import c_int, c_long, c_void_p
from typing import Sequence

import numpy as np
import torch

from ..ops import kernels as K
from .params import SamplingParams

_MIN_T = 1e-6      # floor of a sampling temperature, as in python/logssms/engine/sample.py:87


def sample_tokens(logits: torch.Tensor, temperature: torch.Tensor | None, top_k: torch.Tensor | None,
                  top_p: torch.Tensor | None, seeds: torch.Tensor | None, counters: torch.Tensor | None,
                  status: torch.Tensor | None = None) -> torch.Tensor:
    """One kernel launch: int32 token per row of float32 `logits`.  A row whose temperature is <= 0
    (or all rows, when `temperature` is None) takes the argmax.  With `status` (an int32 word on the device) the
    result has one element more: the word's value, so that it reaches the host in the copy of the ids."""
    K._cuda(logits, temperature, top_k, top_p, seeds, counters)
    K._need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
            "logits must be float32 [rows, vocab] with unit column stride")
    rows, V = logits.shape
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"),
                        (top_p, torch.float32, "top_p"), (seeds, torch.int64, "seeds"), (counters, torch.int64, "counters")):
        if t is not None:
            K._need(t.dtype == dt and t.shape == (rows,) and t.is_contiguous(), f"{name} must be a contiguous {dt} vector, one per row")
    if status is not None:
        K._cuda(status)
        K._need(status.dtype == torch.int32 and status.numel() == 1, "status must be one int32 word")
    out = torch.empty(rows + (status is not None), dtype=torch.int32, device=logits.device)
    f = K._fn("sample", "lb_sample", [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p])
    K._check(f(K._ptr(logits), logits.stride(0), rows, V, K._ptr(temperature), K._ptr(top_k), K._ptr(top_p),
               K._ptr(seeds), K._ptr(counters), K._ptr(out), K._ptr(status), K._stream()), "sample")
    return out


class Sampler:
    """Packs the requests' options into device vectors and calls the kernel.

    Rows are independent: a request's n-th draw uses the counter-based generator at (its seed, n),
    so what it samples does not depend on which other requests share the batch."""

    reports_kernel_errors = True      # sample(..., with_status=True) appends the device's kernel error word

    def __init__(self, device, seed: int = 0):
        self.device = torch.device(device)
        self.seed = seed

    def seed_for(self, params: SamplingParams, request_number: int) -> int:
        if params.seed is not None:
            return params.seed & 0x7FFFFFFFFFFFFFFF
        return (self.seed * 0x9E3779B97F4A7C15 + request_number * 0xD1B54A32D192ED03 + 1) & 0x7FFFFFFFFFFFFFFF

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               counters: Sequence[int], with_status: bool = False) -> torch.Tensor:
        """int32 ids, one per row.  `with_status`: one element more, the device's kernel error word
        (`K.error_word`), for a caller that copies the ids to the host anyway."""
        status = K.error_word(logits.device) if with_status else None
        if all(p.is_greedy for p in params):
            return sample_tokens(logits, None, None, None, None, None, status)
        V = logits.shape[1]
        temp = np.array([0.0 if p.is_greedy else max(p.temperature, _MIN_T) for p in params], dtype=np.float32)
        topk = np.array([p.top_k if 1 <= p.top_k < V else 0 for p in params], dtype=np.int32)
        topp = np.array([p.top_p for p in params], dtype=np.float32)
        dev = lambda a: torch.from_numpy(a).to(self.device, non_blocking=True)
        return sample_tokens(logits, dev(temp), dev(topk), dev(topp),
                             dev(np.asarray(seeds, dtype=np.int64)), dev(np.asarray(counters, dtype=np.int64)), status)
