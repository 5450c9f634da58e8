"""The step function: run a batch of (request, its next tokens) from the cache.

`Engine.step(entries)` takes any mix of prompt portions and single decoded
tokens, cut anywhere, and runs only those tokens as one batch: keys/values go
into the requests' pages, conv windows and SSM states are read from and written
back to the requests' slots, and float32 logits come back for exactly the token
places that were asked for.  Sampling is not part of a step.

One kind of batch only: where the reference distinguishes prefill / decode /
mixed batches with a padded prefill region (python/logssms/core.py:116-193,
python/logssms/engine/engine.py:262-356), a decoded token here is a portion of
length one.  All per-step integers travel to the device in ONE pinned copy, as
in the reference's `BatchIndices` (python/logssms/utils/batch.py:43-101).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache import CacheManager, RequestCache
from ..config import load_model_config
from ..models import build_model
from ..ops import kernels as K
from ..parts import Runtime, StepContext
from ..weights import load_weights

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose logits are wanted."""
    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class _PinnedRing:
    """A few pinned staging buffers used in turn, each guarded by the event of its last copy."""

    def __init__(self, n: int = 4):
        self.bufs: list[torch.Tensor | None] = [None] * n
        self.events: list[torch.cuda.Event | None] = [None] * n
        self.i = 0

    def take(self, size: int) -> tuple[torch.Tensor, int]:
        self.i = (self.i + 1) % len(self.bufs)
        ev = self.events[self.i]
        if ev is not None:
            ev.synchronize()
        buf = self.bufs[self.i]
        if buf is None or buf.numel() < size:
            buf = torch.empty(max(size, 4096), dtype=torch.int32, pin_memory=True)
            self.bufs[self.i] = buf
        return buf, self.i

    def mark(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class Engine:
    """Model + weights + cache on one GPU, and the step function over them."""

    def __init__(self, model_dir: str, dtype="bfloat16", *, max_requests: int = 64, max_seq_len: int = 8192,
                 page_size: int = 64, num_pages: int | None = None, memory_ratio: float = 0.9,
                 device: str = "cuda:0", poison_on_free: bool = False, max_step_tokens: int = 1 << 30,
                 use_graphs: bool = True, max_graphs: int = 16):
        if not torch.cuda.is_available():
            raise RuntimeError("logssms_b200 needs a CUDA device (built for sm_100a); there is no CPU path")
        try:
            self.dtype = _DTYPES[dtype]
        except KeyError:
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.config = load_model_config(model_dir)
        self.model = build_model(self.config)
        self.page_size = page_size
        self.max_seq_len = max_seq_len
        with torch.inference_mode():
            load_weights(self.model, model_dir, self.dtype, self.device)
            self.model.setup(Runtime(self.device, self.dtype, max_seq_len, page_size))
        needs = self.model.cache_needs()
        if num_pages is None:
            num_pages = self._pages_that_fit(needs, max_requests, memory_ratio)
        self.cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                                  max_seq_len=max_seq_len, dtype=self.dtype, device=self.device,
                                  poison_on_free=poison_on_free, max_step_tokens=max_step_tokens)
        self.vocab_size = self.model.spec.vocab_size
        self._ring = _PinnedRing()
        self._staging: torch.Tensor | None = None
        self._staging_half = 0
        self.use_graphs = use_graphs
        self.max_graphs = max_graphs
        self._graphs: dict[int, _DecodeGraph] = {}
        self.steps_run = 0
        self.h2d_bytes = 0          # bytes of step tables copied host -> device so far

    def _pages_that_fit(self, needs, max_requests: int, memory_ratio: float) -> int:
        """Pages for `memory_ratio` of the device after weights and state slots, capped at what
        `max_requests` full-length requests could ever use (the reference plans the same way,
        python/logssms/cache/naive/manager.py:352-399)."""
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - (1.0 - memory_ratio) * total - max_requests * CacheManager.bytes_per_request_state(needs, self.dtype)
        per_page = max(CacheManager.bytes_per_page(needs, self.page_size, self.dtype), 1)
        cap = max_requests * (-(-self.max_seq_len // self.page_size))
        pages = int(min(max(budget, 0) // per_page, cap))
        if pages < 1:
            raise RuntimeError("not enough device memory left for a single cache page")
        return pages

    # ------------------------------------------------------------------ requests
    def new_request(self, reserve_tokens: int = 0) -> RequestCache:
        return self.cache.admit(reserve_tokens)

    def release(self, request: RequestCache) -> None:
        self.cache.release(request)

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens as one batch; return float32 logits [wanted, vocab] in the order
        of the entries and of each entry's `want`.

        A step of single decoded tokens that all want their logits is replayed from a CUDA graph
        (one per batch size, captured the second time that size is seen); the returned tensor is then
        the graph's own output buffer, valid until the next step of the same size."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        if self.use_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._decode_step(entries)
        ctx = self._plan(entries)
        x, residual = self.model.forward(ctx)
        self.steps_run += 1
        if ctx.logit_rows.numel() == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.logits(x, residual, ctx.logit_rows)

    def _decode_step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        B = len(entries)
        slot = self._graphs.get(B)
        if slot is None:
            if len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            slot = self._graphs[B] = _DecodeGraph()
        slot.seen += 1
        if slot.graph is None and slot.seen < 2:
            ctx = self._plan(entries)              # first time: eager (this also builds and loads every kernel)
            x, residual = self.model.forward(ctx)
            self.steps_run += 1
            return self.model.logits(x, residual, ctx.logit_rows)
        ctx = self._plan(entries, slot)
        if slot.graph is None:
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = K.launch_count
            with torch.cuda.graph(graph):
                x, residual = self.model.forward(ctx)
                slot.logits = self.model.logits(x, residual, ctx.logit_rows)
            slot.launches = K.launch_count - before
            K.launch_count = before
            slot.graph = graph
        slot.graph.replay()
        K.launch_count += slot.launches
        self.steps_run += 1
        return slot.logits

    def _plan(self, entries: Sequence[StepEntry], static: "_DecodeGraph | None" = None) -> StepContext:
        """Host side of a step: checks, room in the cache, and every per-step integer packed into one
        pinned buffer and copied to the device at once.  With `static` (a decode graph's slot) the
        tables keep a fixed width and a fixed place on the device, so that a captured graph finds them."""
        B = len(entries)
        seen = set()
        for e in entries:
            if id(e.request) in seen:
                raise ValueError("a request appears twice in one step")
            seen.add(id(e.request))
            if self.cache.live.get(e.request.row) is not e.request:
                raise ValueError("step entry names a request that is not live")
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=B)
        starts = np.fromiter((e.request.length for e in entries), dtype=np.int64, count=B)
        T = int(lens.sum())
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(lens, out=cu[1:])
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= self.vocab_size:
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        for e, n in zip(entries, lens):
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted place {w} is outside the entry's {n} tokens")
        # room in the cache first: this may give back pages a window has passed
        for e, s, n in zip(entries, starts, lens):
            self.cache.extend(e.request, int(s + n))
        token_req = np.repeat(np.arange(B, dtype=np.int64), lens)
        positions = np.arange(T, dtype=np.int64) - np.repeat(cu[:-1], lens) + np.repeat(starts, lens)
        rows = np.fromiter((e.request.row for e in entries), dtype=np.int64, count=B)
        logit_rows = np.asarray([cu[b] + w for b, e in enumerate(entries) for w in e.want], dtype=np.int64)
        groups = self.cache.groups
        ps = self.page_size
        max_context = int((starts + lens).max())
        P = self.cache.max_pages_per_request if static is not None else -(-max_context // ps)
        tables, mappings = [], []
        for g in groups:
            bt = g.block_table[rows, :P]
            page_of_token = bt[token_req, positions // ps].astype(np.int64)
            if (page_of_token < 0).any():
                raise AssertionError("a token of this step has no page")
            tables.append(bt)
            mappings.append(page_of_token * ps + positions % ps)
        # pack -> one pinned buffer -> one copy
        sections = [tokens, positions, token_req, cu, starts, rows, logit_rows]
        for bt, mp in zip(tables, mappings):
            sections += [mp, bt.reshape(-1)]
        sizes = [int(s.size) for s in sections]
        offsets = np.concatenate([[0], np.cumsum([(n + 3) // 4 * 4 for n in sizes])])
        total = int(offsets[-1])
        pinned, ring_slot = self._ring.take(total)
        host = pinned.numpy()
        for s, off, n in zip(sections, offsets[:-1], sizes):
            host[off:off + n] = s
        if static is not None:
            if static.tables is None:
                static.tables = torch.empty(total, dtype=torch.int32, device=self.device)
            dev = static.tables
        else:
            if self._staging is None or self._staging.numel() < 2 * total:
                self._staging = torch.empty(max(total, 4096) * 2, dtype=torch.int32, device=self.device)
            # alternate halves so that a step's tables are not overwritten while an earlier step may still run
            self._staging_half ^= 1
            half = self._staging.numel() // 2
            dev = self._staging[self._staging_half * half: self._staging_half * half + total]
        dev.copy_(pinned[:total], non_blocking=True)
        self.h2d_bytes += total * 4
        self._ring.mark(ring_slot)
        if static is not None and static.ctx is not None:
            return static.ctx

        def view(i, shape=None):
            t = dev[int(offsets[i]): int(offsets[i]) + sizes[i]]
            return t if shape is None else t.view(shape)
        block_tables = [view(8 + 2 * gi, (B, tables[gi].shape[1])) for gi in range(len(groups))]
        slot_mappings = [view(7 + 2 * gi) for gi in range(len(groups))]
        ctx = StepContext(
            num_tokens=T, num_requests=B, max_len=int(lens.max()), token_ids=view(0), positions=view(1),
            token_req=view(2), cu_seqlens=view(3), start_pos=view(4), slots=view(5),
            block_tables=block_tables, slot_mappings=slot_mappings, logit_rows=view(6), cache=self.cache,
            max_context=max_context if static is None else self.max_seq_len,
            host_lens=None if static is not None else lens, host_starts=None if static is not None else starts,
        )
        if static is not None:
            static.ctx = ctx
        return ctx


class _DecodeGraph:
    """A captured decode step for one batch size: its table buffer on the device, the step context
    whose tensors are views of that buffer, the graph, and the logits it writes."""

    def __init__(self):
        self.seen = 0
        self.tables: torch.Tensor | None = None
        self.ctx: StepContext | None = None
        self.graph = None
        self.logits: torch.Tensor | None = None
        self.launches = 0
