"""Host side of a step: from (request, tokens, wanted places) to the device tables a model reads.

`StepPlanner.plan` checks the entries, makes room in the cache, and packs every per-step integer
(token ids, positions, request of each token, run boundaries, start positions, state slots, rows whose
logits are wanted, and per page group the slot of every token and the block tables) into ONE pinned
buffer that goes to the device in one copy, as the reference's `BatchIndices` does
(python/logssms/utils/batch.py:43-101).  It needs only a `CacheManager`, so a single part can be
stepped in a test without a model around it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache import CacheManager, RequestCache
from ..parts import StepContext
from ..parts.context import SHORT_PORTION, Padding


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose logits are wanted.

    `start`: the position of the first of these tokens, when the caller keeps count itself (None: the length of the
    request's cache).  With it a step can be planned a second time: a plan that was made ahead and then dropped has
    grown the caches of its requests already, and planning the same tokens again at the same positions grows nothing."""
    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    start: int | None = None


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


class StaticTables:
    """Fixed place and width for a step's tables, so that a captured CUDA graph finds them again."""

    def __init__(self):
        self.tables: torch.Tensor | None = None
        self.ctx: StepContext | None = None


@dataclass(frozen=True)
class Bucket:
    """Sizes a step is filled up to (see `parts.context.Padding`): requests, tokens, long portions, tokens of short
    portions.  Wanted places are filled up to `requests`."""
    requests: int
    tokens: int
    long_cap: int
    short_cap: int


def _up(n: int, steps) -> int:
    for size, grain in steps:
        if n <= size:
            return -(-n // grain) * grain
    size, grain = steps[-1]
    return -(-n // grain) * grain


def bucket_for(lens, wanted: int) -> Bucket | None:
    """The bucket of a step whose requests bring `lens` tokens and that wants `wanted` places, or None if it has
    none (more wanted places than requests).  Every bucket leaves room for at least one dummy single token and a
    dummy portion of more than SHORT_PORTION tokens: the work lists are filled up with those."""
    B = len(lens)
    requests = _up(B + 2, ((8, 4), (32, 8), (64, 16), (1 << 30, 32)))
    if wanted > requests:
        return None
    singles = requests - B - 1
    tokens = _up(int(sum(lens)) + singles + SHORT_PORTION + 1, ((512, 64), (2048, 128), (1 << 30, 256)))
    n_long = sum(1 for n in lens if n > SHORT_PORTION) + 1
    n_short = sum(int(n) for n in lens if n <= SHORT_PORTION) + singles
    return Bucket(requests, tokens, _up(n_long, ((2, 2), (4, 4), (1 << 30, 8))),
                  _up(n_short, ((8, 8), (32, 8), (64, 16), (1 << 30, 64))))


class StepPlanner:
    def __init__(self, cache: CacheManager, device, vocab_size: int | None = None):
        self.cache = cache
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.page_size = cache.page_size
        self.max_seq_len = cache.max_seq_len
        self._ring = _PinnedRing()
        self._staging: torch.Tensor | None = None
        self._staging_half = 0
        self.h2d_bytes = 0          # bytes of step tables copied host -> device so far

    def plan(self, entries: Sequence[StepEntry], static: StaticTables | None = None,
             bucket: Bucket | None = None, pad_singles: int = 0) -> StepContext:
        """Host side of a step: checks, room in the cache, and every per-step integer packed into one
        pinned buffer and copied to the device at once.  With `static` (a captured step's slot) the
        tables keep a fixed width and a fixed place on the device, so that a captured graph finds them;
        every later step planned into the same slot must bring the same numbers of tokens and wanted
        places, request by request, or, with `bucket`, fit the same bucket: the step is then filled up
        with dummy requests (single tokens and one portion, on a state slot and a cache page of their
        own) to the bucket's numbers of requests, tokens and wanted places, and the context's work lists
        have the bucket's fixed lengths.  `pad_singles` (a step of single decoded tokens replayed from the graph of a
        larger batch): that many dummy requests of one token each, which want their logits like the others, follow
        the real ones."""
        B = len(entries)
        seen = set()
        for e in entries:
            if id(e.request) in seen:
                raise ValueError("a request appears twice in one step")
            seen.add(id(e.request))
            if self.cache.live.get(e.request.row) is not e.request:
                raise ValueError("step entry names a request that is not live")
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=B)
        starts = np.fromiter((e.request.length if e.start is None else e.start for e in entries), dtype=np.int64, count=B)
        for e, s0, n in zip(entries, starts, lens):
            if not s0 <= e.request.length <= s0 + n:
                raise ValueError(f"an entry starts at position {int(s0)}, its request's cache holds {e.request.length} tokens")
        T = int(lens.sum())
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(lens, out=cu[1:])
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if self.vocab_size is not None and (tokens.min() < 0 or tokens.max() >= self.vocab_size):
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        for e, n in zip(entries, lens):
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted place {w} is outside the entry's {n} tokens")
        # room in the cache first, for all entries or for none (a step that cannot run leaves no request grown);
        # extending may give back pages a window has passed
        self.cache.check_room([(e.request, int(s + n)) for e, s, n in zip(entries, starts, lens)])
        for e, s, n in zip(entries, starts, lens):
            self.cache.extend(e.request, int(s + n), first_pos=int(s))
        rows = np.fromiter((e.request.row for e in entries), dtype=np.int64, count=B)
        logit_rows = np.asarray([cu[b] + w for b, e in enumerate(entries) for w in e.want], dtype=np.int64)
        real_entries = B
        if bucket is not None:
            # dummy requests behind the real ones: single tokens, then one portion that takes the rest of the tokens
            singles = bucket.requests - B - 1
            portion = bucket.tokens - T - singles
            if singles < 1 or portion <= SHORT_PORTION or len(logit_rows) > bucket.requests:
                raise ValueError("the step does not fit the bucket it was planned for")
            lens = np.concatenate([lens, np.ones(singles, dtype=np.int64), [portion]])
            starts = np.concatenate([starts, np.zeros(singles + 1, dtype=np.int64)])
            rows = np.concatenate([rows, np.full(singles + 1, self.cache.dummy_row, dtype=np.int64)])
            tokens = np.concatenate([tokens, np.zeros(singles + portion, dtype=np.int64)])
            B, T = bucket.requests, bucket.tokens
            cu = np.zeros(B + 1, dtype=np.int64)
            np.cumsum(lens, out=cu[1:])
            logit_rows = np.concatenate([logit_rows, np.full(bucket.requests - len(logit_rows), T - 1, dtype=np.int64)])
        elif pad_singles > 0:
            lens = np.concatenate([lens, np.ones(pad_singles, dtype=np.int64)])
            starts = np.concatenate([starts, np.zeros(pad_singles, dtype=np.int64)])
            rows = np.concatenate([rows, np.full(pad_singles, self.cache.dummy_row, dtype=np.int64)])
            tokens = np.concatenate([tokens, np.zeros(pad_singles, dtype=np.int64)])
            logit_rows = np.concatenate([logit_rows, T + np.arange(pad_singles, dtype=np.int64)])
            B, T = B + pad_singles, T + pad_singles
            cu = np.zeros(B + 1, dtype=np.int64)
            np.cumsum(lens, out=cu[1:])
        token_req = np.repeat(np.arange(B, dtype=np.int64), lens)
        positions = np.arange(T, dtype=np.int64) - np.repeat(cu[:-1], lens) + np.repeat(starts, lens)
        groups = self.cache.groups
        ps = self.page_size
        max_context = int((starts[:real_entries] + lens[:real_entries]).max())
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
            ctx = static.ctx
            if bucket is not None:
                ctx.host_lens, ctx.host_starts = lens, starts
                ctx.padding = Padding(real_entries, bucket.long_cap, bucket.short_cap)
                ctx.refresh_lists()
            return ctx

        def view(i, shape=None):
            t = dev[int(offsets[i]): int(offsets[i]) + sizes[i]]
            return t if shape is None else t.view(shape)
        block_tables = [view(8 + 2 * gi, (B, tables[gi].shape[1])) for gi in range(len(groups))]
        slot_mappings = [view(7 + 2 * gi) for gi in range(len(groups))]
        ctx = StepContext(
            num_tokens=T, num_requests=B, max_len=int(lens.max()), token_ids=view(0), positions=view(1),
            token_req=view(2), cu_seqlens=view(3), start_pos=view(4), slots=view(5),
            block_tables=block_tables, slot_mappings=slot_mappings, logit_rows=view(6), cache=self.cache,
            # a captured step is replayed for other requests of the same lengths: the most keys any of them may
            # have, and work lists that depend on the lengths only (their order, a matter of speed, is that of
            # the step they were built for)
            max_context=max_context if static is None else self.max_seq_len,
            host_lens=lens, host_starts=starts,
            padding=None if bucket is None else Padding(real_entries, bucket.long_cap, bucket.short_cap),
        )
        if bucket is not None:
            ctx.max_len = T               # an upper bound: the longest real portion differs from step to step
        if static is not None:
            static.ctx = ctx
        return ctx
