"""What a part sees of the running step and of the engine it runs in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import numpy as np
import torch

SHORT_PORTION = 8      # a portion of at most this many tokens is run token by token (the decode kernels)


@dataclass(frozen=True)
class Runtime:
    """Facts about the engine that a part may need to size its own tables."""
    device: torch.device
    dtype: torch.dtype
    max_seq_len: int
    page_size: int
    # choices of the engine's user that a part may honour, by name ("ssm_state_dtype": "float32" | "activation")
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class Padding:
    """A step that was filled up to a bucket of sizes, so that one captured graph serves every step of the bucket.

    Behind the `entries` real requests of the batch lie dummy ones that all use a state slot and a cache page nobody
    else uses: first single tokens, then one portion of more than SHORT_PORTION tokens (the last request of the
    batch).  To the kernels they are requests like any other; nobody reads what they compute.  The work lists below
    have fixed lengths (`*_cap`): lists of tiles and chunks end in entries that name request -1 (no work), lists of
    single tokens and of requests are filled up with a dummy single token.  What the dummy requests compute stays
    finite like any request's, which matters: a tensor-core kernel that reads a box of rows beyond its own request's
    end multiplies them by zero weights, and 0 x NaN is NaN."""
    entries: int          # real requests; requests entries .. num_requests - 1 are dummies
    long_cap: int         # most portions of more than SHORT_PORTION tokens, the dummy one included
    short_cap: int        # most tokens of portions of at most SHORT_PORTION tokens, the dummy ones included


# --------------------------------------------------------------------------- work lists (host side, numpy)
def _fill(rows: list, cap: int | None, filler, width: int) -> np.ndarray:
    if cap is not None:
        if len(rows) > cap:
            raise ValueError(f"a work list of {len(rows)} entries exceeds its fixed length {cap}")
        rows = rows + [filler] * (cap - len(rows))
    return np.asarray(rows, dtype=np.int32).reshape(-1, width) if width > 1 else np.asarray(rows, dtype=np.int32)


def tile_list(lens, starts, tile: int, cap: int | None = None) -> np.ndarray:
    """int32 [n, 2]: (request index in the batch, first token within its portion) for every run of `tile` tokens of
    every portion longer than SHORT_PORTION, the tile that sees the most keys first (a causal tile's cost grows with
    its position).  With `cap` the list has exactly that many rows; the surplus rows name request -1, which the
    kernels skip."""
    pairs = [(b, t0) for b, n in enumerate(lens) if n > SHORT_PORTION for t0 in range(0, int(n), tile)]
    pairs.sort(key=lambda bt: -(int(starts[bt[0]]) + min(bt[1] + tile, int(lens[bt[0]]))))
    return _fill(pairs, cap, (-1, 0), 2)


def short_token_list(lens, cap: int | None = None, filler: int = 0) -> np.ndarray:
    """int32 token indices (rows of the step's batch) of all portions of at most SHORT_PORTION tokens."""
    cu = np.concatenate([[0], np.cumsum(lens)])
    idx = [t for b, n in enumerate(lens) if n <= SHORT_PORTION for t in range(int(cu[b]), int(cu[b + 1]))]
    return _fill(idx, cap, filler, 1)


def chunk_lists(lens, chunk: int, cap_chunks: int | None = None, cap_long: int | None = None) -> tuple[np.ndarray, np.ndarray]:
    """Work lists of a chunked scan over the long portions: int32 [n, 2] (request index, first token of the chunk
    within its portion) and int32 [m, 3] (request index, its first chunk, its number of chunks).  With capacities the
    surplus rows name request -1, which the kernels skip."""
    chunks, per_request = [], []
    for b, n in enumerate(lens):
        if n > SHORT_PORTION:
            first = len(chunks)
            chunks += [(b, t0) for t0 in range(0, int(n), chunk)]
            per_request.append((b, first, len(chunks) - first))
    return _fill(chunks, cap_chunks, (-1, 0), 2), _fill(per_request, cap_long, (-1, 0, 0), 3)


def request_lists(lens, cap_long: int | None = None, cap_short: int | None = None, short_filler: int = 0) -> tuple[np.ndarray, np.ndarray]:
    """(requests with long portions, requests with short ones), int32 indices into the batch."""
    long_r = [b for b, n in enumerate(lens) if n > SHORT_PORTION]
    short_r = [b for b, n in enumerate(lens) if n <= SHORT_PORTION]
    return _fill(long_r, cap_long, len(lens) - 1, 1), _fill(short_r, cap_short, short_filler, 1)


@dataclass
class StepContext:
    """One step's batch as device tensors (all int32) plus a few host integers.

    The batch is a list of requests, each bringing a run of consecutive tokens
    (a portion of its prompt, or one decoded token).  Tokens of all requests lie
    back to back; `cu_seqlens[b] .. cu_seqlens[b+1]` are request b's tokens."""
    num_tokens: int
    num_requests: int
    max_len: int                         # longest run in this step (host); an upper bound in a padded step
    token_ids: torch.Tensor              # [T]
    positions: torch.Tensor              # [T]   absolute position of every token
    token_req: torch.Tensor              # [T]   index of the token's request in this batch
    cu_seqlens: torch.Tensor             # [B+1]
    start_pos: torch.Tensor              # [B]   tokens the request had before this step
    slots: torch.Tensor                  # [B]   the request's state slot
    block_tables: list[torch.Tensor]     # per page group: [B, pages] page ids
    slot_mappings: list[torch.Tensor]    # per page group: [T] token index into the group's page pool
    logit_rows: torch.Tensor             # [n] token indices whose logits are wanted
    cache: Any                           # the CacheManager
    max_context: int = 0                 # most keys any token of this step sees (host)
    attention_splits: int = 0            # fixed number of key ranges per context (0: chosen per call)
    host_lens: Any = None                # numpy [B]: tokens each request brings (None: unknown, treat all as short)
    host_starts: Any = None              # numpy [B]: tokens each request had before this step
    padding: Padding | None = None       # set for a step filled up to a bucket (see `Padding`)
    extras: dict = field(default_factory=dict)
    # work lists of a padded step: key -> (device tensors of fixed length, builder of their numpy content); the
    # planner fills them again for every step that is planned into this context
    fixed_lists: dict = field(default_factory=dict)

    # ---- work lists that kernels for long portions need; built on the host on first use, then cached
    @property
    def has_long_portions(self) -> bool:
        return self.host_lens is not None and self.max_len > SHORT_PORTION

    def _upload(self, array) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(array, dtype=np.int32)).to(self.token_ids.device, non_blocking=True)

    def _lists(self, key, build) -> tuple:
        """The device tensors of a work list.  `build()` gives its numpy arrays for the step as it stands.  In a padded
        step the tensors keep their place and length for every later step (`refresh_lists` fills them again)."""
        if self.padding is not None:
            if key not in self.fixed_lists:
                self.fixed_lists[key] = (tuple(self._upload(a) for a in build()), build)
            return self.fixed_lists[key][0]
        if key not in self.extras:
            self.extras[key] = tuple(self._upload(a) for a in build())
        return self.extras[key]

    def freeze_lists(self) -> None:
        """After the first run of a padded step: move the work lists it asked for into ONE device buffer, so that
        every later step fills them all with one copy from pinned memory.  The tensors that `_lists` hands out
        from now on are views of that buffer; a graph is captured only afterwards."""
        if "frozen" in self.extras or not self.fixed_lists:
            return
        sizes = [int(t.numel()) for tensors, _ in self.fixed_lists.values() for t in tensors]
        offsets = np.concatenate([[0], np.cumsum([(n + 3) // 4 * 4 for n in sizes])])
        total = max(int(offsets[-1]), 4)
        buf = torch.empty(total, dtype=torch.int32, device=self.token_ids.device)
        i = 0
        for key, (tensors, build) in list(self.fixed_lists.items()):
            views = []
            for t in tensors:
                v = buf[int(offsets[i]): int(offsets[i]) + sizes[i]].view(t.shape)
                v.copy_(t)
                views.append(v)
                i += 1
            self.fixed_lists[key] = (tuple(views), build)
        self.extras["frozen"] = {"buf": buf, "offsets": offsets, "sizes": sizes, "turn": 0, "events": [None, None],
                                 "pinned": [torch.empty(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]}

    def refresh_lists(self) -> None:
        """Fill the fixed work lists of a padded step for the requests it holds now (`host_lens`, `host_starts`)."""
        frozen = self.extras.get("frozen")
        arrays = [a for _, build in self.fixed_lists.values() for a in build()]
        if frozen is None:
            tensors = [t for ts, _ in self.fixed_lists.values() for t in ts]
            for t, a in zip(tensors, arrays):
                if t.numel() != a.size:
                    raise AssertionError("a fixed work list changed its length")
                t.copy_(torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).view(t.shape))
            return
        frozen["turn"] ^= 1
        turn = frozen["turn"]
        if frozen["events"][turn] is not None:
            frozen["events"][turn].synchronize()          # the copy that last read this pinned buffer
        host = frozen["pinned"][turn].numpy()
        for a, off, n in zip(arrays, frozen["offsets"][:-1], frozen["sizes"]):
            if a.size != n:
                raise AssertionError("a fixed work list changed its length")
            host[int(off): int(off) + n] = a.reshape(-1)
        frozen["buf"].copy_(frozen["pinned"][turn], non_blocking=True)
        ev = frozen["events"][turn] or torch.cuda.Event()
        ev.record()
        frozen["events"][turn] = ev

    def _first_dummy_single(self) -> tuple[int, int]:
        """(request index, token index) of the first dummy single token of a padded step."""
        b = self.padding.entries
        return b, int(np.sum(self.host_lens[:b]))

    def long_portion_tiles(self, tile: int) -> tuple[torch.Tensor, int]:
        """int32 [n, 2] on the device: (request index in the batch, first token within its portion) for
        every run of `tile` tokens of every portion longer than SHORT_PORTION, the tile that sees the
        most keys first (a causal tile's cost grows with its position)."""
        cap = None if self.padding is None else -(-self.num_tokens // tile) + self.padding.long_cap
        (t,) = self._lists(("tiles", tile), lambda: (tile_list(self.host_lens, self.host_starts, tile, cap),))
        return t, t.shape[0]

    def fork(self):
        """Mark this point of the caller's stream and return `run(work)`, or None where the step has no stream to spare.
        `run(work)` launches `work()` (kernels that depend only on what was launched before the mark) on a spare stream
        of the captured step (`extras["aux_streams"]`, set by the engine while it captures), beside whatever the caller
        has launched since the mark, and returns a function that makes the caller's stream wait for it.  Launch the
        chain that the step waits for first and the side work after it; the side work should take a grid that is
        resident at once, or its waiting CTAs take every SM slot before the chain's later kernels get one.  Whatever
        `work` reads or writes must stay alive until the join."""
        pool = self.extras.get("aux_streams")
        if not pool:
            return None
        turn = self.extras["aux_turn"] = (self.extras.get("aux_turn", -1) + 1) % len(pool)
        aux, cur = pool[turn], torch.cuda.current_stream()
        mark = torch.cuda.Event()
        mark.record(cur)

        def run(work):
            aux.wait_event(mark)
            with torch.cuda.stream(aux):
                work()
                done = torch.cuda.Event()
                done.record(aux)
            return lambda: cur.wait_event(done)
        return run

    def short_portion_tokens(self) -> tuple[torch.Tensor, int]:
        """int32 token indices (rows of this step's batch) of all portions of at most SHORT_PORTION tokens."""
        if self.padding is None:
            (t,) = self._lists("short_tokens", lambda: (short_token_list(self.host_lens),))
        else:
            (t,) = self._lists("short_tokens", lambda: (short_token_list(self.host_lens, self.padding.short_cap,
                                                                          self._first_dummy_single()[1]),))
        return t, t.shape[0]

    def long_portion_chunks(self, chunk: int) -> tuple[torch.Tensor, int, torch.Tensor, int]:
        """Work lists of a chunked scan over the long portions: int32 [n, 2] (request index, first token of
        the chunk within its portion) with its count, and int32 [m, 3] (request index, its first chunk,
        its number of chunks) with its count."""
        if self.padding is None:
            caps = (None, None)
        else:
            caps = (-(-self.num_tokens // chunk) + self.padding.long_cap, self.padding.long_cap)
        c, r = self._lists(("chunks", chunk), lambda: chunk_lists(self.host_lens, chunk, *caps))
        return c, c.shape[0], r, r.shape[0]

    def requests_by_portion(self) -> tuple[torch.Tensor, int, torch.Tensor, int]:
        """(long request indices, their count, short request indices, their count), int32 on the device."""
        if self.padding is None:
            build = lambda: request_lists(self.host_lens)
        else:
            build = lambda: request_lists(self.host_lens, self.padding.long_cap, min(self.padding.short_cap, self.num_requests),
                                          self._first_dummy_single()[0])
        lo, sh = self._lists("requests_by_portion", build)
        return lo, lo.shape[0], sh, sh.shape[0]
