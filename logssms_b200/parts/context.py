"""What a part sees of the running step and of the engine it runs in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

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


@dataclass
class StepContext:
    """One step's batch as device tensors (all int32) plus a few host integers.

    The batch is a list of requests, each bringing a run of consecutive tokens
    (a portion of its prompt, or one decoded token).  Tokens of all requests lie
    back to back; `cu_seqlens[b] .. cu_seqlens[b+1]` are request b's tokens."""
    num_tokens: int
    num_requests: int
    max_len: int                         # longest run in this step (host)
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
    extras: dict = field(default_factory=dict)

    # ---- work lists that kernels for long portions need; built on the host on first use, then cached
    @property
    def has_long_portions(self) -> bool:
        return self.host_lens is not None and self.max_len > SHORT_PORTION

    def _upload(self, array) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(array, dtype=np.int32)).to(self.token_ids.device, non_blocking=True)

    def long_portion_tiles(self, tile: int) -> tuple[torch.Tensor, int]:
        """int32 [n, 2] on the device: (request index in the batch, first token within its portion) for
        every run of `tile` tokens of every portion longer than SHORT_PORTION, the tile that sees the
        most keys first (a causal tile's cost grows with its position)."""
        key = ("tiles", tile)
        if key not in self.extras:
            pairs = [(b, t0) for b, n in enumerate(self.host_lens) if n > SHORT_PORTION for t0 in range(0, int(n), tile)]
            pairs.sort(key=lambda bt: -(int(self.host_starts[bt[0]]) + min(bt[1] + tile, int(self.host_lens[bt[0]]))))
            self.extras[key] = (self._upload(np.asarray(pairs, dtype=np.int32).reshape(-1, 2)), len(pairs))
        return self.extras[key]

    def short_portion_tokens(self) -> tuple[torch.Tensor, int]:
        """int32 token indices (rows of this step's batch) of all portions of at most SHORT_PORTION tokens."""
        key = "short_tokens"
        if key not in self.extras:
            cu = np.concatenate([[0], np.cumsum(self.host_lens)])
            idx = [t for b, n in enumerate(self.host_lens) if n <= SHORT_PORTION for t in range(int(cu[b]), int(cu[b + 1]))]
            self.extras[key] = (self._upload(np.asarray(idx, dtype=np.int32)), len(idx))
        return self.extras[key]

    def long_portion_chunks(self, chunk: int) -> tuple[torch.Tensor, int, torch.Tensor, int]:
        """Work lists of a chunked scan over the long portions: int32 [n, 2] (request index, first token of
        the chunk within its portion) with its count, and int32 [m, 3] (request index, its first chunk,
        its number of chunks) with its count."""
        key = ("chunks", chunk)
        if key not in self.extras:
            chunks, per_request = [], []
            for b, n in enumerate(self.host_lens):
                if n > SHORT_PORTION:
                    first = len(chunks)
                    chunks += [(b, t0) for t0 in range(0, int(n), chunk)]
                    per_request.append((b, first, len(chunks) - first))
            self.extras[key] = (self._upload(np.asarray(chunks, dtype=np.int32).reshape(-1, 2)), len(chunks),
                                self._upload(np.asarray(per_request, dtype=np.int32).reshape(-1, 3)), len(per_request))
        return self.extras[key]

    def requests_by_portion(self) -> tuple[torch.Tensor, int, torch.Tensor, int]:
        """(long request indices, their count, short request indices, their count), int32 on the device."""
        key = "requests_by_portion"
        if key not in self.extras:
            long_r = [b for b, n in enumerate(self.host_lens) if n > SHORT_PORTION]
            short_r = [b for b, n in enumerate(self.host_lens) if n <= SHORT_PORTION]
            self.extras[key] = (self._upload(np.asarray(long_r, dtype=np.int32)), len(long_r),
                                self._upload(np.asarray(short_r, dtype=np.int32)), len(short_r))
        return self.extras[key]
