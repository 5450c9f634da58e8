"""What a part sees of the running step and of the engine it runs in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


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
    extras: dict = field(default_factory=dict)
