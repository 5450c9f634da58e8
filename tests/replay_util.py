"""Building traces for bin/trace_run, running it, and collecting logits per request and position."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from dataclasses import dataclass, field

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")
PAGE = 64


@dataclass
class Trace:
    """Steps for trace_run plus the bookkeeping to map its output rows back to (request, position)."""
    steps: list[dict] = field(default_factory=list)
    rows: list[list[tuple[str, int]]] = field(default_factory=list)     # per step: (request id, position) per wanted row
    progress: dict[str, int] = field(default_factory=dict)
    peak_tokens: int = 0
    page: int = PAGE                     # tokens per page of the engine that will replay this (for `peak_tokens`)
    _live: dict[str, int] = field(default_factory=dict)

    def add_step(self, portions: list[tuple[str, list[int]]], end: list[str] = (), want_all: bool = True) -> None:
        entries, rows = [], []
        for rid, tokens in portions:
            start = self.progress.get(rid, 0)
            want = list(range(len(tokens))) if want_all else [len(tokens) - 1]
            entries.append({"id": rid, "tokens": list(tokens), "want": want})
            rows += [(rid, start + w) for w in want]
            self.progress[rid] = start + len(tokens)
            self._live[rid] = self.progress[rid]
        self.peak_tokens = max(self.peak_tokens, sum(-(-n // self.page) * self.page for n in self._live.values()))
        for rid in end:
            self._live.pop(rid, None)
            self.progress.pop(rid, None)
        self.steps.append({"step": len(self.steps), "entries": entries, "end": list(end)})
        self.rows.append(rows)


def whole(trace: Trace, rid: str, ids: list[int]) -> None:
    trace.add_step([(rid, ids)], end=[rid])


def tail_decoded(trace: Trace, rid: str, ids: list[int], tail: int = 32) -> None:
    head = max(len(ids) - tail, 1)
    trace.add_step([(rid, ids[:head])])
    for i in range(head, len(ids)):
        trace.add_step([(rid, ids[i:i + 1])], end=[rid] if i == len(ids) - 1 else [])
    if head == len(ids):
        trace.add_step([], end=[rid])


def in_portions(trace: Trace, rid: str, ids: list[int], sizes: list[int]) -> None:
    p, i = 0, 0
    while p < len(ids):
        n = min(sizes[i % len(sizes)], len(ids) - p)
        trace.add_step([(rid, ids[p:p + n])], end=[rid] if p + n == len(ids) else [])
        p += n
        i += 1


def mixed(trace: Trace, requests: dict[str, list[int]], max_tokens: int, seed: int, max_live: int = 4,
          prompt_fraction: float = 0.6) -> None:
    """Up to `max_live` requests at a time: portions of some prompts beside single decoded tokens of
    others, a request now and then left out of a step, new requests arriving as room appears."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    rounded = lambda n: -(-n // PAGE) * PAGE
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting[0]
            if sum(rounded(len(requests[r])) for r in live) + rounded(len(ids)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = {"ids": ids, "done": 0, "prompt": max(1, int(len(ids) * prompt_fraction))}
            if rng.random() < 0.5:
                break                                    # staggered arrivals
        portions, ended = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.15:
                continue                                 # left out of this step, goes on later
            left_prompt = st["prompt"] - st["done"]
            if left_prompt > 0:
                n = min(left_prompt, rng.choice([2, 3, 5, 8, 17, 40, 64, 70]))
                if left_prompt - n == 1:
                    n += 1                               # never leave a one-token prompt portion behind
            else:
                n = 1
            portions.append((rid, st["ids"][st["done"]:st["done"] + n]))
            st["done"] += n
            if st["done"] == len(st["ids"]):
                ended.append(rid)
                del live[rid]
        if portions:
            trace.add_step(portions, end=ended)


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int, vocab: int,
              extra_args=(), env=None, python=sys.executable) -> dict[str, torch.Tensor]:
    """Run bin/trace_run over the trace; return request id -> float32 [positions, vocab] (NaN where
    nothing was asked).  A request id that is used again after its end gets a fresh entry only if the
    caller gave it a new id; traces here always use unique ids."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [python, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens),
           *extra_args]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for step in trace.steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {step['step']}", f"trace_run answered {line!r} to step {step['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=300) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    lengths: dict[str, int] = {}
    for rows in trace.rows:
        for rid, pos in rows:
            lengths[rid] = max(lengths.get(rid, 0), pos + 1)
    out = {rid: torch.full((n, vocab), float("nan")) for rid, n in lengths.items()}
    for step, rows in zip(trace.steps, trace.rows):
        path = os.path.join(out_dir, f"{step['step']}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        data = np.fromfile(path, dtype="<f4").reshape(len(rows), vocab)
        for (rid, pos), row in zip(rows, data):
            out[rid][pos] = torch.from_numpy(row.copy())
    return out
