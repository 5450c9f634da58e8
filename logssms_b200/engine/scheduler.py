"""The scheduler above the step function: admit, cut prompts into portions, decode, finish, free.

Rules (the reference's, python/logssms/scheduler/prefill.py:94-152 and :294-324,
python/logssms/scheduler/scheduler.py:194-205 and :264-319, python/logssms/scheduler/ar.py:114-117):

  * Admission is first-come-first-served and stops at the first request that does not fit; nobody
    overtakes.  A request fits when a request row is free and every page group can set aside the
    pages of its whole life (prompt + max_tokens).  Pages are reserved at admission, so a running
    request can never run out of pages; there is no preemption and no swapping.
  * What happens when pages run out: waiting requests wait until finished requests give pages
    back.  A request that could not fit even into an empty pool, or whose prompt does not leave room
    for one new token within max_seq_len, is finished at once with reason "rejected".
    `max_tokens` is clamped so that prompt + max_tokens <= max_seq_len.
  * Policy "mixed" (the default here): every step takes one token from each decoding request, then
    fills what is left of the token budget (`max_step_tokens`) with prompt portions, oldest request
    first; a prompt that does not fit is cut at the budget, anywhere, and goes on in the next step.
    `mixed_prefill_tokens` (the reference's `--mixed-prefill-tokens`) caps the prompt tokens of a step
    that also decodes, so that the decoding requests' step time stays short.
  * Policy "prefill-first" (the reference's default, `--scheduling-policy`): a step is either prompt
    portions or decoded tokens, and prompts win: while any prompt portion can run, the decoding
    requests wait.
  * A request ends after `max_tokens` new tokens or at an end-of-sequence token (unless
    `ignore_eos`); its row, pages and state slot go back at once.
  * Host and device overlap in the steady state of decoding: sampled ids are copied to pinned host memory
    without waiting, and while the same requests go on decoding the next step is launched from the ids
    still on the device before the host reads the previous ones.  A request that ends at an end-of-sequence
    token is then noticed one step late: the step that was already launched for it is discarded (the
    reference finishes such requests one step late as well, python/logssms/scheduler/scheduler.py:164-180).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Iterable, Sequence

import torch

from ..cache import OutOfPages
from ..sampling import Sampler, SamplingParams
from .step import StepEntry

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass(eq=False)
class Request:
    number: int
    prompt: list[int]
    params: SamplingParams
    max_tokens: int                      # after clamping
    state: str = WAITING
    cache: object | None = None          # RequestCache while running
    computed: int = 0                    # tokens (prompt and generated) that have gone through the model
    output: list[int] = field(default_factory=list)
    finish_reason: str | None = None
    seed: int = 0

    @property
    def prompt_done(self) -> bool:
        return self.computed >= len(self.prompt)

    @property
    def total_len(self) -> int:
        return len(self.prompt) + self.max_tokens


@dataclass
class _InFlight:
    """Sampled ids of a step that the host has not read yet."""
    requests: list
    tokens: torch.Tensor          # int32 on the device, one per request
    pinned: torch.Tensor          # their copy in pinned host memory (valid after `event`)
    event: "torch.cuda.Event | None"      # None: the ids are already on the host (a sampler that runs there)
    has_status: bool = False      # pinned[len(requests)] holds the device's kernel error word as the step left it


@dataclass
class StepDecision:
    """What one step runs: (request, first token index, number of tokens, sample afterwards?)."""
    decodes: list[Request]
    portions: list[tuple[Request, int, int, bool]]

    @property
    def num_tokens(self) -> int:
        return len(self.decodes) + sum(n for _, _, n, _ in self.portions)


class Scheduler:
    POLICIES = ("mixed", "prefill-first")

    def __init__(self, engine, *, max_step_tokens: int = 8192, sampler=None, eos_token_ids: Iterable[int] = (),
                 policy: str = "mixed", mixed_prefill_tokens: int | None = None):
        if max_step_tokens < 1:
            raise ValueError("max_step_tokens must be at least 1")
        if policy not in self.POLICIES:
            raise ValueError(f"unknown scheduling policy {policy!r}: one of {', '.join(self.POLICIES)}")
        if mixed_prefill_tokens is not None and mixed_prefill_tokens < 1:
            raise ValueError("mixed_prefill_tokens must be at least 1")
        self.policy = policy
        self.mixed_prefill_tokens = mixed_prefill_tokens
        self.engine = engine
        self.cache = engine.cache
        self.max_step_tokens = max_step_tokens
        self.sampler = sampler if sampler is not None else Sampler(engine.device)
        self.eos = frozenset(eos_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._count = 0
        self.steps = 0
        self.d2h_bytes = 0
        self._inflight: _InFlight | None = None
        self._pinned: list[torch.Tensor] = []
        self.overlap = True           # launch the next decode step before reading the previous step's ids
        # without overlap (every id visits the host before it is fed back): the next decode step planned while the
        # device still runs this one, (handle, requests); and the pinned buffer its ids go through
        self._ahead: tuple | None = None
        self.steps_ahead = 0          # steps that ran from a plan made ahead
        self._ids_pinned: torch.Tensor | None = None

    # ------------------------------------------------------------------ intake
    def add_request(self, prompt: Sequence[int], params: SamplingParams | None = None) -> Request:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        max_seq = self.cache.max_seq_len
        req = Request(self._count, prompt, params, max(0, min(params.max_tokens, max_seq - len(prompt))))
        req.seed = self.sampler.seed_for(params, req.number) if hasattr(self.sampler, "seed_for") else 0
        self._count += 1
        if not prompt:
            return self._finish(req, "rejected: empty prompt")
        if len(prompt) >= max_seq:
            return self._finish(req, f"rejected: prompt of {len(prompt)} tokens leaves no room within max_seq_len {max_seq}")
        if req.max_tokens == 0:
            return self._finish(req, "length")
        if not self.cache.fits_at_all(req.total_len):
            return self._finish(req, f"rejected: {req.total_len} tokens can never fit the page pool")
        self.waiting.append(req)
        return req

    # ------------------------------------------------------------------ one step
    def schedule(self) -> StepDecision:
        decodes = [r for r in self.running if r.prompt_done]
        if self.policy == "prefill-first":
            budget = self.max_step_tokens               # the whole step for prompts, if there are any
        else:
            budget = self.max_step_tokens - len(decodes)
            if decodes and self.mixed_prefill_tokens is not None:
                budget = min(budget, self.mixed_prefill_tokens)
        portions: list[tuple[Request, int, int, bool]] = []

        def give_portion(r: Request) -> None:
            nonlocal budget
            left = len(r.prompt) - r.computed
            n = min(left, budget)
            if n > 0:
                portions.append((r, r.computed, n, n == left))
                budget -= n

        for r in self.running:                       # prompts already under way, oldest first
            if not r.prompt_done and budget > 0:
                give_portion(r)
        while self.waiting and budget > 0:           # then newcomers, in arrival order, no overtaking
            r = self.waiting[0]
            if not self.cache.can_admit(r.total_len):
                break
            self.waiting.popleft()
            r.cache = self.cache.admit(r.total_len)
            r.state = RUNNING
            self.running.append(r)
            give_portion(r)
        if self.policy == "prefill-first":
            return StepDecision([], portions) if portions else StepDecision(decodes, [])
        return StepDecision(decodes, portions)

    def step(self) -> list[Request]:
        """Run one step; return the requests that are known to have finished since the last call."""
        inflight = self._inflight
        if inflight is not None and self.overlap and inflight.event is not None and self._goes_on(inflight):
            # the same requests decode on: launch their next step from the ids on the device, then read the previous ids
            reqs = inflight.requests
            logits = self.engine.step([StepEntry(r.cache, [0], [0], r.computed) for r in reqs], device_tokens=inflight.tokens)
            self.steps += 1
            for r in reqs:
                r.computed += 1
            self._inflight = self._sample(logits, reqs, pending=1)
            return self._read(inflight)
        done = self._read(inflight) if inflight is not None else []
        self._inflight = None
        ahead, self._ahead = self._ahead, None
        if ahead is not None and self._still_right(ahead[1]):
            # the step was planned while the last one ran: its ids go to the device, nothing else is left to do
            handle, reqs = ahead
            n = len(reqs)
            if self._ids_pinned is None or self._ids_pinned.numel() < n:
                self._ids_pinned = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=self.engine.device.type == "cuda")
            self._ids_pinned.numpy()[:n] = [r.output[-1] for r in reqs]
            logits = self.engine.run_prepared(handle, self._ids_pinned[:n])
            self.steps += 1
            self.steps_ahead += 1
            for r in reqs:
                r.computed += 1
            return done + self._after_step(logits, reqs)
        decision = self.schedule()
        if decision.num_tokens == 0:
            if self.waiting and not self.running:
                raise RuntimeError("scheduler is stuck: requests wait but nothing runs and nothing fits")
            return done
        entries, sampled = [], []
        for r in decision.decodes:
            entries.append(StepEntry(r.cache, [r.output[-1]], [0], r.computed))
            sampled.append(r)
        for r, first, n, last in decision.portions:
            entries.append(StepEntry(r.cache, r.prompt[first:first + n], [n - 1] if last else [], r.computed))
            if last:
                sampled.append(r)
        logits = self.engine.step(entries)
        self.steps += 1
        for r in decision.decodes:
            r.computed += 1
        for r, _, n, _ in decision.portions:
            r.computed += n
        if sampled:
            done += self._after_step(logits, sampled)
        return done

    def _after_step(self, logits: torch.Tensor, sampled: list) -> list[Request]:
        """Sample; then either leave the ids in flight (overlap), or read them at once, after planning the next
        decode step while the device still works on this one."""
        self._inflight = self._sample(logits, sampled, pending=0)
        goes_on = self._goes_on(self._inflight)
        if self.overlap and goes_on and self._inflight.event is not None:
            return []
        if goes_on and hasattr(self.engine, "prepare"):
            try:
                handle = self.engine.prepare([StepEntry(r.cache, [0], [0], r.computed) for r in sampled])
            except OutOfPages:                             # (requests that reserved their pages never meet this)
                handle = None
            if handle is not None:
                self._ahead = (handle, list(sampled))
        inflight, self._inflight = self._inflight, None
        return self._read(inflight)                        # nothing to overlap with: read at once

    def _still_right(self, reqs: list) -> bool:
        """Does the step that was planned ahead for `reqs` still stand: the same requests decode on, nobody new can
        come in?  (Else it is dropped: its entries are planned again at their positions, which grows nothing twice.)"""
        if len(reqs) != len(self.running) or any(r is not q or r.state != RUNNING for r, q in zip(reqs, self.running)):
            return False
        if any(len(r.output) >= r.max_tokens for r in reqs):
            return False
        return not (self.waiting and self.cache.can_admit(self.waiting[0].total_len))

    def _sample(self, logits: torch.Tensor, reqs: list, pending: int) -> _InFlight:
        """Sample one id per request and start its copy to pinned host memory; nobody waits here."""
        # a sampler that `reports_kernel_errors` appends the device's kernel error word to the ids, so that the word
        # reaches the host in the copy that is made anyway (a kernel whose bounded wait gave up leaves it non-zero)
        status = bool(getattr(self.sampler, "reports_kernel_errors", False))
        args = (logits, [r.params for r in reqs], [r.seed for r in reqs], [len(r.output) + pending for r in reqs])
        tokens = self.sampler.sample(*args, with_status=True) if status else self.sampler.sample(*args)
        n = len(reqs)
        if not tokens.is_cuda:
            return _InFlight(list(reqs), tokens, tokens, None)
        m = tokens.numel()
        pinned = self._pinned.pop() if self._pinned else None
        if pinned is None or pinned.numel() < m:
            pinned = torch.empty(max(m, 256), dtype=torch.int32, pin_memory=True)
        pinned[:m].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return _InFlight(list(reqs), tokens[:n], pinned, event, has_status=status and m == n + 1)

    def _goes_on(self, inflight: _InFlight) -> bool:
        """Will the next step be exactly one more token for each of these requests, whatever their pending ids
        turn out to be (an end-of-sequence id aside)?  Then it can be launched before they are read."""
        if self.waiting and self.cache.can_admit(self.waiting[0].total_len):
            return False
        decoding = [r for r in self.running if r.prompt_done]
        if len(decoding) != len(self.running) or len(decoding) != len(inflight.requests):
            return False
        for r, q in zip(decoding, inflight.requests):
            if r is not q or r.state != RUNNING or len(r.output) + 2 > r.max_tokens:
                return False               # the pending id is this request's last: read it first
        return True

    def _read(self, inflight: _InFlight) -> list[Request]:
        """Wait for a step's ids, hand them to their requests, finish those that end."""
        n = len(inflight.requests)
        if inflight.event is not None:
            inflight.event.synchronize()
            self._pinned.append(inflight.pinned)
        ids = inflight.pinned[:n].tolist()
        self.d2h_bytes += (n + inflight.has_status) * 4
        if inflight.has_status and int(inflight.pinned[n]) != 0:
            # a kernel of that step (or of one since) gave up on a wait: its logits, and these ids, mean nothing
            code = int(inflight.pinned[n])
            later, self._inflight = self._inflight, None
            for r in {*inflight.requests, *(later.requests if later is not None else ())}:
                if r.state != FINISHED:
                    self._finish(r, "error: a kernel gave up on a wait")
            from ..ops import kernels as K
            K.raise_kernel_error(code, self.engine.device)
        done: list[Request] = []
        for r, tok in zip(inflight.requests, ids):
            if r.state == FINISHED:
                continue                   # ended one step ago (end-of-sequence id, abort): this id is discarded
            r.output.append(int(tok))
            if int(tok) in self.eos and not r.params.ignore_eos:
                done.append(self._finish(r, "stop"))
            elif len(r.output) >= r.max_tokens:
                done.append(self._finish(r, "length"))
        return done

    def drain(self) -> list[Request]:
        """Read what is still in flight (end of a run, or before the caller looks at the outputs)."""
        inflight, self._inflight = self._inflight, None
        return self._read(inflight) if inflight is not None else []

    def abort(self, req: Request) -> None:
        if req.state == WAITING:
            self.waiting.remove(req)
        if req.state != FINISHED:
            self._finish(req, "abort")

    def _finish(self, req: Request, reason: str) -> Request:
        if req.cache is not None:
            self.cache.release(req.cache)
            req.cache = None
        if req in self.running:
            self.running.remove(req)
        req.state, req.finish_reason = FINISHED, reason
        self.finished.append(req)
        return req

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    def run(self) -> None:
        while self.has_work:
            self.step()
        self.drain()
