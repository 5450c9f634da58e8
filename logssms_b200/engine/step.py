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

from typing import Sequence

import torch

from ..cache import CacheManager, RequestCache
from ..config import load_model_config
from ..models import build_model
from ..ops import kernels as K
from ..ops.profiler import PROFILER
from ..parts import Runtime
from ..weights import load_weights
from .plan import StaticTables, StepEntry, StepPlanner, bucket_for

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class Engine:
    """Model + weights + cache on one GPU, and the step function over them."""

    def __init__(self, model_dir: str, dtype="bfloat16", *, max_requests: int = 64, max_seq_len: int = 8192,
                 page_size: int = 64, num_pages: int | None = None, memory_ratio: float = 0.9,
                 device: str = "cuda:0", poison_on_free: bool = False, max_step_tokens: int = 1 << 30,
                 use_graphs: bool = True, max_graphs: int = 64, max_shape_graphs: int = 8, max_bucket_graphs: int = 32,
                 max_graph_tokens: int = 4096, profile: bool = False, nvtx: bool = False,
                 cuda_graph_max_bs: int | None = None, ssm_state_dtype: str = "float32"):
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
            # `ssm_state_dtype`: "float32" (the default), or "activation" to keep recurrent states in the model's dtype
            self.model.setup(Runtime(self.device, self.dtype, max_seq_len, page_size, {"ssm_state_dtype": ssm_state_dtype}))
        needs = self.model.cache_needs()
        if num_pages is None:
            num_pages = self._pages_that_fit(needs, max_requests, memory_ratio)
        self.cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                                  max_seq_len=max_seq_len, dtype=self.dtype, device=self.device,
                                  poison_on_free=poison_on_free, max_step_tokens=max_step_tokens)
        self.vocab_size = self.model.spec.vocab_size
        self.planner = StepPlanner(self.cache, self.device, self.vocab_size)
        # `profile`: every kernel between two CUDA events, summed per kernel class (`profile_report`); such steps run
        # kernel by kernel.  `nvtx`: named ranges per layer and part, for a timeline tool.
        # (one profiler per process: the engine made last decides)
        PROFILER.enabled, PROFILER.nvtx = bool(profile), bool(nvtx)
        if profile:
            PROFILER.reset()
        # `cuda_graph_max_bs` (the reference's --cuda-graph-max-bs / --graph, python/logssms/server/args.py:133-143): 0
        # switches all graphs off; a number is the largest decode batch that gets a graph, and `capture_decode_graphs`
        # captures the batch sizes 1, 2, 4, 8, 16, ... up to it ahead of the first request, as the reference does at
        # start (python/logssms/engine/decode_graph.py:52-68); None: every batch size, captured when it first comes twice
        self.cuda_graph_max_bs = cuda_graph_max_bs
        self.use_graphs = use_graphs and not profile and cuda_graph_max_bs != 0
        self.max_graphs = max_graphs
        self.max_shape_graphs = max_shape_graphs
        self.max_graph_tokens = max_graph_tokens
        self.max_bucket_graphs = max_bucket_graphs
        self._graphs: dict[int, _StepGraph] = {}             # decode steps, by batch size
        self._shape_graphs: dict[tuple, _StepGraph] = {}      # other steps, by (tokens of every entry, wanted places)
        self._bucket_graphs: dict[tuple, _StepGraph] = {}     # other steps filled up to a bucket of sizes, by bucket
        self._sightings: dict[tuple, int] = {}               # shapes seen once: (which kind of graph, key) -> count
        self._often: dict[tuple, int] = {}                   # how often a shape has gone through its bucket's graph
        self._decode_seen: dict[int, int] = {}               # ... and a decode batch size through a larger batch's graph
        # ... before it gets a graph of its own.  A graph of its own costs a shape three slow steps (two kernel by
        # kernel, one captured: tens of milliseconds on a deep model) and saves it the bucket's filling, a few per cent
        # of a step: it pays after dozens of replays.  (With 4, a serving run of 32 requests spent a third of its time
        # on such steps: a 512-token budget beside a changing number of decoding requests keeps making shapes that
        # come back a dozen times.)
        self.exact_after = 32
        self._side_stream: torch.cuda.Stream | None = None
        self._aux_streams: list | None = None
        self.steps_run = 0

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

    @property
    def h2d_bytes(self) -> int:
        """Bytes of step tables copied host -> device so far."""
        return self.planner.h2d_bytes

    # ------------------------------------------------------------------ requests
    def new_request(self, reserve_tokens: int = 0) -> RequestCache:
        return self.cache.admit(reserve_tokens)

    def release(self, request: RequestCache) -> None:
        self.cache.release(request)

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run the entries' tokens as one batch; return float32 logits [wanted, vocab] in the order
        of the entries and of each entry's `want`.

        `device_tokens` (int32 on the device, one per entry; decode steps only) replaces the entries' token
        ids: the ids sampled by the step before need not visit the host before they are fed back.

        Steps are replayed from CUDA graphs where their shape comes again.  A step of single decoded
        tokens that all want their logits has one graph per batch size, captured the second time that size
        is seen.  Any other step of at most `max_graph_tokens` tokens has one per shape (the number of tokens
        of every entry in order, and the number of wanted places), captured the third time the shape is seen:
        a long prompt cut into equal portions, or the same prompt length again.  The host then does nothing
        per kernel; a step whose shape is new runs kernel by kernel.  A replayed step returns the graph's own
        output buffer, valid until the next step of the same shape."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        if self.use_graphs:
            lens = tuple(len(e.tokens) for e in entries)
            if all(n == 1 for n in lens) and all(list(e.want) == [0] for e in entries):
                n = len(entries)
                if self.cuda_graph_max_bs is not None and n > self.cuda_graph_max_bs:
                    return self._run(self.planner.plan(entries), device_tokens)
                own = self._graphs.get(n)
                if own is None or own.graph is None:
                    # No graph of this batch size yet.  Until the size has come `exact_after` times it is replayed from
                    # the graph of the next larger batch that has one, filled up with dummy requests (the reference
                    # pads its decode batches to graph buckets the same way, python/logssms/engine/decode_graph.py:185-193):
                    # a graph of its own costs two slow steps.
                    seen = self._decode_seen[n] = self._decode_seen.get(n, 0) + 1
                    wider = min((b for b, g in self._graphs.items() if b > n and g.graph is not None and b <= max(2 * n, n + 8)),
                                default=None)
                    if wider is not None and seen <= self.exact_after:
                        return self._padded_decode(self._graphs[wider], wider, entries, device_tokens)
                return self._graph_step(self._graphs, n, self.max_graphs, 2, entries, device_tokens)
            if device_tokens is None and sum(lens) <= self.max_graph_tokens:
                # The graph of exactly this shape, if the shape has come before (no padding: a prompt length that
                # recurs, equal portions of a long prompt).  A shape that is new goes through the graph of its bucket:
                # the step filled up with dummy requests to round numbers of requests, tokens and work-list entries.
                wanted = sum(len(e.want) for e in entries)
                key = (lens, wanted)
                bucket = bucket_for(lens, wanted)
                # (the dummy portion that fills the bucket is a request like any other: it must fit the sequence limit)
                if bucket is not None and (bucket.tokens > self.max_graph_tokens + 256
                                           or bucket.tokens - sum(lens) > self.max_seq_len):
                    bucket = None
                often = self._often.get(key, 0) + 1
                if key not in self._shape_graphs and bucket is not None and often <= self.exact_after:
                    # (a graph of its own costs a shape two slow steps, one kernel by kernel and one captured: that pays
                    # only for a shape that keeps coming)
                    self._often.pop(key, None)
                    self._often[key] = often
                    while len(self._often) > 256:
                        self._often.pop(next(iter(self._often)))
                    logits = self._graph_step(self._bucket_graphs, bucket, self.max_bucket_graphs, 2, entries, None, bucket)
                    return logits[:wanted]
                return self._graph_step(self._shape_graphs, key, self.max_shape_graphs, 3, entries, None)
        return self._run(self.planner.plan(entries), device_tokens)

    def capture_decode_graphs(self, sizes: Sequence[int] | None = None) -> list[int]:
        """Capture the decode graphs of these batch sizes now (default: 1, 2, 4, 8, 16, 24, ... up to
        `cuda_graph_max_bs`, or up to the number of request rows), with requests made for the purpose that decode a few
        dummy tokens and are released again.  A server calls this before its first request so that no request pays for
        a capture; without the call every batch size is captured when it comes for the second time.  Returns the sizes
        that now have a graph."""
        if not self.use_graphs:
            return []
        most = min(self.cuda_graph_max_bs or self.cache.max_requests, self.cache.max_requests, self.max_graphs)
        if sizes is None:
            sizes = [b for b in [1, 2, 4] + list(range(8, most + 1, 8)) if b <= most]
        done = []
        for n in sizes:
            slot = self._graphs.get(n)
            if n < 1 or n > most or (slot is not None and slot.graph is not None):
                continue
            if self.cache.rows.num_free < n or not self.cache.can_admit(4 * n):
                break
            requests = [self.cache.admit(4) for _ in range(n)]
            try:
                for _ in range(3):                       # kernel by kernel, captured, replayed
                    with torch.inference_mode():
                        self._graph_step(self._graphs, n, self.max_graphs, 2, [StepEntry(r, [0], [0]) for r in requests], None)
                torch.cuda.synchronize(self.device)
            finally:
                for r in requests:
                    self.cache.release(r)
            if self._graphs.get(n) is not None and self._graphs[n].graph is not None:
                done.append(n)
        return done

    # ------------------------------------------------------------------ a decode step planned ahead
    @torch.inference_mode()
    def prepare(self, entries: Sequence[StepEntry]):
        """Plan a step of single decoded tokens before their ids are known: the caches grow, the step's tables go to
        the device (behind whatever still runs there), and only the ids are missing.  `run_prepared` then costs the
        host one small copy and one graph launch.  Returns a handle, or None where planning ahead is not on offer (no
        captured graph of this batch size yet, other shapes of step): then `step` does it all.  A handle that is not
        run is simply dropped; its entries must then come again with `start` set (see `StepEntry`)."""
        if not self.use_graphs or not entries:
            return None
        if any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return None
        slot = self._graphs.get(len(entries))
        if slot is None or slot.graph is None:
            return None
        self._graphs[len(entries)] = self._graphs.pop(len(entries))       # most recently used last
        self.planner.plan(entries, slot)
        return (slot, len(entries))

    @torch.inference_mode()
    def run_prepared(self, handle, token_ids: torch.Tensor) -> torch.Tensor:
        """Run the step that `prepare` planned on these ids (int32, one per entry, pinned host or device memory)."""
        slot, n = handle
        if token_ids.numel() != n or token_ids.dtype != torch.int32:
            raise ValueError("run_prepared takes one int32 id per prepared entry")
        slot.ctx.token_ids.copy_(token_ids, non_blocking=True)
        if not token_ids.is_cuda:
            self.planner.h2d_bytes += n * 4
        slot.seen += 1
        slot.graph.replay()
        K.launch_count += slot.launches
        self.steps_run += 1
        return slot.logits

    def _padded_decode(self, slot, size: int, entries: Sequence[StepEntry], device_tokens) -> torch.Tensor:
        """A decode step of fewer requests than `size` through the captured graph of that size."""
        n = len(entries)
        self._graphs[size] = self._graphs.pop(size)        # most recently used last
        ctx = self.planner.plan(entries, slot, pad_singles=size - n)
        if device_tokens is not None:
            if device_tokens.numel() != n:
                raise ValueError("device_tokens feeds steps of one token per entry only")
            ctx.token_ids[:n].copy_(device_tokens)
        slot.seen += 1
        slot.graph.replay()
        K.launch_count += slot.launches
        self.steps_run += 1
        return slot.logits[:n]

    def _run(self, ctx, device_tokens: torch.Tensor | None) -> torch.Tensor:
        """The planned step, kernel by kernel."""
        if device_tokens is not None:
            if ctx.num_tokens != ctx.num_requests or device_tokens.numel() != ctx.num_tokens:
                raise ValueError("device_tokens feeds steps of one token per entry only")
            ctx.token_ids.copy_(device_tokens)
        x, residual = self.model.forward(ctx)
        self.steps_run += 1
        PROFILER.steps += PROFILER.enabled
        if ctx.logit_rows.numel() == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.logits(x, residual, ctx.logit_rows)

    def profile_report(self) -> dict:
        """Device time per kernel class and per kernel since the engine started (needs `profile=True`)."""
        return PROFILER.report()

    def _graph_step(self, graphs: dict, key, most: int, capture_at: int, entries: Sequence[StepEntry],
                    device_tokens: torch.Tensor | None, bucket=None) -> torch.Tensor:
        """A step through the graph of its shape.  First sight: kernel by kernel with tables of its own (this
        also builds and loads every kernel).  From the second on its tables lie in the slot's fixed buffer;
        until `capture_at` it still runs kernel by kernel (which builds the work lists that long portions need,
        outside of any capture), then it is captured once and replayed."""
        slot = graphs.get(key)
        if slot is None and bucket is not None:
            # a bucket serves many shapes: it takes its slot (and its fixed tables) at first sight, and its first
            # step runs kernel by kernel on them, which also tells which work lists the model asks for
            if len(graphs) >= most:
                victim = next((k for k, g in graphs.items() if g.graph is None), next(iter(graphs)))
                graphs.pop(victim)
            slot = graphs[key] = _StepGraph()
        elif slot is None:
            # A shape takes a slot (fixed tables on the device, later a graph) only when it comes a second time:
            # until then it is a count in a bounded list, so that shapes that never recur cost no device memory
            # and push no captured graph out.
            seen = self._sightings.pop((id(graphs), key), 0) + 1
            if seen < 2:
                self._sightings[(id(graphs), key)] = seen
                while len(self._sightings) > 64:
                    self._sightings.pop(next(iter(self._sightings)))
                return self._run(self.planner.plan(entries), device_tokens)
            if len(graphs) >= most:
                # room: a slot that holds no graph yet goes first, then the graph used longest ago
                victim = next((k for k, g in graphs.items() if g.graph is None), next(iter(graphs)))
                graphs.pop(victim)
            slot = graphs[key] = _StepGraph()
            slot.seen = seen - 1
        else:
            graphs[key] = graphs.pop(key)                 # most recently used last
        slot.seen += 1
        if slot.graph is None and slot.seen < capture_at:
            ctx = self.planner.plan(entries, slot, bucket)
            logits = self._run(ctx, device_tokens)
            if bucket is not None:
                ctx.freeze_lists()
            return logits
        ctx = self.planner.plan(entries, slot, bucket)
        if device_tokens is not None:
            ctx.token_ids.copy_(device_tokens)            # before the capture / replay, on the same stream
        if slot.graph is None:
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = K.launch_count
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(self.device)
            # blocks may fork their mixers onto a second stream while capturing (measured: without it a batch-8 decode
            # step takes 30 % longer, a 2,048-token prompt 8.3 instead of 6.4 ms)
            ctx.extras["side_stream"] = self._side_stream
            # ... and a part may put work of its own beside the rest of its branch (`StepContext.fork`)
            if self._aux_streams is None:
                self._aux_streams = [torch.cuda.Stream(self.device) for _ in range(2)]
            ctx.extras["aux_streams"] = self._aux_streams
            with torch.cuda.graph(graph):
                x, residual = self.model.forward(ctx)
                if ctx.logit_rows.numel() == 0:
                    slot.logits = torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
                else:
                    slot.logits = self.model.logits(x, residual, ctx.logit_rows)
            ctx.extras.pop("side_stream", None)
            ctx.extras.pop("aux_streams", None)
            ctx.extras.pop("aux_turn", None)
            slot.launches = K.launch_count - before
            K.launch_count = before
            slot.graph = graph
        slot.graph.replay()
        K.launch_count += slot.launches
        self.steps_run += 1
        return slot.logits

class _StepGraph(StaticTables):
    """A captured step of one shape: its table buffer on the device, the step context whose tensors are
    views of that buffer, the graph, and the logits it writes."""

    def __init__(self):
        super().__init__()
        self.seen = 0
        self.graph = None
        self.logits: torch.Tensor | None = None
        self.launches = 0
