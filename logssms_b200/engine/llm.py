"""The Python entry point: `LLM(model_path, ...).generate(prompts, sampling_params)`.

The reference has no in-process entry point (its tests pump the scheduler by hand,
tests/mtp/test_mtp_e2e.py:63-127); this one wraps engine + scheduler + sampler and keeps the
reference's option names where it has them (python/logssms/server/args.py:60-251).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Sequence

from ..sampling import Sampler, SamplingParams
from .scheduler import Scheduler
from .step import Engine


@dataclass
class Output:
    token_ids: list[int]
    finish_reason: str
    text: str | None = None
    prompt_token_ids: list[int] | None = None


class LLM:
    def __init__(self, model_path: str, dtype: str = "bfloat16", *, max_running_requests: int = 64,
                 max_seq_len_override: int | None = None, page_size: int = 64, num_pages: int | None = None,
                 memory_ratio: float = 0.9, max_prefill_tokens: int = 8192, seed: int = 0,
                 device: str = "cuda:0", tokenizer=None, eos_token_ids: Sequence[int] | None = None,
                 poison_on_free: bool = False, use_graphs: bool = True, scheduling_policy: str = "mixed",
                 mixed_prefill_tokens: int | None = None, profile: bool = False, nvtx: bool = False,
                 cuda_graph_max_bs: int | None = None, ssm_state_dtype: str = "float32"):
        from ..config import load_model_config
        config = load_model_config(model_path)
        max_seq_len = max_seq_len_override or min(getattr(config, "max_position_embeddings", 8192), 8192)
        if dtype == "auto":
            dtype = "float32" if getattr(config, "torch_dtype", "bfloat16") == "float32" else "bfloat16"
        self.engine = Engine(model_path, dtype, max_requests=max_running_requests, max_seq_len=max_seq_len,
                             page_size=page_size, num_pages=num_pages, memory_ratio=memory_ratio, device=device,
                             poison_on_free=poison_on_free, max_step_tokens=max_prefill_tokens, use_graphs=use_graphs,
                             profile=profile, nvtx=nvtx, cuda_graph_max_bs=cuda_graph_max_bs,
                             ssm_state_dtype=ssm_state_dtype)
        if cuda_graph_max_bs:
            # asked for by size: the decode graphs are captured now, before the first request (as the reference does)
            self.engine.capture_decode_graphs()
        self.tokenizer = tokenizer if tokenizer is not None else _maybe_tokenizer(model_path)
        if eos_token_ids is None:
            eos = getattr(self.tokenizer, "eos_token_id", None) if self.tokenizer is not None else None
            eos_token_ids = [] if eos is None else [eos]
        self.sampler = Sampler(self.engine.device, seed)
        self.scheduler = Scheduler(self.engine, max_step_tokens=max_prefill_tokens, sampler=self.sampler,
                                   eos_token_ids=eos_token_ids, policy=scheduling_policy,
                                   mixed_prefill_tokens=mixed_prefill_tokens)

    # ------------------------------------------------------------------ step-wise use
    def add_request(self, prompt_ids: Sequence[int], sampling_params: SamplingParams | None = None):
        """Queue one prompt (token ids); returns the scheduler's `Request`, whose `output` grows as
        `step()` is called."""
        return self.scheduler.add_request(prompt_ids, sampling_params)

    def step(self):
        """Run one scheduled step (prompt portions and one token of every decoding request); returns
        the requests that finished in it.  In the steady state of decoding the sampled ids are fed back on the
        device and read by the host one step late (`scheduler.overlap`; switch it off to have every step's ids
        visit the host before the next step is launched from them)."""
        return self.scheduler.step()

    def abort(self, request) -> None:
        self.scheduler.abort(request)

    @property
    def d2h_bytes(self) -> int:
        """Bytes of sampled token ids read back to the host so far."""
        return self.scheduler.d2h_bytes

    def generate(self, prompts, sampling_params: SamplingParams | Sequence[SamplingParams] | None = None) -> list[Output]:
        """`prompts`: a list of token-id lists, or of strings when the model folder has a tokenizer.
        Returns one `Output` per prompt, in order."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt")
        ids = []
        for p in prompts:
            if isinstance(p, str):
                if self.tokenizer is None:
                    raise ValueError("text prompts need a tokenizer in the model folder; pass token ids instead")
                ids.append(list(self.tokenizer.encode(p)))
            else:
                ids.append(list(p))
        requests = [self.scheduler.add_request(i, sp) for i, sp in zip(ids, sampling_params)]
        self.scheduler.run()
        outs = []
        for r in requests:
            text = self.tokenizer.decode(r.output) if self.tokenizer is not None else None
            outs.append(Output(list(r.output), r.finish_reason or "", text, r.prompt))
        return outs


def _maybe_tokenizer(model_path: str):
    if not any(os.path.isfile(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer.model")):
        return None
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(model_path)
