"""Whole-model logits of the unmodified reference on tiny random Falcon-H1 models, for `tests/test_plain.py`.

Run once on a machine with a GPU and the reference installed under `baseline/_ref` (the same install the benchmark's
reference arm uses): `python tests/golden/make_reference_model_golden.py`.  It writes
`tests/golden/reference_model_<name>.safetensors` (prompt ids, the reference's greedy tokens and the logits it
sampled them from) for every configuration below; the weights are not stored, `tests/tiny.make_model_dir` makes
them again from the seed.

The reference runs as it does in the benchmark: its own `Scheduler` and `Engine` through their public constructors
and `overlap_loop` (python/logssms/scheduler/scheduler.py), real weights read by its own loader
(python/logssms/models/weight.py), bfloat16, default cache type, attention backend and graphs.  One request at a
time, greedy: every call of the engine's sampling step then holds one row of logits, the last prompt position
first (after one call per earlier portion of a prompt that is cut) and one decoded token per call after it.  Only that one bound method of the engine OBJECT is wrapped here to
copy the logits out; no file of the reference is changed.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

# sizes the reference's own kernels take (heads of 64, 128-token chunks), every multiplier and option off its default
_BASE = {
    "architectures": ["FalconH1ForCausalLM"], "model_type": "falcon_h1",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 384, "vocab_size": 1024, "rms_norm_eps": 1e-5, "max_position_embeddings": 2048,
    "rope_theta": 1e11, "tie_word_embeddings": True,
    "mamba_d_ssm": 256, "mamba_n_heads": 4, "mamba_d_head": 64, "mamba_d_state": 128, "mamba_n_groups": 1,
    "mamba_d_conv": 4, "mamba_chunk_size": 128, "mamba_conv_bias": True, "mamba_proj_bias": False,
    "projectors_bias": False, "mamba_rms_norm": False, "mamba_norm_before_gate": False,
    "embedding_multiplier": 5.0, "lm_head_multiplier": 0.25, "attention_in_multiplier": 1.5,
    "attention_out_multiplier": 0.8, "key_multiplier": 0.5, "ssm_in_multiplier": 1.2, "ssm_out_multiplier": 0.7,
    "ssm_multipliers": [0.6, 1.1, 0.9, 1.3, 0.8], "mlp_multipliers": [0.9, 1.1],
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
}
CONFIGS = {
    "gate": dict(_BASE),                                                        # the bare gate, tied head
    "gated_norm": {**_BASE, "mamba_rms_norm": True, "mamba_n_groups": 2, "tie_word_embeddings": False,
                   "num_hidden_layers": 3, "mamba_proj_bias": True, "projectors_bias": True},
}
# the same model again for long prompts that the reference cuts into portions of 512 tokens
CONFIGS["long"] = {**_BASE, "max_position_embeddings": 4096, "rope_theta": 1e4, "num_key_value_heads": 1}
# heads of 128 in both mixers, three query heads per KV head, a state of 256, the norm before the gate, llama3
# frequency scaling
CONFIGS["wide"] = {**_BASE, "hidden_size": 384, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128,
                   "intermediate_size": 512, "mamba_d_ssm": 384, "mamba_n_heads": 3, "mamba_d_head": 128,
                   "mamba_d_state": 256, "mamba_rms_norm": True, "mamba_norm_before_gate": True, "rope_theta": 1e5,
                   "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                    "original_max_position_embeddings": 64}}
SEEDS = {"gate": 71, "gated_norm": 72, "long": 73, "wide": 74}
# prompt lengths and the reference's `max_prefill_tokens`; 150 and 300 cross a 128-token chunk of the SSD form
RUNS = {"gate": ((150, 37, 300), 1024), "gated_norm": ((150, 37, 300), 1024), "long": ((1100, 2200, 700), 512),
        "wide": ((150, 37, 300), 1024)}
NEW_TOKENS = 8


def run_reference(name: str) -> dict:
    import numpy as np
    import torch
    from tiny import make_model_dir
    from baseline.reference_arm import REF, _named_dlpack_include, _write_model_folder

    raw = CONFIGS[name]
    tmp = tempfile.mkdtemp(prefix=f"logssms_golden_{name}_")
    make_model_dir(tmp, raw, seed=SEEDS[name], dtype=torch.bfloat16)
    with open(os.path.join(tmp, "config.json")) as f:
        written = json.load(f)
    _write_model_folder(written, tmp)              # the same config.json again, plus the tokenizer files the scheduler wants

    sys.path.insert(0, REF)
    shim = _named_dlpack_include()
    if shim is not None and shim not in os.environ.get("NVCC_PREPEND_FLAGS", ""):
        os.environ["NVCC_PREPEND_FLAGS"] = (os.environ.get("NVCC_PREPEND_FLAGS", "") + f" -I{shim}").strip()
    from logssms.core import SamplingParams
    from logssms.distributed import DistributedInfo
    from logssms.message import UserMsg
    from logssms.scheduler import SchedulerConfig
    from logssms.scheduler.scheduler import Scheduler

    class InProcessScheduler(Scheduler):
        def __init__(self, config):
            self._pending: list = []
            self.results: list = []
            super().__init__(config)
            self.receive_msg = self._take
            self.send_result = self.results.extend

        def _take(self, blocking: bool = False):
            out, self._pending = self._pending, []
            return out

    config = SchedulerConfig(model_path=tmp, tp_info=DistributedInfo(0, 1), dtype=torch.bfloat16, max_running_req=4,
                             use_dummy_weight=False, max_seq_len_override=4096 if name == "long" else 1024,
                             max_prefill_tokens=RUNS[name][1])
    sched = InProcessScheduler(config)
    seen: list = []
    inner = sched.engine._sample_batch

    def recording(logits, batch, args):
        seen.append(logits[:batch.size].float().cpu().clone())
        return inner(logits, batch, args)
    sched.engine._sample_batch = recording

    rng = np.random.default_rng(SEEDS[name])
    out: dict = {}
    state = None
    with torch.inference_mode():
        for i, n in enumerate(RUNS[name][0]):
            ids = rng.integers(0, raw["vocab_size"], n).astype(np.int32)
            seen.clear()
            first = len(sched.results)
            sched._pending.append(UserMsg(uid=i, input_ids=torch.from_numpy(ids),
                                          sampling_params=SamplingParams(temperature=0.0, max_tokens=NEW_TOKENS, ignore_eos=True)))
            deadline = time.time() + 300
            while not any(m.uid == i and m.finished for m in sched.results[first:]):
                state = sched.overlap_loop(state)
                if time.time() > deadline:
                    raise RuntimeError(f"{name}: request {i} did not finish")
            for _ in range(4):                         # let the step that overlapped the last token drain
                state = sched.overlap_loop(state)
            torch.cuda.synchronize()
            tokens = []
            for m in sched.results[first:]:
                if m.uid == i:
                    tokens += m.next_token if isinstance(m.next_token, list) else [m.next_token]
            # a prompt that is cut into portions passes the sampling step once per portion: the rows before the
            # last portion's are not this request's tokens (the check below holds the alignment)
            earlier = -(-n // RUNS[name][1]) - 1
            rows = [t for t in seen if t.shape[0] == 1][earlier:earlier + NEW_TOKENS]
            if len(tokens) != NEW_TOKENS or len(rows) != NEW_TOKENS:
                raise RuntimeError(f"{name}: request {i}: {len(tokens)} tokens, {len(rows)} rows of logits")
            logits = torch.cat(rows)
            if logits.argmax(-1).tolist() != tokens:
                raise RuntimeError(f"{name}: request {i}: the recorded logits are not the ones its tokens were sampled from")
            out[f"prompt_{i}"] = torch.from_numpy(ids.astype(np.int64))
            out[f"tokens_{i}"] = torch.tensor(tokens, dtype=torch.int64)
            out[f"logits_{i}"] = logits.contiguous()
            print(f"[golden] {name}: prompt of {n} tokens -> {tokens}", flush=True)
    return out


def main() -> int:
    from safetensors.torch import save_file
    names = sys.argv[1:] or list(CONFIGS)
    for name in names:
        if len(names) > 1:
            # one engine per process: the reference's scheduler owns process-wide state
            import subprocess
            rc = subprocess.call([sys.executable, os.path.abspath(__file__), name])
            if rc != 0:
                return rc
            continue
        data = run_reference(name)
        path = os.path.join(HERE, f"reference_model_{name}.safetensors")
        save_file(data, path, metadata={"config": json.dumps(CONFIGS[name]), "seed": str(SEEDS[name])})
        print(f"[golden] wrote {path}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
