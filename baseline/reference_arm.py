"""The reference arm of bench.py: the unmodified dakingffo/LogSSMs, installed under baseline/_ref.

It runs the reference's own `Scheduler` (python/logssms/scheduler/scheduler.py) and `Engine` through
their public constructors and the scheduler's own loop (`overlap_loop`, the body of `run_forever`), fed
in process the way the reference's own end-to-end test feeds it (tests/mtp/test_mtp_e2e.py:63-127:
`receive_msg` / `send_result` replaced by in-memory lists, everything else stock).  Weights are the
reference's `use_dummy_weight` random weights on the same config.json as our arm, prompts the same
seeded token ids.  Nothing of logssms_b200 is on this path.

What is timed is what our arm times: K scheduler iterations in the steady decode state (one new token
per request and iteration, sampling and the host read-back of the ids included), on the device with
CUDA events, after W warm-up iterations.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _write_model_folder(model: dict, path: str) -> None:
    """config.json plus the smallest tokenizer the scheduler's `load_tokenizer` accepts (the benchmark
    feeds token ids; the tokenizer only supplies an end-of-sequence id, which `ignore_eos` overrides)."""
    os.makedirs(path, exist_ok=True)
    cfg = dict(model)
    cfg.setdefault("torch_dtype", "bfloat16")
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    from tokenizers import Tokenizer, models
    vocab = {f"t{i}": i for i in range(256)}
    vocab["<eos>"] = 256
    tok = Tokenizer(models.WordLevel(vocab, unk_token="t0"))
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "unk_token": "t0"}, f)


def _named_dlpack_include() -> str | None:
    """A folder to put FIRST on nvcc's include path: a copy of the installed tvm-ffi `dlpack/dlpack.h`, made here
    at run time, in which every `typedef struct { ... } Name;` reads `typedef struct Name { ... } Name;`.

    Why: the reference's `csrc/include/logssms/tensor.hpp` holds `std::vector<DLDataType>` in a class with a
    defaulted destructor and is compiled with `-std=c++20` (python/logssms/tvm/utils.py:20-21).  nvcc 12.9's
    front end aborts (`lexical.c`, `find_allocated_name_reference`) on `std::destroy_at` of a struct that has a
    typedef name only, which is how dlpack declares `DLDataType` and `DLDevice`.  Naming the structs changes
    neither layout nor ABI, and neither the reference nor the installed package is touched: the folder reaches
    nvcc through the NVCC_PREPEND_FLAGS environment variable of this process only."""
    import re
    try:
        import tvm_ffi
    except ImportError:
        return None
    src = os.path.join(os.path.dirname(tvm_ffi.__file__), "include", "dlpack", "dlpack.h")
    if not os.path.isfile(src):
        return None
    with open(src) as f:
        text = f.read()
    pieces, pos = [], 0
    for m in re.finditer(r"typedef struct \{", text):
        close = re.compile(r"\n\} (\w+);").search(text, m.end())
        if close is None:
            continue
        pieces += [text[pos:m.start()], f"typedef struct {close.group(1)} {{"]
        pos = m.end()
    pieces.append(text[pos:])
    out = tempfile.mkdtemp(prefix="logssms_ref_dlpack_")
    os.makedirs(os.path.join(out, "dlpack"))
    with open(os.path.join(out, "dlpack", "dlpack.h"), "w") as f:
        f.write("".join(pieces))
    return out


def run(args, model: dict, context: int, max_seq_len: int) -> dict:
    if not os.path.isdir(os.path.join(REF, "logssms")):
        raise RuntimeError("baseline/_ref holds no installed reference (pip install --target baseline/_ref did not run)")
    sys.path.insert(0, REF)
    shim = _named_dlpack_include()
    if shim is not None:
        os.environ["NVCC_PREPEND_FLAGS"] = (os.environ.get("NVCC_PREPEND_FLAGS", "") + f" -I{shim}").strip()
    import numpy as np
    import torch
    from logssms.core import SamplingParams
    from logssms.distributed import DistributedInfo
    from logssms.message import UserMsg
    from logssms.scheduler import SchedulerConfig
    from logssms.scheduler.scheduler import Scheduler

    tmp = tempfile.mkdtemp(prefix="logssms_ref_bench_")
    _write_model_folder(model, tmp)
    batch = args.batch
    new_tokens = args.warmup + args.steps + 8
    rng = np.random.default_rng(1234)
    next_uid = [0]

    def messages(count: int, prompt_len: int, max_tokens: int) -> list:
        out = []
        for _ in range(count):
            ids = torch.from_numpy(rng.integers(0, model["vocab_size"], prompt_len).astype(np.int32))
            out.append(UserMsg(uid=next_uid[0], input_ids=ids,
                               sampling_params=SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)))
            next_uid[0] += 1
        return out

    class InProcessScheduler(Scheduler):
        def __init__(self, config, pending):
            self._pending = list(pending)
            self.results: list = []
            super().__init__(config)
            self.receive_msg = self._take
            self.send_result = self.results.extend

        def _take(self, blocking: bool = False):
            out, self._pending = self._pending, []
            return out

    config = SchedulerConfig(model_path=tmp, tp_info=DistributedInfo(0, 1), dtype=torch.bfloat16, max_running_req=64,
                             use_dummy_weight=True, max_seq_len_override=max_seq_len,
                             max_prefill_tokens=args.prefill_budget)      # cache type, attention backend, graphs: the defaults
    t0 = time.time()
    sched = InProcessScheduler(config, messages(batch, context - 1, new_tokens))
    print(f"[bench] reference engine up in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    state = {"data": None}

    def pump():
        state["data"] = sched.overlap_loop(state["data"])

    def decode_point(count: int, first_uid: int) -> dict:
        """The `count` requests already fed: prompts, W warm-up iterations, K timed ones, then the rest of their tokens."""
        deadline = time.time() + 600
        while len({m.uid for m in sched.results if m.uid >= first_uid}) < count:      # every request has its first token
            pump()
            if time.time() > deadline:
                raise RuntimeError("reference scheduler did not finish the prompts within 600 s")
        for _ in range(args.warmup):
            pump()
        torch.cuda.synchronize()
        before = len(sched.results)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        start.record()
        for _ in range(args.steps):
            pump()
        stop.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        produced = len(sched.results) - before
        ms = start.elapsed_time(stop)
        if produced < count * (args.steps - 1):
            raise RuntimeError(f"reference produced {produced} tokens in {args.steps} iterations of batch {count}: not in steady decode")
        for _ in range(16):                                # the requests end by length within a few more iterations
            pump()
        return {"tok_s": produced / (ms / 1e3), "ms_per_step": ms / args.steps, "wall_tok_s": produced / wall}

    with torch.inference_mode():
        main = decode_point(batch, 0)
        points, prefill = {}, None
        try:                                               # further points of the same benchmark; the headline stands without them
            for count in (1, 64):
                first = next_uid[0]
                sched._pending.extend(messages(count, context - 1, new_tokens))
                points[f"decode_b{count}"] = decode_point(count, first)["tok_s"]
            times = []
            for _ in range(4):                             # a 2,048-token prompt to its first token, through the scheduler
                first = next_uid[0]
                sched._pending.extend(messages(1, 2048, 1))
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                deadline = time.time() + 120
                while not any(m.uid == first for m in sched.results) and time.time() < deadline:
                    pump()
                stop.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(stop))
                for _ in range(4):
                    pump()
            prefill = {"tokens": 2048, "ms": min(times[1:]), "value": 2048 / (min(times[1:]) / 1e3),
                       "path": "one prompt through Scheduler.overlap_loop until its first token"}
        except Exception as exc:
            print(f"[bench] reference: further points failed: {type(exc).__name__}: {exc}", file=sys.stderr, flush=True)
    out = {
        "impl": "reference", "metric": "decode tok/s (batch 8, 2,048-token contexts; 0.5B-class Falcon-H1)",
        "value": main["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform token ids, the reference's dummy weights)",
        "config": {"model": "Falcon-H1-0.5B-class", "layers": model["num_hidden_layers"], "global_batch": batch,
                   "seq_len": context, "context_budget": max_seq_len, "parallelism": "single GPU",
                   "path": "Scheduler.overlap_loop, default cache type and attention backend"},
        "e2e": {"value": main["wall_tok_s"], "unit": "tokens/s"},
        "points": points,
    }
    if prefill is not None:
        out["prefill"] = prefill
    return out


def main() -> int:
    """Child process of `bench.py --impl reference`: prints the JSON line, or the reason it could not."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-json", required=True)
    ap.add_argument("--context", type=int, required=True)
    ap.add_argument("--max-seq-len", type=int, required=True)
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--warmup", type=int, required=True)
    ap.add_argument("--batch", type=int, required=True)
    ap.add_argument("--prefill-budget", type=int, default=8192)
    args = ap.parse_args()
    with open(args.model_json) as f:
        model = json.load(f)
    try:
        line = run(args, model, args.context, args.max_seq_len)
    except BaseException as exc:                 # also SystemExit / KeyboardInterrupt raised inside the reference
        import traceback
        traceback.print_exc()
        text = f"{type(exc).__name__}: {exc}".splitlines()
        detail = next((t.strip() for t in text[1:] if "error" in t.lower() and "FAILED" not in t), "")
        line = {"impl": "reference", "unavailable": (text[0] + (" | " + detail if detail else ""))[:400]}
    print("RESULT " + json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
