#!/usr/bin/env python3
"""Decode and prefill throughput of the Falcon-H1 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config 0p5b|1p5b-deep|7b] [--no-extra] [--no-check]

Prints ONE JSON line.  The default run is the 0.5B-class configuration: `value` is decoded tokens per
second at batch 8 from 2,048-token contexts.  A timed region is exactly K decode steps (one new token per
request and step, sampling included) between two CUDA events, after W warm-up steps; regions are repeated
back to back (within the benchmark's 256 new tokens per request, and for about a second) and the median
region is reported, so that clock samples fall inside the timed work.  `e2e` is the same K-step region
through the Python entry point with the token ids visiting the host every step (sampled ids are read back,
the next step's ids are copied in from pinned memory; wall clock).  `prefill` is one 2,048-token prompt as
one step; `points` holds decode at batch 1 and 64; `roofline` compares the decode step with the bytes it
has to read.

The default run then adds the two larger workloads as further `points` with their details under
`workloads` (`--no-extra` leaves them out): the 1.5B-Deep-class mixed serving run (32 requests, prompts of
128..4,096 tokens in portions of at most 512 tokens per step, 128 new tokens each at temperature 0.8), and
the 7B-class run (decode at batch 64 from 4,096-token contexts, one 32,768-token prompt in scheduled
portions) with fewer layers than the configuration has, both numbers named.  `--config 1p5b-deep` or
`--config 7b` runs one of them alone with ALL its layers and prints its own line.

Before anything is timed each configuration generates 8 greedy tokens from a 300-token prompt on a
2-layer model of the same layer sizes and compares them with the plain implementation under tests/plain
(`--no-check` skips this).

Models have random bfloat16 weights written through the random-weights mode, prompts are seeded uniform
token ids (the reference's own load generator synthesises random-token prompts as well,
benchmarks/bench_common.py:266-279).  Every decode step reads about 1 GB of weights plus the live requests'
caches, more than the 126 MB L2, so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_MUP = {
    "embedding_multiplier": 5.0, "lm_head_multiplier": 0.25, "attention_in_multiplier": 1.5,
    "attention_out_multiplier": 0.8, "key_multiplier": 0.5, "ssm_in_multiplier": 1.2, "ssm_out_multiplier": 0.7,
    "ssm_multipliers": [0.6, 1.1, 0.9, 1.3, 0.8], "mlp_multipliers": [0.9, 1.1],
}
_COMMON = {
    "architectures": ["FalconH1ForCausalLM"], "model_type": "falcon_h1", "rms_norm_eps": 1e-5, "rope_theta": 1e11,
    "mamba_n_groups": 1, "mamba_d_conv": 4, "mamba_chunk_size": 128, "mamba_conv_bias": True, "mamba_proj_bias": False,
    "projectors_bias": False, "mamba_rms_norm": False, "mamba_norm_before_gate": False,
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False, **_MUP,
}
# the three benchmark configurations: 0.5B-class (the default line), 1.5B-Deep-class, 7B-class layer sizes
MODELS = {
    "0p5b": {**_COMMON, "num_hidden_layers": 36, "hidden_size": 1024, "num_attention_heads": 8, "num_key_value_heads": 2,
             "head_dim": 64, "intermediate_size": 2048, "vocab_size": 32784, "max_position_embeddings": 8192,
             "tie_word_embeddings": True, "mamba_d_ssm": 1536, "mamba_n_heads": 24, "mamba_d_head": 64, "mamba_d_state": 128},
    "1p5b-deep": {**_COMMON, "num_hidden_layers": 66, "hidden_size": 1280, "num_attention_heads": 6, "num_key_value_heads": 2,
                  "head_dim": 128, "intermediate_size": 3072, "vocab_size": 65536, "max_position_embeddings": 8192,
                  "tie_word_embeddings": True, "mamba_d_ssm": 1536, "mamba_n_heads": 24, "mamba_d_head": 64,
                  "mamba_d_state": 256},
    "7b": {**_COMMON, "num_hidden_layers": 44, "hidden_size": 3072, "num_attention_heads": 12, "num_key_value_heads": 2,
           "head_dim": 128, "intermediate_size": 12288, "vocab_size": 130048, "max_position_embeddings": 40960,
           "tie_word_embeddings": False, "mamba_d_ssm": 3072, "mamba_n_heads": 24, "mamba_d_head": 128,
           "mamba_d_state": 256},
}
NAMES = {"0p5b": "Falcon-H1-0.5B-class", "1p5b-deep": "Falcon-H1-1.5B-Deep-class", "7b": "Falcon-H1-7B-class"}
MODEL = MODELS["0p5b"]
CONTEXT = 2048            # tokens each request holds when decoding starts
NEW_TOKENS = 256          # tokens each request decodes in the benchmark's definition
MAX_SEQ_LEN = 8192        # the benchmark's context budget
PREFILL_TOKENS = 2048
LAYERS_7B_DEFAULT = 8     # layers of the 7B-class model in the default run (all 44 with --config 7b)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def log(msg: str) -> None:
    print(f"[bench] {msg}", file=sys.stderr, flush=True)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        idx = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
        try:
            self.proc = subprocess.Popen([exe, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", idx], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        deadline = time.time() + 5.0                      # the first sample takes nvidia-smi a moment
        while not self.lines and time.time() < deadline:
            time.sleep(0.05)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self, lo: int = 0, hi: int | None = None) -> dict:
        sm, mx, reasons = [], [], set()
        span = self.lines[lo:hi]
        if not span:                                      # a region shorter than one sampling period: its neighbours
            span = self.lines[max(lo - 2, 0):(hi or len(self.lines)) + 2]
        for line in span:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- model arithmetic
def model_numbers(cfg: dict, layers: int) -> dict:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    nh, P, N, G, K = (cfg["mamba_n_heads"], cfg["mamba_d_head"], cfg["mamba_d_state"], cfg["mamba_n_groups"],
                      cfg["mamba_d_conv"])
    inner = nh * P
    conv_dim = inner + 2 * G * N
    per_layer_matrix = (H * (Hq + 2 * Hkv) * hd + Hq * hd * H + H * (inner + conv_dim + nh) + inner * H + 3 * H * I)
    matrix_params = layers * per_layer_matrix
    head_params = V * H
    kv_bytes_per_token = layers * 2 * Hkv * hd * 2
    state_bytes = layers * nh * P * N * 4
    conv_bytes = layers * conv_dim * (K - 1) * 2
    return {
        "matrix_params": matrix_params, "head_params": head_params, "kv_bytes_per_token": kv_bytes_per_token,
        "state_bytes": state_bytes, "conv_bytes": conv_bytes,
        # multiply-adds of one token: projections, plus per-token SSD work (state update and read-out)
        "linear_flops_per_token": 2 * matrix_params,
        "ssd_flops_per_token": layers * (2 * 2 * nh * P * N + 2 * 2 * nh * P * cfg["mamba_chunk_size"] // 2
                                         + 2 * G * N * cfg["mamba_chunk_size"] // 2),
        "attn_flops_per_pair": layers * 4 * Hq * hd,
    }


def decode_bytes(num: dict, batch: int, ctx: float) -> float:
    """Bytes a decode step has to read: every weight once (projections and the output head) and the
    live requests' caches (keys/values, SSM state read and written, conv window read and written)."""
    weights = 2 * (num["matrix_params"] + num["head_params"])
    per_request = ctx * num["kv_bytes_per_token"] + 2 * num["state_bytes"] + 2 * num["conv_bytes"]
    return weights + batch * per_request


def prefill_flops(num: dict, T: int, start: int = 0, heads: int = 1) -> float:
    """Multiply-adds (x2) of a prompt portion of T tokens that begins at position `start`; `heads` rows go
    through the output head."""
    pairs = T * start + T * (T + 1) / 2
    return T * (num["linear_flops_per_token"] + num["ssd_flops_per_token"]) + num["attn_flops_per_pair"] * pairs \
        + 2 * num["head_params"] * heads


def step_bound_seconds(num: dict, entries: list[tuple[int, int]], wanted: int, pk: dict) -> float:
    """Lower bound of one step's time: the larger of (bytes it must move / copy bandwidth) and (FLOPs / bf16 peak).
    `entries`: (tokens the request brings, tokens it held before)."""
    flops = sum(prefill_flops(num, n, s, 0) for n, s in entries) + 2 * num["head_params"] * wanted
    byts = 2 * (num["matrix_params"] + (num["head_params"] if wanted else 0))
    for n, s in entries:
        byts += (s + n) * num["kv_bytes_per_token"] + 2 * num["state_bytes"] + 2 * num["conv_bytes"]
    return max(byts / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))


# --------------------------------------------------------------------------- pieces shared by the workloads
def write_model(cfg: dict, path: str) -> None:
    import torch
    from logssms_b200.config import make_model_config
    from logssms_b200.weights import write_random_model
    t0 = time.time()
    write_random_model(make_model_config(cfg), path, seed=0, dtype=torch.bfloat16)
    log(f"wrote random model ({cfg['num_hidden_layers']} layers, hidden {cfg['hidden_size']}) in {time.time() - t0:.1f} s")


def check_against_plain(name: str) -> dict:
    """8 greedy tokens from a 300-token prompt on a 2-layer model of the configuration's layer sizes, each compared
    with the plain implementation's logits of the whole sequence so far (as `__graft_entry__.smoke` does)."""
    import numpy as np
    import torch
    tests = os.path.join(ROOT, "tests")
    if tests not in sys.path:
        sys.path.insert(0, tests)
    from tiny import TOL, make_model_dir, plain_logits
    from logssms_b200.engine import LLM
    from logssms_b200.ops import kernels as K
    from logssms_b200.sampling import SamplingParams
    cfg = {**MODELS[name], "num_hidden_layers": 2}
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, cfg["vocab_size"], 300).tolist()
    tmp = tempfile.mkdtemp(prefix="logssms_b200_check_")
    try:
        model_dir = make_model_dir(os.path.join(tmp, "m"), cfg, seed=3, dtype=torch.bfloat16, perturb=False)
        llm = LLM(model_dir, "bfloat16", max_running_requests=2, max_seq_len_override=512, num_pages=8,
                  max_prefill_tokens=8192)
        out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0]
        K.check_kernel_errors(llm.engine.device)
        del llm
        torch.cuda.empty_cache()
        logits = plain_logits(model_dir, prompt + out.token_ids[:-1], "bfloat16")[len(prompt) - 1:]
        worst, agree = 0.0, 0
        for tok, row in zip(out.token_ids, logits):
            best = int(row.argmax())
            gap = float(row[best] - row[tok]) / float(row.abs().max())
            worst = max(worst, gap)
            agree += int(tok == best)
        if worst > TOL["bfloat16"]:
            raise RuntimeError(f"{name}: the engine's greedy tokens {out.token_ids} are not the plain implementation's "
                               f"(worst logit gap {worst:.3g} of the largest logit)")
        log(f"check {name}: 8 greedy tokens after a 300-token prompt, {agree}/8 equal the plain argmax, worst gap {worst:.2g}")
        return {"tokens": 8, "equal_argmax": agree, "worst_gap": worst}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


class TimedRegions:
    """K-step regions, each between two CUDA events, repeated back to back."""

    def __init__(self, clocks: ClockSampler):
        self.clocks = clocks

    def run(self, step, K: int, regions: int) -> dict:
        import torch
        ms, wall = [], []
        lo = self.clocks.mark()
        for _ in range(regions):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            w0 = time.perf_counter()
            start.record()
            for _ in range(K):
                step()
            stop.record()
            torch.cuda.synchronize()
            wall.append(time.perf_counter() - w0)
            ms.append(start.elapsed_time(stop))
        return {"ms": statistics.median(ms), "wall": statistics.median(wall), "regions": regions,
                "clock_span": (lo, self.clocks.mark()), "all_ms": ms}


def decode_run(llm, cfg: dict, rng, clocks, batch: int, context: int, K: int, W: int, budget: int, *, through_host: bool,
               max_regions: int | None = None) -> dict:
    """Prefill `batch` prompts of `context` - 1 tokens (untimed), then W warm-up steps and timed regions of K decode
    steps.  `through_host`: every step's ids are read by the host before the next step is launched from them."""
    import torch
    from logssms_b200.ops import kernels as Kn
    from logssms_b200.sampling import SamplingParams
    regions = max(1, (NEW_TOKENS - W) // K)
    if max_regions is not None:
        regions = min(regions, max_regions)
    # requests whose prompts finish first decode beside the others' portions: room for those tokens too, so that
    # none ends (and the batch shrinks) inside the timed steps
    prompt_steps = -(-batch * context // budget) + batch
    sp = SamplingParams(temperature=0.0, max_tokens=W + regions * K + 8 + prompt_steps, ignore_eos=True)
    llm.scheduler.overlap = not through_host
    reqs = [llm.add_request(rng.integers(0, cfg["vocab_size"], context - 1).tolist(), sp) for _ in range(batch)]
    while not all(r.prompt_done for r in reqs):
        llm.step()
    for _ in range(W):
        llm.step()
    torch.cuda.synchronize()
    # about a second of regions, within the 256 new tokens of the benchmark
    probe = TimedRegions(clocks).run(llm.step, K, 1)
    regions = max(1, min(regions - 1, int(1000.0 / max(probe["ms"], 1e-3))))
    Kn.launch_count = 0
    h2d0, d2h0 = llm.engine.h2d_bytes, llm.d2h_bytes
    timed = TimedRegions(clocks).run(llm.step, K, regions)
    launches = Kn.launch_count // regions
    steps = K * regions
    Kn.check_kernel_errors(llm.engine.device)
    if any(r.state != "running" for r in reqs):
        raise RuntimeError("a request ended inside the timed decode steps")
    out = {"ms_per_step": timed["ms"] / K, "tok_s": batch * K / (timed["ms"] / 1e3), "launches": launches,
           "wall_tok_s": batch * K / timed["wall"], "clock_span": timed["clock_span"], "regions": regions,
           "h2d": (llm.engine.h2d_bytes - h2d0) / steps, "d2h": (llm.d2h_bytes - d2h0) / steps,
           "ctx_mid": context + W + K + steps / 2}
    for r in reqs:
        llm.abort(r)
    llm.scheduler.overlap = True
    return out


def config_keys(cfg: dict, layers: int, **more) -> dict:
    """Every size of the model, flat."""
    return {
        "layers": layers, "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
        "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
        "vocab": cfg["vocab_size"], "mamba_heads": cfg["mamba_n_heads"], "mamba_d_head": cfg["mamba_d_head"],
        "mamba_d_state": cfg["mamba_d_state"], "mamba_d_conv": cfg["mamba_d_conv"], "mamba_chunk": cfg["mamba_chunk_size"],
        **more,
    }


# --------------------------------------------------------------------------- configs[2]: the default line
def run_0p5b(args, clocks) -> dict:
    import numpy as np
    import torch

    from logssms_b200.engine import LLM, StepEntry
    from logssms_b200.ops import kernels as K

    pk, pk_src = peaks()
    cfg = dict(MODEL)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    num = model_numbers(cfg, layers)
    rng = np.random.default_rng(1234)
    tmp = tempfile.mkdtemp(prefix="logssms_b200_bench_")
    try:
        write_model(cfg, tmp)
        llm = LLM(tmp, "bfloat16", max_running_requests=64, max_seq_len_override=MAX_SEQ_LEN,
                  max_prefill_tokens=args.prefill_budget, seed=0)

        def run(batch, through_host, **kw):
            return decode_run(llm, cfg, rng, clocks, batch, CONTEXT, args.steps, args.warmup, args.prefill_budget,
                              through_host=through_host, **kw)

        def prefill_run() -> dict:
            ids = rng.integers(0, cfg["vocab_size"], PREFILL_TOKENS).tolist()
            times = []
            # the same length over and over: after `exact_after` steps through its bucket's graph the shape gets a graph
            # of its own (three slow steps), which the timed steps replay
            kWarm = llm.engine.exact_after + 8
            for i in range(kWarm + 5):
                req = llm.engine.new_request()
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                llm.engine.step([StepEntry(req, ids, [PREFILL_TOKENS - 1])])
                stop.record()
                torch.cuda.synchronize()
                if i >= kWarm:
                    times.append(start.elapsed_time(stop))
                llm.engine.release(req)
            K.check_kernel_errors(llm.engine.device)
            ms = statistics.median(times)
            flops = prefill_flops(num, PREFILL_TOKENS)
            return {"value": PREFILL_TOKENS / (ms / 1e3), "tokens": PREFILL_TOKENS, "ms": ms,
                    "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12}

        def new_length_run() -> float:
            """Prompts of lengths that have never come before (2,041, 2,039, ...): each runs through the graph of its
            bucket, filled up with dummy requests to 2,176 tokens.  Median device time of the later ones."""
            times = []
            for i, n in enumerate(range(PREFILL_TOKENS - 7, PREFILL_TOKENS - 7 - 2 * 8, -2)):
                ids = rng.integers(0, cfg["vocab_size"], n).tolist()
                req = llm.engine.new_request()
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                llm.engine.step([StepEntry(req, ids, [n - 1])])
                stop.record()
                torch.cuda.synchronize()
                if i >= 3:
                    times.append(start.elapsed_time(stop))
                llm.engine.release(req)
            return statistics.median(times)

        def prefill_both() -> dict:
            """A prompt length that keeps coming is replayed from a CUDA graph of its own (`ms`, `value`, `frac`);
            `first_ms` is a prompt of a length that has never come before, through the graph of its bucket;
            `eager_ms` the same step launched kernel by kernel (graphs off)."""
            out = prefill_run()
            out["first_ms"] = new_length_run()
            llm.engine.use_graphs = False
            try:
                out["eager_ms"] = prefill_run()["ms"]
            finally:
                llm.engine.use_graphs = True
            out["path"] = ("graph of the shape (a length that keeps coming); first_ms: a new length through the graph "
                           "of its bucket; eager_ms: kernel by kernel")
            return out

        main = run(args.batch, False)
        e2e = run(args.batch, True)
        points = {}
        for b in (1, 64):
            points[f"decode_b{b}"] = run(b, False, max_regions=4)["tok_s"]
        prefill = prefill_both()
        bytes_step = decode_bytes(num, args.batch, main["ctx_mid"])
        achieved = bytes_step / (main["ms_per_step"] / 1e3) / 1e9
        ck = clocks.summary(*main["clock_span"])
        del llm
        torch.cuda.empty_cache()
        return {
            "metric": "decode tok/s (batch 8, 2,048-token contexts; 0.5B-class Falcon-H1)",
            "value": main["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "impl": "ours",
            "config": config_keys(cfg, layers, model=NAMES["0p5b"], layers_of_config=full_layers, global_batch=args.batch,
                                  seq_len=CONTEXT, context_budget=MAX_SEQ_LEN, parallelism="single GPU",
                                  l2="no flush: each step reads >1 GB of weights and caches (L2 is 126 MB)"),
            "timed_regions": main["regions"],
            "e2e": {"value": e2e["wall_tok_s"], "unit": "tokens/s", "device_timed": e2e["tok_s"],
                    "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                    "path": "LLM.add_request / LLM.step, token ids through the host every step",
                    "overlapped_value": main["wall_tok_s"]},
            "gpu_launches": main["launches"],
            "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "frac", "first_ms", "eager_ms", "path")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "bytes_per_step": bytes_step, "peaks": pk_src},
            "points": points,
            "clocks": {"sm_mhz": ck["sm_mhz"], "sm_max_mhz": ck["sm_max_mhz"], "reasons": ck["reasons"]},
        }
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# --------------------------------------------------------------------------- configs[3]: mixed serving
def run_1p5b_deep(args, clocks, layers: int | None = None) -> dict:
    """32 requests with seeded prompt lengths in 128..4,096, at most 512 prompt tokens per step beside the decoding
    requests (the reference cuts prompts the same way: python/logssms/scheduler/prefill.py:109-117), 128 new tokens
    each at temperature 0.8.  The whole run is timed: from the first step to the last token."""
    import numpy as np
    import torch

    from logssms_b200.engine import LLM
    from logssms_b200.ops import kernels as K
    from logssms_b200.sampling import SamplingParams

    pk, pk_src = peaks()
    cfg = dict(MODELS["1p5b-deep"])
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    layers = cfg["num_hidden_layers"]
    num = model_numbers(cfg, layers)
    requests, new_tokens, budget = 32, 128, 512
    tmp = tempfile.mkdtemp(prefix="logssms_b200_bench_")
    try:
        write_model(cfg, tmp)
        llm = LLM(tmp, "bfloat16", max_running_requests=requests, max_seq_len_override=4096 + new_tokens + 64,
                  max_prefill_tokens=budget, seed=0)
        shapes: list[tuple[list[tuple[int, int]], int]] = []
        inner = llm.engine.step

        def recording_step(entries, device_tokens=None):
            shapes.append(([(len(e.tokens), e.request.length) for e in entries], sum(len(e.want) for e in entries)))
            return inner(entries, device_tokens)

        def once(seed: int) -> dict:
            rng = np.random.default_rng(seed)
            lengths = rng.integers(128, 4097, requests).tolist()
            prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
            shapes.clear()
            lo = clocks.mark()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            w0 = time.perf_counter()
            start.record()
            reqs = [llm.add_request(p, SamplingParams(temperature=0.8, max_tokens=new_tokens, ignore_eos=True, seed=seed * 1000 + i))
                    for i, p in enumerate(prompts)]
            steps0 = llm.scheduler.steps
            llm.scheduler.run()
            stop.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - w0
            K.check_kernel_errors(llm.engine.device)
            assert all(len(r.output) == new_tokens for r in reqs), [r.finish_reason for r in reqs]
            ms = start.elapsed_time(stop)
            return {"ms": ms, "wall": wall, "steps": llm.scheduler.steps - steps0, "prompt_tokens": sum(lengths),
                    "clock_span": (lo, clocks.mark()), "bound_s": sum(step_bound_seconds(num, e, w, pk) for e, w in shapes)}

        llm.engine.step = recording_step
        once(99)                                   # warm-up with other prompts and lengths: builds kernels,
        once(98)                                   # captures the graphs of the buckets that such steps fall into
        # three timed passes over requests that were never seen before (other prompts and lengths each time); the
        # median pass is reported: a pass is seconds of host-driven serving on a machine that other jobs share
        passes = sorted((once(seed) for seed in (4321, 4322, 4323)), key=lambda r: r["ms"])
        run = passes[1]
        ck = clocks.summary(*run["clock_span"])
        gen = requests * new_tokens
        del llm
        torch.cuda.empty_cache()
        return {
            "metric": "generated tok/s (32 requests, prompts 128..4,096, 512 prompt tokens per step, 128 new tokens each, "
                      "temperature 0.8; 1.5B-Deep-class Falcon-H1)",
            "value": gen / (run["ms"] / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": run["steps"], "warmup": run["steps"],
            "ms_per_step": run["ms"] / run["steps"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids and prompt lengths, seeded random weights)",
            "impl": "ours",
            "config": config_keys(cfg, layers, model=NAMES["1p5b-deep"], layers_of_config=full_layers, global_batch=requests,
                                  seq_len="128..4096 + 128", prefill_tokens_per_step=budget, temperature=0.8,
                                  parallelism="single GPU"),
            "total_tok_s": (gen + run["prompt_tokens"]) / (run["ms"] / 1e3), "prompt_tokens": run["prompt_tokens"],
            "generated_tokens": gen, "total_ms": run["ms"], "passes_ms": [round(r["ms"], 1) for r in passes],
            "e2e": {"value": gen / run["wall"], "unit": "tokens/s", "path": "LLM.add_request / Scheduler.run, wall clock"},
            "roofline": {"bound": "per step max(bytes / copy bandwidth, FLOPs / bf16 peak), summed", "bound_ms": run["bound_s"] * 1e3,
                         "frac": run["bound_s"] * 1e3 / run["ms"], "peaks": pk_src},
            "clocks": {"sm_mhz": ck["sm_mhz"], "sm_max_mhz": ck["sm_max_mhz"], "reasons": ck["reasons"]},
        }
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# --------------------------------------------------------------------------- configs[4]: 7B-class
def run_7b(args, clocks, layers: int | None = None) -> dict:
    """Decode at batch 64 from 4,096-token contexts (K-step regions as in the default run), and one 32,768-token
    prompt through the scheduler in portions of the step budget."""
    import numpy as np
    import torch

    from logssms_b200.engine import LLM
    from logssms_b200.ops import kernels as K
    from logssms_b200.sampling import SamplingParams

    pk, pk_src = peaks()
    cfg = dict(MODELS["7b"])
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    layers = cfg["num_hidden_layers"]
    num = model_numbers(cfg, layers)
    batch, context, long_prompt, budget = 64, 4096, 32768, 8192
    rng = np.random.default_rng(77)
    tmp = tempfile.mkdtemp(prefix="logssms_b200_bench_")
    try:
        write_model(cfg, tmp)
        llm = LLM(tmp, "bfloat16", max_running_requests=batch, max_seq_len_override=long_prompt + 64,
                  max_prefill_tokens=budget, seed=0, num_pages=batch * (context + 512) // 64 + (long_prompt + 64) // 64 + 8)
        dec = decode_run(llm, cfg, rng, clocks, batch, context, args.steps, args.warmup, budget, through_host=False,
                         max_regions=6)
        bytes_step = decode_bytes(num, batch, dec["ctx_mid"])
        achieved = bytes_step / (dec["ms_per_step"] / 1e3) / 1e9
        ck = clocks.summary(*dec["clock_span"])
        times = []
        for i in range(3):
            ids = rng.integers(0, cfg["vocab_size"], long_prompt).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = llm.generate([ids], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))[0]
            stop.record()
            torch.cuda.synchronize()
            assert len(out.token_ids) == 1
            times.append(start.elapsed_time(stop))
        K.check_kernel_errors(llm.engine.device)
        ms = min(times[1:])
        flops = sum(prefill_flops(num, min(budget, long_prompt - s), s, 0) for s in range(0, long_prompt, budget)) \
            + 2 * num["head_params"]
        del llm
        torch.cuda.empty_cache()
        return {
            "metric": "decode tok/s (batch 64, 4,096-token contexts; 7B-class Falcon-H1)",
            "value": dec["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dec["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)", "impl": "ours",
            "config": config_keys(cfg, layers, model=NAMES["7b"], layers_of_config=full_layers, global_batch=batch,
                                  seq_len=context, long_prompt=long_prompt, prefill_tokens_per_step=budget,
                                  parallelism="single GPU"),
            "timed_regions": dec["regions"], "gpu_launches": dec["launches"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "bytes_per_step": bytes_step, "peaks": pk_src},
            "prefill": {"value": long_prompt / (ms / 1e3), "tokens": long_prompt, "ms": ms,
                        "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12,
                        "path": f"LLM.generate: {-(-long_prompt // budget)} scheduled portions of at most {budget} tokens"},
            "clocks": {"sm_mhz": ck["sm_mhz"], "sm_max_mhz": ck["sm_max_mhz"], "reasons": ck["reasons"]},
        }
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# --------------------------------------------------------------------------- our arm
def run_ours(args) -> dict:
    clocks = ClockSampler()
    checks = {}
    try:
        wanted = [args.config] if args.config != "0p5b" or args.no_extra else ["0p5b", "1p5b-deep", "7b"]
        if not args.no_check:
            for name in wanted:
                checks[name] = check_against_plain(name)
        clocks.start()
        if args.config == "1p5b-deep":
            line = run_1p5b_deep(args, clocks, args.layers or None)
        elif args.config == "7b":
            line = run_7b(args, clocks, args.layers or None)
        else:
            line = run_0p5b(args, clocks)
            if not args.no_extra:
                work = {}
                for name, fn, lay in (("1p5b-deep", run_1p5b_deep, None), ("7b", run_7b, LAYERS_7B_DEFAULT)):
                    try:
                        work[name] = fn(args, clocks, lay)
                    except Exception as exc:           # the default line stands even if a larger workload fails
                        work[name] = {"error": f"{type(exc).__name__}: {exc}".splitlines()[0][:300]}
                        log(f"workload {name} failed: {work[name]['error']}")
                mixed, big = work["1p5b-deep"], work["7b"]
                if "value" in mixed:
                    line["points"]["mixed_1p5b_deep_generated_tok_s"] = mixed["value"]
                    line["points"]["mixed_1p5b_deep_total_tok_s"] = mixed["total_tok_s"]
                if "value" in big:
                    tag = f"7b_{big['config']['layers']}of{big['config']['layers_of_config']}layers"
                    line["points"][f"decode_b64_ctx4096_{tag}"] = big["value"]
                    line["points"][f"prefill_32768_{tag}"] = big["prefill"]["value"]
                line["workloads"] = work
        if checks:
            line["checks"] = checks
        return line
    finally:
        clocks.stop()


# --------------------------------------------------------------------------- a short run for profilers
def run_probe(args) -> int:
    """`--probe decode|prefill|mixed`: a few steps of one kind on a model of `--layers` layers (default 4), with
    the CUDA profiler range switched on around the last ones, for `ncu --profile-from-start off`.  Prints a
    line with the device time of the unprofiled steps; nothing here is a benchmark value.  This is the one
    tracked way to reproduce the commands in the files under profiles/."""
    import numpy as np
    import torch

    from logssms_b200.engine import LLM, StepEntry
    from logssms_b200.sampling import SamplingParams

    cfg = dict(MODELS[args.config])
    cfg["num_hidden_layers"] = args.layers or 4
    context = args.context or CONTEXT
    tmp = tempfile.mkdtemp(prefix="logssms_b200_probe_")
    try:
        write_model(cfg, tmp)
        llm = LLM(tmp, "bfloat16", max_running_requests=64, max_seq_len_override=max(MAX_SEQ_LEN, context + 256),
                  max_prefill_tokens=8192)
        rng = np.random.default_rng(0)
        if args.probe == "decode":
            sp = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True)
            reqs = [llm.add_request(rng.integers(0, cfg["vocab_size"], context - 1).tolist(), sp) for _ in range(args.batch)]
            while not all(r.prompt_done for r in reqs):
                llm.step()
            for _ in range(5):
                llm.step()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(10):
                llm.step()
            stop.record()
            torch.cuda.synchronize()
            print(f"probe decode: batch {args.batch}, {cfg['num_hidden_layers']} layers, {start.elapsed_time(stop) / 10:.3f} ms/step", flush=True)
            torch.cuda.profiler.start()
            llm.step()
            llm.step()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        elif args.probe == "mixed":
            # `--batch` requests decode from `context`-token contexts beside a prompt that comes in portions of changing
            # length (none twice): such steps replay the graph of their bucket
            decoding = [llm.engine.new_request() for _ in range(args.batch)]
            for r in decoding:
                llm.engine.step([StepEntry(r, rng.integers(0, cfg["vocab_size"], context).tolist(), [])])
            prompt = llm.engine.new_request()

            def mixed(n):
                return [StepEntry(r, [5], [0]) for r in decoding] + [StepEntry(prompt, rng.integers(0, cfg["vocab_size"], n).tolist(), [n - 1])]
            for n in (480, 481, 482, 483, 484):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                llm.engine.step(mixed(n))
                torch.cuda.synchronize()
                print(f"probe mixed: {args.batch} decoding + {n} prompt tokens, {cfg['num_hidden_layers']} layers, {(time.perf_counter() - t0) * 1e3:.3f} ms", flush=True)
            torch.cuda.profiler.start()
            llm.engine.step(mixed(485))
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            ids = rng.integers(0, cfg["vocab_size"], PREFILL_TOKENS).tolist()
            for i in range(3):
                req = llm.engine.new_request()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                llm.engine.step([StepEntry(req, ids, [PREFILL_TOKENS - 1])])
                torch.cuda.synchronize()
                print(f"probe prefill: {PREFILL_TOKENS} tokens, {cfg['num_hidden_layers']} layers, {(time.perf_counter() - t0) * 1e3:.3f} ms", flush=True)
                llm.engine.release(req)
            req = llm.engine.new_request()
            torch.cuda.profiler.start()
            llm.engine.step([StepEntry(req, ids, [PREFILL_TOKENS - 1])])
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# --------------------------------------------------------------------------- the reference arm
def run_reference(args) -> dict:
    """The reference runs in a child process (its own CUDA context, streams and JIT caches), with a time
    limit; whatever goes wrong there becomes the `unavailable` line."""
    tmp = tempfile.mkdtemp(prefix="logssms_ref_cfg_")
    try:
        cfg = dict(MODEL)
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        path = os.path.join(tmp, "model.json")
        with open(path, "w") as f:
            json.dump(cfg, f)
        cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--model-json", path,
               "--context", str(CONTEXT), "--max-seq-len", str(MAX_SEQ_LEN), "--steps", str(args.steps),
               "--warmup", str(args.warmup), "--batch", str(args.batch), "--prefill-budget", str(args.prefill_budget)]
        try:
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=args.reference_timeout)
        except subprocess.TimeoutExpired:
            return {"impl": "reference", "unavailable": f"the reference did not finish within {args.reference_timeout} s"}
        sys.stderr.write(proc.stderr[-6000:])
        for line in reversed(proc.stdout.splitlines()):
            if line.startswith("RESULT "):
                return json.loads(line[len("RESULT "):])
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
        return {"impl": "reference", "unavailable": f"the reference process ended with code {proc.returncode}: {tail[0][:240]}"}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="0p5b", choices=sorted(MODELS),
                    help="0p5b: the default line (with the two larger workloads as further points unless --no-extra); "
                         "1p5b-deep, 7b: that workload alone, all its layers")
    ap.add_argument("--no-extra", action="store_true", help="default run without the 1.5B-Deep and 7B workloads")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison with the plain implementation")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (both are reported)")
    ap.add_argument("--context", type=int, default=0, help="--probe decode: tokens each request holds (default 2,048)")
    ap.add_argument("--prefill-budget", type=int, default=8192, help="token budget of one scheduled step")
    ap.add_argument("--reference-timeout", type=int, default=900, help="seconds the reference arm may take")
    ap.add_argument("--probe", choices=["decode", "prefill", "mixed"], default=None,
                    help="a short run of one kind of step for a profiler (see profiles/); prints no benchmark line")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench.py: this engine runs on one GPU; --gpus N>1 is not built")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.probe:
        return run_probe(args)
    if args.impl == "reference":
        try:
            line = run_reference(args)
        except Exception as exc:     # the reference arm never fails the run: it reports why it could not run
            line = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}".splitlines()[0][:300]}
        print(json.dumps(line))
        return 0
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
