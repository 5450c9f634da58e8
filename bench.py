#!/usr/bin/env python3
"""Decode and prefill throughput of the Falcon-H1 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at the default batch (8 requests, each
with a 2,048-token context): K decode steps (one new token per request and step, sampling
included) timed on the device with CUDA events after W warm-up steps.  `e2e` is the same loop
through the Python entry point (`LLM.add_request` / `LLM.step`): token ids travel from pinned host
memory to the device and the sampled ids come back to the host every step.  `prefill` is one
2,048-token prompt as one step; `points` holds decode at batch 1 and 64; `roofline` compares the
decode step with the bytes it has to read.

The model is the 0.5B-class Falcon-H1 configuration (random bfloat16 weights written through the
random-weights mode, seeded synthetic token ids).  Every decode step reads about 1 GB of weights plus
the live requests' caches, more than the 126 MB L2, so no L2 flush is needed between steps.
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

# BASELINE.json configs[2]: "Falcon-H1-0.5B-class"
MODEL = {
    "architectures": ["FalconH1ForCausalLM"], "model_type": "falcon_h1",
    "num_hidden_layers": 36, "hidden_size": 1024, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 2048, "vocab_size": 32784, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 8192, "rope_theta": 1e11, "tie_word_embeddings": True,
    "mamba_d_ssm": 1536, "mamba_n_heads": 24, "mamba_d_head": 64, "mamba_d_state": 128, "mamba_n_groups": 1,
    "mamba_d_conv": 4, "mamba_chunk_size": 128, "mamba_conv_bias": True, "mamba_proj_bias": False,
    "projectors_bias": False, "mamba_rms_norm": False, "mamba_norm_before_gate": False,
    "embedding_multiplier": 5.0, "lm_head_multiplier": 0.25, "attention_in_multiplier": 1.5,
    "attention_out_multiplier": 0.8, "key_multiplier": 0.5, "ssm_in_multiplier": 1.2, "ssm_out_multiplier": 0.7,
    "ssm_multipliers": [0.6, 1.1, 0.9, 1.3, 0.8], "mlp_multipliers": [0.9, 1.1],
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
}
CONTEXT = 2048            # tokens each request holds when decoding starts
MAX_SEQ_LEN = 8192        # the benchmark's context budget
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


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
                                          "-lms", "100", "-i", idx], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
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


def prefill_flops(num: dict, T: int) -> float:
    return T * (num["linear_flops_per_token"] + num["ssd_flops_per_token"]) \
        + num["attn_flops_per_pair"] * T * (T + 1) / 2 + 2 * num["head_params"]


# --------------------------------------------------------------------------- our arm
def run_ours(args) -> dict:
    import numpy as np
    import torch

    from logssms_b200.config import make_model_config
    from logssms_b200.engine import LLM
    from logssms_b200.ops import kernels as K
    from logssms_b200.sampling import SamplingParams
    from logssms_b200.weights import write_random_model

    pk, pk_src = peaks()
    cfg = dict(MODEL)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    num = model_numbers(cfg, layers)
    rng = np.random.default_rng(1234)
    tmp = tempfile.mkdtemp(prefix="logssms_b200_bench_")
    clocks = ClockSampler()
    try:
        t0 = time.time()
        write_random_model(make_model_config(cfg), tmp, seed=0, dtype=torch.bfloat16)
        print(f"[bench] wrote random model ({layers} layers) in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        new_tokens = args.warmup + args.steps + 8
        llm = LLM(tmp, "bfloat16", max_running_requests=64, max_seq_len_override=MAX_SEQ_LEN,
                  max_prefill_tokens=args.prefill_budget, seed=0)
        clocks.start()

        def prompts(batch):
            return [rng.integers(0, cfg["vocab_size"], CONTEXT - 1).tolist() for _ in range(batch)]

        def decode_run(batch: int, through_host: bool) -> dict:
            """Prefill `batch` prompts (untimed), then W + K decode steps; the K are timed."""
            # requests whose prompts finish first decode beside the others' portions: room for those tokens too,
            # so that none ends (and the batch shrinks) inside the timed steps
            prompt_steps = -(-batch * CONTEXT // args.prefill_budget) + batch
            sp = SamplingParams(temperature=0.0, max_tokens=new_tokens + prompt_steps, ignore_eos=True)
            reqs = [llm.add_request(p, sp) for p in prompts(batch)]
            while not all(r.prompt_done for r in reqs):
                llm.step(device_loop=not through_host)
            for _ in range(args.warmup):
                llm.step(device_loop=not through_host)
            torch.cuda.synchronize()
            lo = clocks.mark()
            K.launch_count = 0
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            h2d0, d2h0 = llm.engine.h2d_bytes, llm.d2h_bytes
            wall0 = time.perf_counter()
            start.record()
            for _ in range(args.steps):
                llm.step(device_loop=not through_host)
            stop.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - wall0
            ms = start.elapsed_time(stop)
            launches = K.launch_count
            hi = clocks.mark()
            if any(r.state != "running" for r in reqs):
                raise RuntimeError("a request ended inside the timed decode steps")
            out = {"ms_per_step": ms / args.steps, "tok_s": batch * args.steps / (ms / 1e3), "launches": launches,
                   "wall_tok_s": batch * args.steps / wall, "clock_span": (lo, hi),
                   "h2d": (llm.engine.h2d_bytes - h2d0) / args.steps, "d2h": (llm.d2h_bytes - d2h0) / args.steps}
            for r in reqs:
                llm.abort(r)
            return out

        def prefill_run() -> dict:
            ids = rng.integers(0, cfg["vocab_size"], PREFILL_TOKENS).tolist()
            times = []
            for i in range(3 + 5):
                req = llm.engine.new_request()
                from logssms_b200.engine import StepEntry
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                llm.engine.step([StepEntry(req, ids, [PREFILL_TOKENS - 1])])
                stop.record()
                torch.cuda.synchronize()
                if i >= 3:
                    times.append(start.elapsed_time(stop))
                llm.engine.release(req)
            ms = statistics.median(times)
            flops = prefill_flops(num, PREFILL_TOKENS)
            return {"value": PREFILL_TOKENS / (ms / 1e3), "tokens": PREFILL_TOKENS, "ms": ms,
                    "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12}

        def prefill_both() -> dict:
            """The engine replays a step whose shape it has seen twice from a CUDA graph (`ms`, `value`, `frac`);
            `first_ms` is the same step launched kernel by kernel, as a prompt of a new length runs."""
            out = prefill_run()
            llm.engine.use_graphs = False
            try:
                first = prefill_run()
            finally:
                llm.engine.use_graphs = True
            out["first_ms"] = first["ms"]
            out["path"] = "step graph (third and later steps of a shape); first_ms: kernel by kernel"
            return out

        main = decode_run(args.batch, through_host=False)
        e2e = decode_run(args.batch, through_host=True)
        points = {}
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_run(b, through_host=False)["tok_s"]
        prefill = prefill_both()
        clocks.stop()
        ctx_mid = CONTEXT + args.warmup + args.steps / 2
        bytes_step = decode_bytes(num, args.batch, ctx_mid)
        achieved = bytes_step / (main["ms_per_step"] / 1e3) / 1e9
        ck = clocks.summary(*main["clock_span"])
        line = {
            "metric": "decode tok/s (batch 8, 2,048-token contexts; 0.5B-class Falcon-H1)",
            "value": main["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "impl": "ours",
            "config": {
                "model": "Falcon-H1-0.5B-class", "layers": layers, "layers_of_config": full_layers,
                "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                "mamba_heads": cfg["mamba_n_heads"], "mamba_d_head": cfg["mamba_d_head"],
                "mamba_d_state": cfg["mamba_d_state"], "mamba_d_conv": cfg["mamba_d_conv"],
                "mamba_chunk": cfg["mamba_chunk_size"], "global_batch": args.batch, "seq_len": CONTEXT,
                "context_budget": MAX_SEQ_LEN, "parallelism": "single GPU",
                "l2": "no flush: each step reads >1 GB of weights and caches (L2 is 126 MB)",
            },
            "e2e": {"value": e2e["wall_tok_s"], "unit": "tokens/s", "device_timed": e2e["tok_s"],
                    "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
            "gpu_launches": main["launches"],
            "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "frac", "first_ms", "path")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "bytes_per_step": bytes_step, "peaks": pk_src},
            "points": points,
            "clocks": {"sm_mhz": ck["sm_mhz"], "sm_max_mhz": ck["sm_max_mhz"], "reasons": ck["reasons"]},
        }
        return line
    finally:
        clocks.stop()
        shutil.rmtree(tmp, ignore_errors=True)


# --------------------------------------------------------------------------- a short run for profilers
def run_probe(args) -> int:
    """`--probe decode|prefill`: a few steps of one kind on a model of `--layers` layers (default 4), with
    the CUDA profiler range switched on around the last ones, for `ncu --profile-from-start off`.  Prints a
    line with the device time of the unprofiled steps; nothing here is a benchmark value."""
    import numpy as np
    import torch

    from logssms_b200.config import make_model_config
    from logssms_b200.engine import LLM, StepEntry
    from logssms_b200.sampling import SamplingParams
    from logssms_b200.weights import write_random_model

    cfg = dict(MODEL)
    cfg["num_hidden_layers"] = args.layers or 4
    tmp = tempfile.mkdtemp(prefix="logssms_b200_probe_")
    try:
        write_random_model(make_model_config(cfg), tmp, seed=0, dtype=torch.bfloat16)
        llm = LLM(tmp, "bfloat16", max_running_requests=64, max_seq_len_override=MAX_SEQ_LEN, max_prefill_tokens=8192)
        rng = np.random.default_rng(0)
        if args.probe == "decode":
            sp = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True)
            reqs = [llm.add_request(rng.integers(0, cfg["vocab_size"], CONTEXT - 1).tolist(), sp) for _ in range(args.batch)]
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
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (both are reported)")
    ap.add_argument("--prefill-budget", type=int, default=8192, help="token budget of one scheduled step")
    ap.add_argument("--reference-timeout", type=int, default=900, help="seconds the reference arm may take")
    ap.add_argument("--probe", choices=["decode", "prefill"], default=None,
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
