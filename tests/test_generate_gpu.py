"""Generation through the public entry points: `LLM.generate`, the scheduler underneath it, and the
command line, on tiny random Falcon-H1 models, against the plain implementation.

Greedy tokens are checked one by one: the engine's choice must be the plain implementation's argmax of
the whole sequence so far, or within the tolerance of it when two logits nearly tie.
"""
import subprocess
import sys

import pytest
import torch

from tiny import TINY, TOL, make_model_dir, plain_logits

pytestmark = pytest.mark.gpu


def check_greedy(model_dir, dtype, prompt, tokens):
    ids = list(prompt)
    exact = 0
    for tok in tokens:
        logits = plain_logits(model_dir, ids, dtype)[-1]
        best = int(logits.argmax())
        gap = float(logits[best] - logits[tok]) / float(logits.abs().max())
        assert gap <= TOL[dtype], f"engine chose {tok}, plain implementation {best} (gap {gap:.3g}) after {len(ids)} tokens"
        exact += int(tok == best)
        ids.append(tok)
    return exact


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_of_several_prompts_through_a_small_pool(tmp_path, name, dtype):
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    raw = TINY[name]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=21, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for n in (1, 5, 13, 70, 33)]
    new = 12
    # 3 pages of 64: the 70-token prompt with its 12 new tokens takes two of them, so requests queue and
    # pages and state slots are used again; the token budget of 24 cuts the longer prompts into portions
    llm = LLM(model_dir, dtype, max_running_requests=3, max_seq_len_override=128, num_pages=3, max_prefill_tokens=24,
              poison_on_free=True)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o.finish_reason for o in outs] == ["length"] * len(prompts)
    exact = sum(check_greedy(model_dir, dtype, p, o.token_ids) for p, o in zip(prompts, outs))
    assert all(len(o.token_ids) == new for o in outs)
    assert exact >= 0.8 * new * len(prompts)
    llm.engine.cache.check_integrity()
    assert not llm.engine.cache.live
    # a second call on the same engine reuses everything and gives the same tokens
    again = llm.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o.token_ids for o in again] == [o.token_ids for o in outs[:2]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("policy", [("prefill-first", None), ("mixed", 8)])
def test_the_other_scheduling_policies_drive_the_real_engine(tmp_path, policy, dtype):
    """`prefill-first` (a step is prompt portions or decoded tokens, never both) and a cap on the prompt tokens of a step
    that also decodes, through the real engine and a small pool: the steps have the promised shapes and every token
    is the plain implementation's choice."""
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    name, cap = policy
    raw = TINY["B"]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=27, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for n in (40, 3, 61, 17, 29)]
    new = 10
    llm = LLM(model_dir, dtype, max_running_requests=3, max_seq_len_override=128, num_pages=4, max_prefill_tokens=24,
              poison_on_free=True, scheduling_policy=name, mixed_prefill_tokens=cap)
    steps = []
    inner = llm.engine.step

    def recording(entries, device_tokens=None):
        steps.append([len(e.tokens) if e.tokens is not None else 1 for e in entries])
        return inner(entries, device_tokens)
    llm.engine.step = recording
    planned = llm.engine.run_prepared

    def recording_planned(handle, token_ids):     # a decode step that was planned ahead: single tokens only
        steps.append([1] * len(token_ids))
        return planned(handle, token_ids)
    llm.engine.run_prepared = recording_planned
    llm.scheduler.overlap = False                  # every step with its ids through the host: all of them are recorded
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o.finish_reason for o in outs] == ["length"] * len(prompts) and all(len(o.token_ids) == new for o in outs)
    for p, o in zip(prompts, outs):
        check_greedy(model_dir, dtype, p, o.token_ids)
    portions = [[n for n in st if n > 1] for st in steps]
    singles = [sum(n == 1 for n in st) for st in steps]
    assert any(portions) and any(singles)
    if name == "prefill-first":
        # a 1-token rest of a prompt looks like a decoded token: steps with portions hold at most such rests beside them
        assert all(not (pt and sg) or sum(pt) + sg <= 24 for pt, sg in zip(portions, singles))
        assert all(sum(st) <= 24 for st in steps)
        mixed_steps = sum(1 for pt, sg in zip(portions, singles) if pt and sg)
        assert mixed_steps <= len(prompts)          # only where a prompt's last portion is a single token
    else:
        assert all(sum(pt) <= cap for pt, sg in zip(portions, singles) if sg and pt), steps
        assert any(sum(pt) > cap for pt, sg in zip(portions, singles) if not sg), steps
    llm.engine.cache.check_integrity()
    assert not llm.engine.cache.live


def test_eos_and_max_tokens_end_requests(tmp_path):
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    model_dir = make_model_dir(tmp_path / "m", TINY["A"], seed=22)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    free = LLM(model_dir, "float32", max_running_requests=2, max_seq_len_override=64, num_pages=2)
    tokens = free.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids
    del free
    stop_at = tokens[3]
    first = tokens.index(stop_at)
    llm = LLM(model_dir, "float32", max_running_requests=2, max_seq_len_override=64, num_pages=2, eos_token_ids=[stop_at])
    out = llm.generate([prompt], SamplingParams(max_tokens=8))[0]
    assert out.finish_reason == "stop" and out.token_ids == tokens[:first + 1]
    out = llm.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0]
    assert out.finish_reason == "length" and out.token_ids == tokens
    # prompt + max_tokens beyond the sequence limit: clamped, not refused
    out = llm.generate([list(range(60))], SamplingParams(max_tokens=50, ignore_eos=True))[0]
    assert len(out.token_ids) == 4 and out.finish_reason == "length"


def test_overlapped_decoding_gives_the_same_tokens_and_notices_eos_one_step_late(tmp_path):
    """With the next step launched before the previous ids are read, outputs are the same as without, for
    requests that end by length, by an end-of-sequence id (noticed a step late, the extra step discarded)
    and at different times."""
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    model_dir = make_model_dir(tmp_path / "m", TINY["B"], seed=31)
    prompts = [[5, 6, 7, 8], [9, 10], [11, 12, 13, 14, 15, 16]]
    params = [SamplingParams(max_tokens=9, ignore_eos=True), SamplingParams(max_tokens=20), SamplingParams(max_tokens=14)]
    probe = LLM(model_dir, "float32", max_running_requests=4, max_seq_len_override=128, num_pages=6)
    free = probe.generate(prompts, [SamplingParams(max_tokens=20, ignore_eos=True)] * 3)
    eos = free[1].token_ids[6]                              # an id the second request reaches after a few tokens
    del probe
    results = {}
    for overlap in (False, True):
        llm = LLM(model_dir, "float32", max_running_requests=4, max_seq_len_override=128, num_pages=6, eos_token_ids=[eos])
        llm.scheduler.overlap = overlap
        outs = llm.generate(prompts, params)
        results[overlap] = [(o.token_ids, o.finish_reason) for o in outs]
        assert llm.scheduler.steps > 0 and not llm.engine.cache.live
        # without overlap the next decode step is planned while the device runs this one; some of those plans are
        # dropped here (a request ends, by its end-of-sequence id too), the others run once their ids have come
        assert (llm.scheduler.steps_ahead > 0) == (not overlap)
        llm.engine.cache.check_integrity()
        del llm
    assert results[True] == results[False]
    assert results[True][0][1] == "length" and len(results[True][0][0]) == 9
    assert results[True][1][1] == "stop" and results[True][1][0][-1] == eos


def test_temperature_sampling_is_seeded_per_request_and_independent_of_the_batch(tmp_path):
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    model_dir = make_model_dir(tmp_path / "m", TINY["B"], seed=23)
    llm = LLM(model_dir, "float32", max_running_requests=4, max_seq_len_override=128, num_pages=8, seed=7)
    prompt, other = [9, 8, 7, 6, 5], [1, 2, 3]
    sp = SamplingParams(temperature=0.9, top_k=20, top_p=0.95, max_tokens=10, ignore_eos=True, seed=1234)
    alone = llm.generate([prompt], sp)[0].token_ids
    crowd = llm.generate([other, prompt, other], [SamplingParams(temperature=1.3, max_tokens=6, ignore_eos=True, seed=5), sp,
                                                  SamplingParams(max_tokens=3, ignore_eos=True)])
    assert crowd[1].token_ids == alone                          # same seed, same draws, whatever else is in the batch
    assert llm.generate([prompt], sp)[0].token_ids == alone
    other_seed = SamplingParams(temperature=0.9, top_k=20, top_p=0.95, max_tokens=10, ignore_eos=True, seed=99)
    assert llm.generate([prompt], other_seed)[0].token_ids != alone
    greedy = llm.generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0].token_ids
    assert greedy != alone


def test_command_line_generates_from_random_weights(tmp_path):
    """`python -m logssms_b200 --model-path DIR --dummy-weight --prompt-ids ...` needs only a config.json."""
    import json
    import os
    cfg_dir = tmp_path / "cfg"
    cfg_dir.mkdir()
    (cfg_dir / "config.json").write_text(json.dumps(TINY["A"]))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "logssms_b200", "--model-path", str(cfg_dir), "--dummy-weight", "--dtype", "float32",
           "--seed", "3", "--max-seq-len-override", "64", "--num-pages", "2", "--max-running-requests", "2",
           "--temperature", "0", "--max-tokens", "5", "--ignore-eos", "--prompt-ids", "5,6,7"]
    first = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300)
    assert first.returncode == 0, first.stderr[-2000:]
    ids = [int(t) for t in first.stdout.split()]
    assert len(ids) == 5 and all(0 <= t < TINY["A"]["vocab_size"] for t in ids)
    # ... and they are the plain implementation's tokens for the weights that seed gives
    from logssms_b200.config import make_model_config
    from logssms_b200.weights import write_random_model
    same_weights = write_random_model(make_model_config(TINY["A"]), str(tmp_path / "same"), seed=3, dtype=torch.float32)
    check_greedy(same_weights, "float32", [5, 6, 7], ids)
    second = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300)
    assert second.stdout == first.stdout                         # seeded weights, greedy: the same ids again


def word_tokenizer(model_dir, vocab_size):
    """The smallest tokenizer folder `AutoTokenizer` reads: words t0 .. t<V-2> and an end-of-sequence word."""
    import json
    import os
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {f"t{i}": i for i in range(vocab_size - 1)}
    vocab["<eos>"] = vocab_size - 1
    tok = Tokenizer(models.WordLevel(vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(model_dir, "tokenizer.json"))
    with open(os.path.join(model_dir, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "unk_token": "t0"}, f)


def test_text_prompts_go_through_the_folders_tokenizer_and_the_chat_loop(tmp_path):
    import io
    from logssms_b200.cli import Chat
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    raw = TINY["A"]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=24)
    word_tokenizer(model_dir, raw["vocab_size"])
    llm = LLM(model_dir, "float32", max_running_requests=2, max_seq_len_override=128, num_pages=4)
    assert llm.tokenizer is not None and llm.scheduler.eos == {raw["vocab_size"] - 1}
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    by_text = llm.generate(["t5 t17 t3 t200"], sp)[0]
    by_ids = llm.generate([[5, 17, 3, 200]], sp)[0]
    assert by_text.prompt_token_ids == [5, 17, 3, 200] and by_text.token_ids == by_ids.token_ids
    assert by_text.text == " ".join(f"t{i}" if i < raw["vocab_size"] - 1 else "<eos>" for i in by_text.token_ids)
    check_greedy(model_dir, "float32", [5, 17, 3, 200], by_text.token_ids)
    # the chat loop on the real engine: two turns of one conversation, the second sees the first
    out = io.StringIO()
    chat = Chat(llm, sp, system=None, out=out)
    chat.loop(iter(["t5 t17 t3 t200", "t9", "/history", "/exit"]))
    said = out.getvalue().splitlines()
    assert said[0] == by_text.text
    turns = chat.conversations["chat-1"]
    assert [r for r, _ in turns] == ["user", "assistant", "user", "assistant"]
    second_prompt = llm.tokenizer.encode("\n".join(["t5 t17 t3 t200", by_text.text, "t9"]))
    assert llm.tokenizer.decode(llm.generate([list(second_prompt)], sp)[0].token_ids) == turns[3][1]
    # without a tokenizer a text prompt is refused with a clear error
    bare = make_model_dir(tmp_path / "bare", raw, seed=24)
    with pytest.raises(ValueError, match="tokenizer"):
        LLM(bare, "float32", max_running_requests=2, max_seq_len_override=64, num_pages=2).generate(["t1"], sp)


def test_a_kernel_that_gave_up_ends_the_requests_of_its_step_with_an_error(tmp_path):
    """The error word that the kernels with bounded waits write is read with every step's sampled ids.  Here the
    host sets the word itself (no kernel is made to give up): the next step's requests end with an error, the
    word is cleared, the cache is whole, and the engine goes on."""
    from logssms_b200.engine import LLM
    from logssms_b200.ops import kernels as K
    from logssms_b200.sampling import SamplingParams
    model_dir = make_model_dir(tmp_path / "m", TINY["A"], seed=25)
    llm = LLM(model_dir, "float32", max_running_requests=2, max_seq_len_override=64, num_pages=2)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    good = llm.generate([[1, 2, 3]], sp)[0].token_ids
    word = K.error_word(llm.engine.device)
    word.fill_((3 << 24) | (17 << 12) | 5)
    a = llm.add_request([1, 2, 3], sp)
    b = llm.add_request([4, 5], sp)
    with pytest.raises(K.KernelError, match="role 3, block 17, step 5"):
        llm.scheduler.run()
    assert a.state == b.state == "finished" and a.finish_reason.startswith("error") and b.finish_reason.startswith("error")
    assert int(word.item()) == 0 and not llm.engine.cache.live and not llm.scheduler.has_work
    llm.engine.cache.check_integrity()
    assert llm.generate([[1, 2, 3]], sp)[0].token_ids == good
    word.fill_(7)
    with pytest.raises(K.KernelError):
        K.check_kernel_errors(llm.engine.device)
    K.check_kernel_errors(llm.engine.device)        # cleared by the report


def test_profile_times_every_kernel_by_class_and_changes_no_token(tmp_path):
    """`profile=True`: CUDA events around every launch, summed per kernel class; `nvtx=True`: named ranges per layer
    and part.  The tokens are those of an ordinary run."""
    import json
    from logssms_b200.engine import LLM
    from logssms_b200.ops.profiler import PROFILER
    from logssms_b200.sampling import SamplingParams
    model_dir = make_model_dir(tmp_path / "m", TINY["D"], seed=26, dtype=torch.bfloat16)
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    prompts = [list(range(3, 150)), [7, 8, 9]]
    plain_run = [o.token_ids for o in LLM(model_dir, "bfloat16", max_running_requests=2, max_seq_len_override=256,
                                           num_pages=8).generate(prompts, sp)]
    llm = LLM(model_dir, "bfloat16", max_running_requests=2, max_seq_len_override=256, num_pages=8, profile=True, nvtx=True)
    assert not llm.engine.use_graphs and PROFILER.enabled and PROFILER.nvtx
    assert [o.token_ids for o in llm.generate(prompts, sp)] == plain_run
    report = llm.engine.profile_report()
    assert report["steps"] >= 5
    for cls in ("attention", "mamba2", "products", "norms and gates", "embedding", "sampling"):
        assert report["classes"][cls]["launches"] > 0 and report["classes"][cls]["ms"] > 0, cls
    assert any(k.startswith("attention_prefill_tc.") for k in report["kernels"])       # the prompt ran on the tcgen05 kernel
    assert abs(sum(c["ms"] for c in report["classes"].values()) - sum(k["ms"] for k in report["kernels"].values())) < 1e-3
    json.dumps(report)
    # the engine made next switches the profiler off again
    LLM(model_dir, "bfloat16", max_running_requests=2, max_seq_len_override=256, num_pages=8)
    assert not PROFILER.enabled and not PROFILER.nvtx


@pytest.mark.parametrize("name", ["gate", "gated_norm", "long", "wide"])
def test_engine_logits_match_the_reference_engines_golden_logits(tmp_path, name):
    """The stored whole-model logits of the unmodified reference (tests/golden/make_reference_model_golden.py): this
    engine on the same weights, the prompt in one step and the reference's own tokens decoded one by one."""
    import json
    import os
    from safetensors import safe_open
    from logssms_b200.engine import Engine, StepEntry
    from tiny import rel_err
    here = os.path.dirname(os.path.abspath(__file__))
    with safe_open(os.path.join(here, "golden", f"reference_model_{name}.safetensors"), "pt") as f:
        meta = f.metadata()
        data = {k: f.get_tensor(k) for k in f.keys()}
    raw, seed = json.loads(meta["config"]), int(meta["seed"])
    model_dir = make_model_dir(tmp_path / "m", raw, seed=seed, dtype=torch.bfloat16)
    engine = Engine(model_dir, "bfloat16", max_requests=2, max_seq_len=2560, num_pages=40, poison_on_free=True)
    for i in range(3):
        prompt, tokens, want = data[f"prompt_{i}"].tolist(), data[f"tokens_{i}"].tolist(), data[f"logits_{i}"]
        r = engine.new_request()
        rows = [engine.step([StepEntry(r, prompt, [len(prompt) - 1])]).float().cpu()]
        for tok in tokens[:-1]:
            rows.append(engine.step([StepEntry(r, [tok], [0])]).float().cpu())
        engine.release(r)
        err = rel_err(torch.cat(rows), want)
        assert err <= TOL["bfloat16"], f"{name}, prompt of {len(prompt)} tokens: error {err:.3g}"
    engine.cache.check_integrity()
