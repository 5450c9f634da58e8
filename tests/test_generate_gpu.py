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
    second = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300)
    assert second.stdout == first.stdout                         # seeded weights, greedy: the same ids again
