"""Trace replay at the lengths and batch sizes that the benchmark times, against the plain implementation.

Per (configuration, dtype) one bin/trace_run process replays, through a page pool too small to hold everything at
once (freed memory poisoned with NaN):

  * `whole`: one request of about 2,200 tokens in one step (block tables of 35 pages, the tensor-core prompt
    kernels going round their rings many times, the state pass over 18 chunks, rotation angles above 2,000);
  * `equal`: two requests of that length in equal portions of 512 tokens, so that the step graph of that shape is
    captured and then REPLAYED for other positions and other pages; the last portion is shorter;
  * `tail`: most of such a request in one step, its last 32 tokens one by one;
  * `rows40`, `rows24`: 40 and 24 live requests decoding side by side for 8 steps after short prompts (the
    products, the conv step and the decode attention take other paths above 16 and above 32 rows).

Attention is sharpened in the `-sharp` models so that single far keys decide the logits.
"""
import random

import pytest
import torch

from replay_util import Trace, in_portions, run_trace, tail_decoded, whole
from test_replay_gpu import sharpen
from tiny import TINY, TOL, make_model_dir, plain_logits, rel_err

pytestmark = pytest.mark.gpu

LONG = 2200
SCENARIOS = ("whole", "equal", "tail", "rows40", "rows24")
PAGE_OF = {"E": 128, "T5": 128}        # two configurations replay through pages of 128 tokens

_cache: dict = {}


def replayed(tmp_path_factory, name, dtype):
    key = (name, dtype)
    if key in _cache:
        return _cache[key]
    base = name.split("-")[0]
    raw = TINY[base]
    page = PAGE_OF.get(base, 64)
    tmp = tmp_path_factory.mktemp(f"long_{name}_{dtype}")
    model_dir = make_model_dir(tmp / "model", raw, seed=31 + len(name),
                               dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    if name.endswith("-sharp"):
        sharpen(model_dir)
    rng = random.Random(17)
    V = raw["vocab_size"]
    seqs = {"L0": [rng.randrange(V) for _ in range(LONG)], "L1": [rng.randrange(V) for _ in range(LONG - 77)]}
    for i in range(40):
        seqs[f"s{i}"] = [rng.randrange(V) for _ in range(rng.randint(2, 20) + 8)]
    want = {rid: plain_logits(model_dir, ids, dtype) for rid, ids in seqs.items()}

    trace = Trace(page=page)
    ids_of: dict[str, str] = {}

    def uid(scn, rid):
        ids_of[f"{scn}:{rid}"] = rid
        return f"{scn}:{rid}"
    whole(trace, uid("whole", "L0"), seqs["L0"])
    in_portions(trace, uid("equal", "L0"), seqs["L0"], [512])
    in_portions(trace, uid("equal", "L1"), seqs["L1"], [512])
    tail_decoded(trace, uid("tail", "L1"), seqs["L1"])
    for rows in (40, 24):
        rids = [f"s{i}" for i in range(rows)]
        # prompts (all but the last 8 tokens) in two steps of mixed portions, then 8 steps of `rows` single tokens
        trace.add_step([(uid(f"rows{rows}", r), seqs[r][:len(seqs[r]) - 8]) for r in rids[:rows // 2]])
        trace.add_step([(uid(f"rows{rows}", r), seqs[r][:len(seqs[r]) - 8]) for r in rids[rows // 2:]])
        for j in range(8):
            trace.add_step([(uid(f"rows{rows}", r), [seqs[r][len(seqs[r]) - 8 + j]]) for r in rids],
                           end=[uid(f"rows{rows}", r) for r in rids] if j == 7 else [])
    max_tokens = 40 * page                     # one long request takes 35 pages of 64; forty short ones a page each
    assert trace.peak_tokens <= max_tokens, trace.peak_tokens
    got = run_trace(model_dir, dtype, trace, str(tmp / "out"), max_tokens, V,
                    extra_args=["--poison", "--max-requests", "40", "--page-size", str(page)])
    _cache[key] = (got, want, ids_of, trace)
    return _cache[key]


@pytest.mark.parametrize("scenario", SCENARIOS)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "D-sharp", "E", "T5"])
def test_long_requests_and_many_rows_match_plain(tmp_path_factory, name, dtype, scenario):
    got, want, ids_of, trace = replayed(tmp_path_factory, name, dtype)
    checked = 0
    for u, rid in ids_of.items():
        if u.split(":")[0] != scenario:
            continue
        g = got[u]
        w = want[rid][:g.shape[0]]
        assert g.shape[0] == len(w) and not torch.isnan(g).any(), f"{u}: positions without logits"
        err = rel_err(g, w)
        assert err <= TOL[dtype], f"{name} {dtype} {u}: error {err:.3g} > {TOL[dtype]}; first bad position " \
                                  f"{int(((g - w).abs().amax(1) / w.abs().max() > TOL[dtype]).nonzero()[0])}"
        checked += 1
    assert checked > 0


def test_the_long_trace_has_the_steps_it_claims(tmp_path_factory):
    _, _, _, trace = replayed(tmp_path_factory, "D", "bfloat16")
    sizes = [[len(e["tokens"]) for e in s["entries"]] for s in trace.steps]
    assert [LONG] in sizes and sizes.count([512]) == 8
    assert any(len(s) == 40 and set(s) == {1} for s in sizes) and any(len(s) == 24 and set(s) == {1} for s in sizes)
