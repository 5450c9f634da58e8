"""Trace replay on the GPU against the plain implementation: every way of cutting the same requests.

One bin/trace_run process per (configuration, dtype) replays all scenarios back to back through one
small page pool, so pages and state slots are used again between and within scenarios (freed memory
is poisoned with NaN).  Every position's logits are asked for and compared.
"""
import random

import pytest
import torch

from replay_util import PAGE, Trace, in_portions, mixed, run_trace, tail_decoded, whole
from tiny import TINY, TOL, make_model_dir, plain_logits, rel_err

pytestmark = pytest.mark.gpu

LENGTHS = {"r0": 150, "r1": 97, "r2": 130, "r3": 70, "r4": 3, "r5": 65}
MAX_TOKENS = 8 * PAGE            # eight pages: the mixed scenarios need thirteen over time
SCENARIOS = ("whole", "tail", "portions", "mixed", "long_decode", "first_tokens")


def sharpen(model_dir):
    """Scale the query/key projections so that softmax picks single keys (also far ones) instead
    of averaging: a wrong or missing key then moves the logits by far more than the tolerance."""
    import os
    from safetensors.torch import load_file, save_file
    path = os.path.join(model_dir, "model.safetensors")
    t = load_file(path)
    for k in t:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            t[k] = (t[k].float() * 12.0).to(t[k].dtype)
    save_file(t, path)


_cache: dict = {}


def replayed(tmp_path_factory, name, dtype, state="float32"):
    key = (name, dtype, state)
    if key in _cache:
        return _cache[key]
    base_name = name.split("-")[0]
    raw = TINY[base_name]
    tmp = tmp_path_factory.mktemp(f"replay_{name}_{dtype}_{state}")
    model_dir = make_model_dir(tmp / "model", raw, seed=11 + len(name),
                               dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    if name.endswith("-sharp"):
        sharpen(model_dir)
    rng = random.Random(7)
    seqs = {rid: [rng.randrange(raw["vocab_size"]) for _ in range(n)] for rid, n in LENGTHS.items()}
    want = {rid: plain_logits(model_dir, ids, dtype) for rid, ids in seqs.items()}

    trace = Trace()
    ids_of: dict[str, str] = {}         # unique trace id -> base request
    def uid(scn, rid):
        u = f"{scn}:{rid}"
        ids_of[u] = rid
        return u
    for rid, ids in seqs.items():
        whole(trace, uid("whole", rid), ids)
    for rid in ("r0", "r1", "r5"):
        tail_decoded(trace, uid("tail", rid), seqs[rid])
    in_portions(trace, uid("portions", "r0"), seqs["r0"], [7, 2, 16, 3, 33, 2, 64, 5])
    in_portions(trace, uid("portions", "r2"), seqs["r2"], [2, 62, 2, 3, 61])       # lands on and around page edges
    in_portions(trace, uid("portions", "r5"), seqs["r5"], [63, 2])
    mixed(trace, {uid("mixed", rid): seqs[rid] for rid in ("r1", "r3", "r4", "r5", "r0", "r2")}, MAX_TOKENS, seed=3)
    mixed(trace, {uid("mixed2", rid): seqs[rid] for rid in ("r3", "r4", "r5", "r1", "r2", "r0")}, MAX_TOKENS, seed=4,
          prompt_fraction=0.3)
    long_ids = seqs["r0"]
    trace.add_step([(uid("long_decode", "r0"), long_ids[:5])])
    for i in range(5, len(long_ids)):
        trace.add_step([(uid("long_decode", "r0"), long_ids[i:i + 1])],
                       end=[uid("long_decode", "r0")] if i == len(long_ids) - 1 else [])
    for n in (1, 2, 3):
        whole(trace, uid(f"first_tokens{n}", "r1"), seqs["r1"][:n])
    assert trace.peak_tokens <= MAX_TOKENS, trace.peak_tokens
    got = run_trace(model_dir, dtype, trace, str(tmp / "out"), MAX_TOKENS, raw["vocab_size"],
                    extra_args=["--poison", "--ssm-state-dtype", state])
    _cache[key] = (got, want, ids_of, trace)
    return _cache[key]


@pytest.mark.parametrize("scenario", SCENARIOS)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "Bl", "C", "D", "E", "B-sharp", "D-sharp", "R5", "R10", "R11-sharp", "R14"])
def test_replay_matches_plain(tmp_path_factory, name, dtype, scenario):
    got, want, ids_of, trace = replayed(tmp_path_factory, name, dtype)
    checked = 0
    for u, rid in ids_of.items():
        if not u.split(":")[0].startswith(scenario):
            continue
        g = got[u]
        w = want[rid][:g.shape[0]]
        assert not torch.isnan(g).any(), f"{u}: positions without logits"
        err = rel_err(g, w)
        assert err <= TOL[dtype], f"{name} {dtype} {u}: error {err:.3g} > {TOL[dtype]}; first bad position " \
                                  f"{int(((g - w).abs().amax(1) / w.abs().max() > TOL[dtype]).nonzero()[0])}"
        checked += 1
    assert checked > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_scenario_really_mixes_and_reuses_pages(tmp_path_factory, dtype):
    _, _, _, trace = replayed(tmp_path_factory, "B", dtype)
    mixed_steps = [s for s in trace.steps if any(e["id"].startswith("mixed") for e in s["entries"])]
    assert any(len(s["entries"]) == 4 for s in mixed_steps), "never four live requests in a step"
    assert any(len({len(e["tokens"]) > 1 for e in s["entries"]}) == 2 for s in mixed_steps), \
        "never a prompt portion beside a decoded token"
    assert any(len(e["tokens"]) == 2 for s in mixed_steps for e in s["entries"]), "no two-token portion"
    total = sum(-(-n // PAGE) for n in LENGTHS.values())
    assert total * 2 > MAX_TOKENS // PAGE, "the pool is not small enough to force reuse"


@pytest.mark.parametrize("name", ["D", "R14"])
def test_replay_with_the_recurrent_state_kept_in_bfloat16(tmp_path_factory, name):
    """`--ssm-state-dtype activation` (the reference's way of keeping the state): every cutting of the same requests
    within the same tolerance of the plain implementation, which never rounds the state."""
    got, want, ids_of, trace = replayed(tmp_path_factory, name, "bfloat16", state="activation")
    for u, rid in ids_of.items():
        g = got[u]
        assert not torch.isnan(g).any(), f"{u}: positions without logits"
        err = rel_err(g, want[rid][:g.shape[0]])
        assert err <= TOL["bfloat16"], f"{name} {u}: error {err:.3g}"
