"""The plain implementation against the reference's own code, and against itself.

`tests/golden/reference_blocks.safetensors` holds what the parts of dakingffo/LogSSMs that run on a
CPU produced for the seeded inputs of `tests/golden/make_golden.py` (its Triton kernels under the
Triton interpreter: both norms, both gates, the packed conv; its rotary tables; the recurrence oracle
of its kernel tests).  The functions of tests/plain must reproduce them.

`tests/golden/reference_model_*.safetensors` hold whole-model logits of the unmodified reference, run on a GPU
through its own scheduler and engine on tiny Falcon-H1 models with real (seeded random) weights and every
multiplier off its default (`tests/golden/make_reference_model_golden.py`): the last prompt position and the
decoded tokens of three prompts each, of up to 300 tokens in one step and of up to 2,200 tokens in the reference's
portions of 512.  The plain implementation, given the same weights, must give the same
logits: this pins what no part alone shows (where each multiplier sits, the key multiplier before the rotation,
the feed-forward's output joining the residual in the next norm, attention over the cache, the chunked scan).

Beyond that the plain implementation is checked for what must hold whatever the weights are: causality, and the
cache-free recomputation being independent of what follows a position.
"""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import make_golden                                        # noqa: E402
from plain import falcon_h1_plain as P                    # noqa: E402
from tiny import TINY, TOL, make_model_dir, plain_logits, rel_err       # noqa: E402

# The Triton interpreter converts float32 to bfloat16 by dropping the low bits where a GPU rounds to
# nearest, so the stored bfloat16 outputs sit up to one unit in the last place off per conversion; the
# float32 outputs pin the formulas to 1e-6 and the bfloat16 ones only check that nothing else differs.
BF16_ULP = 2 ** -5          # a chain of up to three truncating conversions


@pytest.fixture(scope="module")
def golden():
    from safetensors.torch import load_file
    return load_file(os.path.join(HERE, "golden", "reference_blocks.safetensors")), make_golden.inputs()


def near(got, want, tag):
    tol = 1e-6 if tag == "f32" else BF16_ULP
    got, want = got.double(), want.double()
    err = float((got - want).abs().max() / want.abs().max())
    assert err <= tol, f"error {err:.3g} > {tol}"


def rounder(tag):
    return P._rounder(None if tag == "f32" else torch.bfloat16)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_norms_match_the_reference_kernels(golden, tag):
    out, t = golden
    f = lambda n: t[f"{n}.{tag}"].float()
    rnd = rounder(tag)
    (o0, o1), r = P.rms_norm_branches(f("norm.x"), f("norm.weight"), 1e-5, f("norm.residual"), f("norm.other"),
                                      (0.8, 0.7), (1.5, 1.2), rnd)
    near(o0, out[f"norm.two.out0.{tag}"], tag)
    near(o1, out[f"norm.two.out1.{tag}"], tag)
    near(r, out[f"norm.two.residual.{tag}"], tag)
    (o0,), r = P.rms_norm_branches(f("norm.x"), f("norm.weight"), 1e-6, rnd=rnd)
    near(o0, out[f"norm.one.out0.{tag}"], tag)
    near(r, out[f"norm.one.residual.{tag}"], tag)
    y, gate, w = f("gated.y"), f("gated.gate"), f("gated.weight")
    near(P.gated_group_norm(y, gate, w, 1e-5, 2, True, 0.6, rnd), out[f"gated.before.{tag}"], tag)
    near(P.gated_group_norm(y, gate, w, 1e-5, 3, False, 0.6, rnd), out[f"gated.after.{tag}"], tag)
    near(P.silu_gate(y, gate, 0.6, rnd), out[f"gated.none.{tag}"], tag)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_swiglu_and_conv_match_the_reference_kernels(golden, tag):
    out, t = golden
    f = lambda n: t[f"{n}.{tag}"].float()
    rnd = rounder(tag)
    gu = f("mlp.gate_up")
    act = rnd(rnd(P.silu(rnd(gu[:, :50] * 0.9))) * gu[:, 50:])
    near(act, out[f"mlp.swiglu.{tag}"], tag)
    x = f("conv.x")
    scale = torch.cat([torch.full((8,), 1.1), torch.full((6,), 0.9), torch.full((6,), 1.3)])
    w, b = f("conv.weight")[:, 0, :], f("conv.bias")
    got = torch.cat([P.causal_conv_silu(rnd(x[:75] * scale), w, b, rnd), P.causal_conv_silu(rnd(x[75:] * scale), w, b, rnd)])
    near(got, out[f"conv.out.{tag}"], tag)


def test_recurrence_matches_the_reference_oracle(golden):
    out, t = golden
    xbc, dt = t["ssm.xbc"].float(), t["ssm.dt"].float()
    x, B, C = xbc.split([16, 16, 16], 1)
    rnd = rounder("bf16")
    y = P.ssm_recurrence(x.reshape(11, 2, 8), dt, t["ssm.A_log"], t["ssm.dt_bias"], B.reshape(11, 1, 16),
                         C.reshape(11, 1, 16), t["ssm.D"], 1.0, rnd)
    near(y, rnd(out["ssm.y"]), "bf16")


@pytest.mark.parametrize("name", sorted(make_golden.ROPE_CASES))
def test_rotary_tables_match_the_reference(golden, name):
    out, _ = golden
    hd, rd, theta, scaling = make_golden.ROPE_CASES[name]
    inv = P.rope_inv_freq(rd, theta, scaling)
    angle = torch.arange(make_golden.ROPE_POSITIONS, dtype=torch.float32)[:, None] * inv[None, :]
    assert torch.allclose(torch.cat([angle.cos(), angle.sin()], -1), out[f"rope.{name}"], rtol=0, atol=1e-6)
    # the engine's own frequency code (host side) agrees too
    from logssms_b200.config.specs import RopeSpec
    from logssms_b200.parts.rope import inverse_frequencies
    spec = RopeSpec(hd, rd, theta, make_golden.ROPE_POSITIONS, tuple(sorted(scaling.items())) if scaling else None)
    assert torch.equal(inverse_frequencies(spec), inv)


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(0)
    T, Hq, Hkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, h, hd, generator=g, dtype=torch.float64) for h in (Hq, Hkv, Hkv))
    full = P.causal_attention(q, k, v, hd ** -0.5)
    # by hand for one head and one position
    t, h = 5, 3
    s = (q[t, h] @ k[:t + 1, h // 2].T) * hd ** -0.5
    assert torch.allclose(full[t, h], torch.softmax(s, -1) @ v[:t + 1, h // 2])
    # the future does not matter
    k2, v2 = k.clone(), v.clone()
    k2[6:], v2[6:] = 7.0, -3.0
    assert torch.equal(P.causal_attention(q, k2, v2, hd ** -0.5)[:6], full[:6])
    # a window of w keys keeps the query's own position and the w-1 before it
    win = P.causal_attention(q, k, v, hd ** -0.5, window=3)
    s = (q[t, h] @ k[t - 2:t + 1, h // 2].T) * hd ** -0.5
    assert torch.allclose(win[t, h], torch.softmax(s, -1) @ v[t - 2:t + 1, h // 2])
    assert torch.allclose(win[:3], full[:3])


@pytest.mark.parametrize("name", sorted(TINY))
def test_whole_model_logits_do_not_depend_on_later_tokens(tmp_path, name):
    model_dir = make_model_dir(tmp_path / "m", TINY[name], seed=3)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, TINY[name]["vocab_size"], (21,), generator=g).tolist()
    whole = plain_logits(model_dir, ids, "float32")
    assert whole.shape == (21, TINY[name]["vocab_size"]) and torch.isfinite(whole).all()
    prefix = plain_logits(model_dir, ids[:13], "float32")
    assert float((whole[:13] - prefix).abs().max() / whole.abs().max()) < 1e-9
    # bfloat16 rounding points move the result a little, not a lot
    rounded = plain_logits(model_dir, ids, "bfloat16")
    assert float((rounded - whole).abs().max() / whole.abs().max()) < 0.05


@pytest.mark.parametrize("name", ["gate", "gated_norm", "long", "wide"])
def test_whole_model_logits_match_the_reference_engine(tmp_path, name):
    """The reference's own bfloat16 engine on a GPU against the plain implementation on the same weights."""
    import json
    from safetensors import safe_open
    with safe_open(os.path.join(HERE, "golden", f"reference_model_{name}.safetensors"), "pt") as f:
        meta = f.metadata()
        data = {k: f.get_tensor(k) for k in f.keys()}
    raw, seed = json.loads(meta["config"]), int(meta["seed"])
    model_dir = make_model_dir(tmp_path / "m", raw, seed=seed, dtype=torch.bfloat16)
    requests = sorted(int(k.split("_")[1]) for k in data if k.startswith("prompt_"))
    assert len(requests) == 3
    for i in requests:
        prompt, tokens, want = data[f"prompt_{i}"].tolist(), data[f"tokens_{i}"].tolist(), data[f"logits_{i}"]
        got = plain_logits(model_dir, prompt + tokens[:-1], "bfloat16")[len(prompt) - 1:]
        assert got.shape == want.shape
        err = rel_err(got, want)
        assert err <= TOL["bfloat16"], f"{name}, prompt of {len(prompt)} tokens: error {err:.3g}"
        # the reference's greedy choice is the plain model's, or within the tolerance of it
        for row, tok in zip(got, tokens):
            assert float(row.max() - row[tok]) / float(row.abs().max()) <= TOL["bfloat16"]
