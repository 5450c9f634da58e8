"""Each part of a layer alone on the GPU against the plain functions, at sizes of its own: norm,
position encoding, attention (through the page cache, in portions), Mamba2 (through its state slots,
in portions), feed-forward, embedding and head, a block with a single mixer, and a layer schedule that
runs a layer twice and lets a layer read another layer's keys and values.

The parts get their tensors the way a model does (declared `param_specs`, drawn by their own
initialisers, placed by the loader's rules), a cache manager sized from their own `cache_needs`, and a
step context from the engine's planner; no model file is involved.
"""
import pytest
import torch

from plain import falcon_h1_plain as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def close(got, want, dtype, tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (tol or TOL[dtype]), f"error {err:.3g}"


def rounder(dtype):
    return P._rounder(None if dtype == torch.float32 else dtype)


def ref_dtype(dtype):
    return torch.float64 if dtype == torch.float32 else torch.float32


def give_weights(part, dtype, seed=0):
    """Draw the part's tensors from its own declarations, place them as the loader would, bind them.
    Returns the stored (CPU) tensors by name for the plain side."""
    from logssms_b200.weights.loader import check_and_place
    from logssms_b200.weights.random_init import random_tensors
    stored = random_tensors(part, seed, dtype)
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    return stored


def runtime(dtype, max_seq_len=256, page_size=16):
    from logssms_b200.parts import Runtime
    return Runtime(torch.device("cuda"), dtype, max_seq_len, page_size)


def cache_for(needs, dtype, num_pages=40, max_requests=4, max_seq_len=256, page_size=16):
    from logssms_b200.cache import CacheManager
    from logssms_b200.engine import StepPlanner
    cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                         max_seq_len=max_seq_len, dtype=dtype, device="cuda", poison_on_free=True)
    return cache, StepPlanner(cache, "cuda")


def step_in_portions(planner, cache, lengths, cuts, run):
    """Run every request's rows through `run(ctx, rows)` in the portions `cuts` (a list of lists of
    portion sizes; 0 leaves the request out of that step).  Returns per request the concatenated output."""
    from logssms_b200.engine import StepEntry
    reqs = [cache.admit() for _ in lengths]
    done = [0] * len(lengths)
    outs = [[] for _ in lengths]
    for step in cuts:
        entries, spans = [], []
        for r, n in enumerate(step):
            n = min(n, lengths[r] - done[r])
            if n > 0:
                entries.append(StepEntry(reqs[r], [0] * n))
                spans.append((r, done[r], done[r] + n))
        if not entries:
            continue
        ctx = planner.plan(entries)
        y = run(ctx, spans)
        at = 0
        for r, lo, hi in spans:
            outs[r].append(y[at:at + hi - lo].float().cpu())
            at += hi - lo
            done[r] = hi
    assert done == list(lengths)
    for rq in reqs:
        cache.release(rq)
    cache.check_integrity()
    return [torch.cat(o) for o in outs]


CUTS = [[37, 0, 9], [5, 20, 1], [1, 1, 1], [64, 3, 1], [1, 30, 2], [200, 200, 200]]
LENGTHS = [120, 61, 40]


# --------------------------------------------------------------------------- norm, rope, MLP, embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from logssms_b200.config.specs import NormSpec
    from logssms_b200.parts import RMSNorm
    norm = RMSNorm(NormSpec(72, 3e-6), perturb_init=True)
    w = give_weights(norm, dtype)
    g = torch.Generator().manual_seed(1)
    x, other, res = (torch.randn(11, 72, generator=g).to(dtype) for _ in range(3))
    rd, rnd = ref_dtype(dtype), rounder(dtype)
    (a, b), r = norm.forward(x.cuda(), res.cuda().clone(), other=other.cuda(), in_scales=(0.8, 0.7), out_scales=(1.5, 1.2))
    (wa, wb), wr = P.rms_norm_branches(x.to(rd), w["weight"].to(rd), 3e-6, res.to(rd), other.to(rd), (0.8, 0.7), (1.5, 1.2), rnd)
    close(a, wa, dtype), close(b, wb, dtype), close(r, wr, dtype)


def test_rotary_part_builds_the_reference_table():
    from logssms_b200.config.specs import RopeSpec
    from logssms_b200.parts import RotaryEmbedding
    scaling = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64}
    spec = RopeSpec(48, 24, 1e5, 4096, tuple(sorted(scaling.items())))
    rope = RotaryEmbedding(spec)
    rope.setup(runtime(torch.float32, max_seq_len=300))
    inv = P.rope_inv_freq(24, 1e5, scaling)
    angle = torch.arange(300, dtype=torch.float32)[:, None] * inv[None, :]
    want = torch.cat([angle.cos(), angle.sin()], -1)
    assert rope.table.shape == (300, 24)
    assert float((rope.table.cpu() - want).abs().max()) < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [5, 100])                 # few rows: the weight-streaming kernel; many: the library
def test_gated_mlp_part(dtype, rows):
    from logssms_b200.config.specs import GatedMLPSpec
    from logssms_b200.parts import GatedMLP
    mlp = GatedMLP(GatedMLPSpec(72, 136, 0.9, 1.1))
    w = give_weights(mlp, dtype)
    x = torch.randn(rows, 72, generator=torch.Generator().manual_seed(2)).to(dtype)
    rd, rnd = ref_dtype(dtype), rounder(dtype)
    linear = lambda a, m, b=None: rnd(a @ m.to(rd).T)
    want = P.gated_mlp(x.to(rd), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"], 0.9, 1.1, rnd, linear)
    close(mlp.forward(x.cuda()), want, dtype)
    # the output multiplier left to the norm that reads the output next: the same rows, the same residual
    from logssms_b200.config.specs import NormSpec
    from logssms_b200.parts import RMSNorm
    from logssms_b200.ops import kernels as K
    norm = RMSNorm(NormSpec(72, 1e-5), perturb_init=True)
    give_weights(norm, dtype)
    res = torch.randn(rows, 72, generator=torch.Generator().manual_seed(3)).to(dtype).cuda()
    lazy = mlp.forward(x.cuda(), lazy_scale=True)
    if dtype == torch.bfloat16 and rows > 64:              # the library product: no epilogue for the multiplier
        assert isinstance(lazy, K.ScaledRows) and lazy.scale == pytest.approx(1.1)
        assert torch.equal(lazy.tensor(), mlp.forward(x.cuda()))
    (a,), ra = norm.forward(lazy, res.clone())
    (b,), rb = norm.forward(mlp.forward(x.cuda()), res.clone())
    assert torch.equal(a, b) and torch.equal(ra, rb)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from logssms_b200.parts import Embedding, LMHead
    emb = Embedding(301, 72, 5.0)
    w = give_weights(emb, dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    rd, rnd = ref_dtype(dtype), rounder(dtype)
    x = emb.forward(ids.cuda())
    close(x, rnd(w["weight"].to(rd)[ids.long()] * 5.0), dtype, tol=1e-6)
    tied = LMHead(301, 72, 0.25, emb)
    assert not tied.param_specs()
    logits = tied.forward(x)
    assert logits.dtype == torch.float32
    close(logits, rnd(rnd(x.cpu().to(rd) @ w["weight"].to(rd).T) * 0.25), dtype)
    own = LMHead(301, 72, 0.25, None)
    w2 = give_weights(own, dtype, seed=4)
    close(own.forward(x), rnd(rnd(x.cpu().to(rd) @ w2["weight"].to(rd).T) * 0.25), dtype)


# --------------------------------------------------------------------------- attention through the cache
def plain_attention_part(x, w, spec, rnd, rd, window=None):
    T = x.shape[0]
    lin = lambda a, m: rnd(a @ m.to(rd).T)
    q = lin(x, w["q_proj.weight"]).reshape(T, spec.num_heads, spec.head_dim)
    k = lin(x, w["k_proj.weight"]).reshape(T, spec.num_kv_heads, spec.head_dim)
    v = lin(x, w["v_proj.weight"]).reshape(T, spec.num_kv_heads, spec.head_dim)
    k = rnd(k * spec.key_scale)
    if spec.position is not None:
        inv = P.rope_inv_freq(spec.position.rotary_dim, spec.position.theta, dict(spec.position.scaling) if spec.position.scaling else None)
        pos = torch.arange(T)
        q = P.rope_apply(q, pos, inv, spec.position.rotary_dim, rnd)
        k = P.rope_apply(k, pos, inv, spec.position.rotary_dim, rnd)
    scale = spec.softmax_scale if spec.softmax_scale is not None else spec.head_dim ** -0.5
    o = P.causal_attention(q, k, v, scale, window, rnd).reshape(T, -1)
    return lin(o, w["o_proj.weight"]), (k, v)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("variant", ["rope_partial_gqa", "no_rope_window_mha"])
def test_attention_part_in_portions(dtype, variant):
    from logssms_b200.config.specs import AttentionSpec, RopeSpec
    from logssms_b200.parts import Attention
    if variant == "rope_partial_gqa":
        spec = AttentionSpec(80, 6, 2, 32, RopeSpec(32, 16, 1e5, 4096), key_scale=0.5)
    else:
        spec = AttentionSpec(80, 3, 3, 48, None, key_scale=1.0, softmax_scale=0.2, window=50)
    att = Attention(spec)
    w = give_weights(att, dtype, seed=3)
    for k_ in ("q_proj.weight", "k_proj.weight"):                      # sharpen: single keys stand out
        w[k_] = (w[k_].float() * 12).to(w[k_].dtype)
    from logssms_b200.weights.loader import check_and_place
    att.bind_tree(check_and_place(att, w, dtype, "cuda"))
    att.setup(runtime(dtype))
    cache, planner = cache_for([att.cache_needs()], dtype)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, 80, generator=g).to(dtype) for n in LENGTHS]
    rd, rnd = ref_dtype(dtype), rounder(dtype)

    def run(ctx, spans):
        x = torch.cat([xs[r][lo:hi] for r, lo, hi in spans]).cuda()
        return att.forward(x, ctx, 0)
    got = step_in_portions(planner, cache, LENGTHS, CUTS, run)
    for r, x in enumerate(xs):
        want, _ = plain_attention_part(x.to(rd), w, spec, rnd, rd, spec.window)
        close(got[r], want, dtype)


# --------------------------------------------------------------------------- Mamba2 through its state slots
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("variant", ["gate_only", "norm_before", "norm_after"])
def test_mamba2_part_in_portions(dtype, variant):
    from logssms_b200.config.specs import Mamba2Spec
    from logssms_b200.parts import Mamba2
    gated = variant != "gate_only"
    spec = Mamba2Spec(hidden_size=56, num_heads=6, head_dim=8, state_dim=24, num_groups=3, conv_kernel=3, conv_bias=True,
                      proj_bias=gated, out_bias=True, gated_norm=gated, norm_before_gate=variant == "norm_before",
                      norm_eps=2e-6, multipliers=(0.6, 1.1, 0.9, 1.3, 0.8), chunk_size=32)
    mixer = Mamba2(spec, perturb_init=True)
    w = give_weights(mixer, dtype, seed=6)
    mixer.setup(runtime(dtype))
    cache, planner = cache_for([mixer.cache_needs()], dtype)
    assert not cache.groups and set(cache.states[0]) == {"conv", "ssm"}
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(n, 56, generator=g).to(dtype) for n in LENGTHS]
    rd, rnd = ref_dtype(dtype), rounder(dtype)
    cfg = {"mamba_n_heads": 6, "mamba_d_head": 8, "mamba_d_state": 24, "mamba_n_groups": 3, "mamba_d_conv": 3,
           "ssm_multipliers": list(spec.multipliers), "mamba_rms_norm": gated, "rms_norm_eps": 2e-6,
           "mamba_norm_before_gate": variant == "norm_before"}
    wr = {"m." + k: v.to(rd) for k, v in w.items()}

    def linear(a, m, b=None):
        y = a @ m.T
        return rnd(y if b is None else y + b)

    def run(ctx, spans):
        x = torch.cat([xs[r][lo:hi] for r, lo, hi in spans]).cuda()
        return mixer.forward(x, ctx, 0)
    got = step_in_portions(planner, cache, LENGTHS, CUTS, run)
    for r, x in enumerate(xs):
        close(got[r], P.mamba2_mixer(x.to(rd), wr, "m.", cfg, rnd, linear), dtype)


# --------------------------------------------------------------------------- a block with one mixer
@pytest.mark.parametrize("dtype", DTYPES)
def test_block_with_a_single_mixer_is_the_plain_prenorm_layer(dtype):
    from logssms_b200.config.specs import AttentionSpec, BlockSpec, GatedMLPSpec, MixerSlot, NormSpec, RopeSpec
    from logssms_b200.parts import PreNormParallelBlock
    att = AttentionSpec(64, 4, 2, 16, RopeSpec(16, 16, 1e4, 1024))
    spec = BlockSpec(prefix="layer.", mixers=(MixerSlot(att, "attn.", 1.0, 0.5),), mixer_norm=NormSpec(64, 1e-5),
                     mixer_norm_name="n1.", feed_forward=GatedMLPSpec(64, 96), feed_forward_name="ff.",
                     feed_forward_norm=NormSpec(64, 1e-5), feed_forward_norm_name="n2.")
    block = PreNormParallelBlock(spec, perturb_init=True)
    w = give_weights(block, dtype, seed=8)
    block.setup(runtime(dtype))
    cache, planner = cache_for([block.cache_needs()], dtype)
    g = torch.Generator().manual_seed(9)
    lengths = [70, 33]
    xs = [torch.randn(n, 64, generator=g).to(dtype) for n in lengths]
    rs = [torch.randn(n, 64, generator=g).to(dtype) for n in lengths]
    rd, rnd = ref_dtype(dtype), rounder(dtype)
    out_res = {}

    def run(ctx, spans):
        x = torch.cat([xs[r][lo:hi] for r, lo, hi in spans]).cuda()
        res = torch.cat([rs[r][lo:hi] for r, lo, hi in spans]).cuda()
        y, new_res = block.forward(x, res, ctx, 0)
        at = 0
        for r, lo, hi in spans:
            out_res.setdefault(r, []).append(new_res[at:at + hi - lo].float().cpu())
            at += hi - lo
        return y
    got = step_in_portions(planner, cache, lengths, [[40, 33], [30, 0]], run)
    lin = lambda a, m, b=None: rnd(a @ m.to(rd).T)
    for r in range(2):
        x, res = xs[r].to(rd), rs[r].to(rd)
        (n1,), res1 = P.rms_norm_branches(x, w["n1.weight"].to(rd), 1e-5, res, rnd=rnd)
        a, _ = plain_attention_part(n1, {k[5:]: v for k, v in w.items() if k.startswith("attn.")}, att, rnd, rd)
        (n2,), res2 = P.rms_norm_branches(rnd(a * 0.5), w["n2.weight"].to(rd), 1e-5, res1, rnd=rnd)
        want = P.gated_mlp(n2, w["ff.gate_proj.weight"], w["ff.up_proj.weight"], w["ff.down_proj.weight"], 1.0, 1.0, rnd, lin)
        close(got[r], want, dtype)
        close(torch.cat(out_res[r]), res2, dtype)


# --------------------------------------------------------------------------- the order of layers is data
@pytest.mark.parametrize("dtype", DTYPES)
def test_schedule_runs_a_layer_twice_and_shares_a_cache(dtype):
    """Schedule: layer 0 (cache 0), layer 1 (cache 1), layer 0 again (cache 2), layer 1 again reading
    cache 1 without writing.  The by-hand side runs the same weights in the same order; the last entry
    attends with its own queries over the keys and values that the second entry stored."""
    from logssms_b200.config.specs import (AttentionSpec, BlockSpec, GatedMLPSpec, MixerSlot, ModelSpec, NormSpec,
                                           RopeSpec, ScheduleEntry)
    from logssms_b200.models import DecoderModel
    H = 48
    att = AttentionSpec(H, 3, 1, 16, RopeSpec(16, 16, 1e4, 1024))
    norm = NormSpec(H, 1e-5)
    layers = tuple(BlockSpec(prefix=f"l{i}.", mixers=(MixerSlot(att, "attn."),), mixer_norm=norm, mixer_norm_name="n1.",
                             feed_forward=GatedMLPSpec(H, 64), feed_forward_name="ff.", feed_forward_norm=norm,
                             feed_forward_norm_name="n2.") for i in range(2))
    schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 1, writes_cache=False))
    spec = ModelSpec(vocab_size=97, hidden_size=H, embedding_name="emb.", embedding_multiplier=2.0, lm_head_name="head.",
                     lm_head_multiplier=0.5, tie_word_embeddings=True, final_norm=norm, final_norm_name="fn.",
                     layers=layers, schedule=schedule)
    model = DecoderModel(spec, perturb_init=True)
    assert model.num_cache_layers == 3
    w = give_weights(model, dtype, seed=10)
    model.setup(runtime(dtype))
    cache, planner = cache_for(model.cache_needs(), dtype)
    assert len(cache.groups) == 1 and cache.groups[0].layers == [0, 1, 2]
    from logssms_b200.engine import StepEntry
    ids = torch.randint(0, 97, (45,), generator=torch.Generator().manual_seed(11)).tolist()
    req = cache.admit()
    got = []
    for lo, hi in ((0, 30), (30, 44), (44, 45)):
        ctx = planner.plan([StepEntry(req, ids[lo:hi], list(range(hi - lo)))])
        x, res = model.forward(ctx)
        got.append(model.logits(x, res, ctx.logit_rows).cpu())
    cache.release(req)
    rd, rnd = ref_dtype(dtype), rounder(dtype)
    lin = lambda a, m, b=None: rnd(a @ m.to(rd).T)
    x = rnd(w["emb.weight"].to(rd)[torch.tensor(ids)] * 2.0)
    res, stored = None, {}
    for e in schedule:
        p = f"l{e.layer}."
        (n1,), res = P.rms_norm_branches(x, w[p + "n1.weight"].to(rd), 1e-5, res, rnd=rnd)
        aw = {k[len(p) + 5:]: v for k, v in w.items() if k.startswith(p + "attn.")}
        if e.writes_cache:
            a, stored[e.cache] = plain_attention_part(n1, aw, att, rnd, rd)
        else:
            T = n1.shape[0]
            q = lin(n1, aw["q_proj.weight"]).reshape(T, 3, 16)
            q = P.rope_apply(q, torch.arange(T), P.rope_inv_freq(16, 1e4), 16, rnd)
            k, v = stored[e.cache]
            a = lin(P.causal_attention(q, k, v, 16 ** -0.5, None, rnd).reshape(T, -1), aw["o_proj.weight"])
        (n2,), res = P.rms_norm_branches(a, w[p + "n2.weight"].to(rd), 1e-5, res, rnd=rnd)
        x = P.gated_mlp(n2, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"],
                        1.0, 1.0, rnd, lin)
    (hN,), _ = P.rms_norm_branches(x, w["fn.weight"].to(rd), 1e-5, res, rnd=rnd)
    want = rnd(lin(hN, w["emb.weight"]) * 0.5)
    close(torch.cat(got), want, dtype)
