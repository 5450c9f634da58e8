"""Plain, slow Falcon-H1: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the
`logssms_b200` package: it reads the raw config.json mapping and the raw
safetensors name -> tensor mapping, and computes the logits of every position
of one whole sequence with ordinary torch tensor maths on the CPU.

It rests on the formulas of the reference (dakingffo/LogSSMs); every function
cites the file:line it was written from.  Where the reference's own kernels can
run on the CPU (its Triton kernels under the Triton interpreter), the functions
here were compared with them once: see tests/golden/make_golden.py and the
stored outputs next to it.  The whole model was compared once with the
reference's own bfloat16 engine on a GPU, on tiny models with real weights:
tests/golden/make_reference_model_golden.py and the logits stored next to it
(tests/test_plain.py checks both).

Two knobs, both about arithmetic only:
  * `compute`: the dtype all maths runs in (float64 for an oracle of the 32-bit
    engine, float32 otherwise).
  * `act`: None, or torch.bfloat16 to round to bfloat16 wherever the reference's
    bfloat16 engine stores an activation ("rounded to act" in its kernels).
"""
from __future__ import annotations

import math
from typing import Mapping

import torch


def _rounder(act):
    if act is None:
        return lambda t: t
    return lambda t: t.to(act).to(t.dtype)


# --------------------------------------------------------------------------- norms
def rms_norm_branches(x, weight, eps, residual=None, other=None, in_scales=(1.0, 1.0),
                      out_scales=(1.0,), rnd=lambda t: t):
    """Residual add + RMSNorm with one or two scaled outputs.

    python/logssms/kernel/norm.py:16-35: with a second input, the two inputs are
    scaled, each rounded, summed and rounded; the residual is added in 32-bit;
    the sum is stored (rounded) as the new residual while the statistics use the
    unrounded sum; the normalised row is rounded, then scaled per output.
    Returns (outputs, new_residual)."""
    if other is not None:
        x = rnd(rnd(x * in_scales[0]) + rnd(other * in_scales[1]))
    if residual is not None:
        x = x + residual
    new_residual = rnd(x)
    variance = (x * x).mean(-1, keepdim=True)
    normalized = rnd(x * torch.rsqrt(variance + eps) * weight)
    return tuple(rnd(normalized * s) for s in out_scales), new_residual


def silu(v):
    return v * torch.sigmoid(v)


def gated_group_norm(y, gate, weight, eps, groups, before_gate, gate_scale, rnd=lambda t: t):
    """Grouped RMSNorm with a SiLU gate.

    python/logssms/kernel/norm.py:55-86: gate scaled and rounded; z = silu(gate)
    in 32-bit; norm over each group of width/groups channels either before the
    gate is applied (`before_gate`) or on the gated values."""
    T, width = y.shape
    z = silu(rnd(gate * gate_scale))
    yg = y.reshape(T, groups, width // groups)
    zg = z.reshape(T, groups, width // groups)
    wg = weight.reshape(groups, width // groups)
    if not before_gate:
        yg = yg * zg
    variance = (yg * yg).mean(-1, keepdim=True)
    out = yg * torch.rsqrt(variance + eps) * wg
    if before_gate:
        out = out * zg
    return rnd(out.reshape(T, width))


def silu_gate(y, gate, gate_scale, rnd=lambda t: t):
    """y * silu(gate * scale) when the mixer has no norm.
    python/logssms/kernel/fused.py:9-19: the scaled gate is rounded, and so is
    its SiLU, before the product."""
    g = rnd(gate * gate_scale)
    return rnd(y * rnd(silu(g)))


# --------------------------------------------------------------------------- rotary
def rope_inv_freq(rotary_dim, theta, scaling=None):
    """Inverse frequencies, with the `llama3` / `yarn` post-processing.
    python/logssms/layers/rotary.py:24-26 and :63-122.  Always float32 there."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return inv
    if kind == "llama3":
        factor = scaling["factor"]
        low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
        orig = scaling["original_max_position_embeddings"]
        wave = 2 * math.pi / inv
        if low == high:
            return torch.where(wave < orig / high, inv, inv / factor)
        smooth = torch.clamp((orig / wave - low) / (high - low), 0, 1)
        return ((1 - smooth) / factor + smooth) * inv
    if kind == "yarn":
        factor = scaling["factor"]
        beta_fast, beta_slow = scaling.get("beta_fast", 32.0), scaling.get("beta_slow", 1.0)
        orig = scaling["original_max_position_embeddings"]

        def corr(rot):
            return rotary_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))
        lo = max(math.floor(corr(beta_fast)), 0)
        hi = min(math.ceil(corr(beta_slow)), rotary_dim // 2 - 1)
        ramp = torch.clamp((torch.arange(rotary_dim // 2, dtype=torch.float32) - lo) / max(hi - lo, 1), 0, 1)
        return (inv / factor) * ramp + inv * (1 - ramp)
    raise ValueError(f"Unsupported rope_scaling {scaling!r}")


def rope_apply(x, positions, inv_freq, rotary_dim, rnd=lambda t: t):
    """Half-split rotation of the first `rotary_dim` columns of every head.

    python/logssms/kernel/fused.py:186-194 with the float32 cos/sin table of
    python/logssms/layers/rotary.py:27-32 (angle = position * inv_freq in float32).
    x: [T, heads, head_dim]."""
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # float32, as the table
    cos, sin = angle.cos().to(x.dtype)[:, None, :], angle.sin().to(x.dtype)[:, None, :]
    half = rotary_dim // 2
    a, b, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
    return rnd(torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1))


# --------------------------------------------------------------------------- attention
def causal_attention(q, k, v, scale, window=None, rnd=lambda t: t):
    """softmax(q k^T * scale + causal mask) v per head, grouped-query.

    Oracle of the reference's model test (tests/hybrid/test_falcon_h1.py:24-37);
    default scale head_dim ** -0.5 (python/logssms/layers/attention_backend/trtllm.py:44).
    q: [T, Hq, hd]; k, v: [T, Hkv, hd].  `window` (not used by Falcon-H1) keeps
    the last `window` keys, the query's own position included."""
    T, Hq, hd = q.shape
    rep = Hq // k.shape[1]
    kk = k.repeat_interleave(rep, 1)
    vv = v.repeat_interleave(rep, 1)
    scores = torch.einsum("thd,shd->hts", q, kk) * scale
    i = torch.arange(T)
    mask = i[None, :] <= i[:, None]
    if window is not None:
        mask &= i[None, :] > i[:, None] - window
    scores = scores.masked_fill(~mask[None], float("-inf"))
    probs = torch.softmax(scores, -1)
    return rnd(torch.einsum("hts,shd->thd", probs, vv))


# --------------------------------------------------------------------------- Mamba2
def causal_conv_silu(u, weight, bias, rnd=lambda t: t):
    """Depthwise causal conv over time, then SiLU.

    python/logssms/kernel/linear_attention/packed_conv.py:96-140: tap j of K
    multiplies the input K-1-j steps back; inputs before the sequence are zero;
    bias added; the sum is rounded, then SiLU.  u: [T, C]; weight: [C, K]."""
    T, C = u.shape
    K = weight.shape[-1]
    padded = torch.cat([u.new_zeros(K - 1, C), u], 0)
    acc = u.new_zeros(T, C)
    for j in range(K):
        acc = acc + padded[j:j + T] * weight[:, j]
    if bias is not None:
        acc = acc + bias
    acc = rnd(acc)
    return rnd(acc / (1.0 + torch.exp(-acc)))


def softplus20(v):
    """softplus with the reference's threshold: v if v > 20 else log1p(exp(v)).
    python/logssms/kernel/linear_attention/mamba2.py:35."""
    return torch.where(v > 20, v, torch.log1p(torch.exp(torch.clamp(v, max=20.0))))


def ssm_recurrence(x, dt_raw, A_log, dt_bias, B, C, D, dt_scale, rnd=lambda t: t):
    """Token-by-token selective state-space recurrence.

    dt and decay: python/logssms/kernel/linear_attention/mamba2.py:27-36;
    recurrence and output: tests/kernel/test_mamba2.py:22-38 (oracle of the
    reference's kernel tests).  x: [T, nh, P]; B, C: [T, G, N]; dt_raw: [T, nh].
    Returns y: [T, nh, P]."""
    T, nh, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = nh // G
    Bh, Ch = B.repeat_interleave(rep, 1), C.repeat_interleave(rep, 1)      # [T, nh, N]
    dt = softplus20(rnd(dt_raw * dt_scale) + dt_bias)                        # [T, nh]
    decay = torch.exp(-torch.exp(A_log) * dt)                                # [T, nh]
    state = x.new_zeros(nh, N, P)
    ys = []
    for t in range(T):
        update = rnd(x[t] * dt[t, :, None])                                  # [nh, P]
        state = state * decay[t, :, None, None] + Bh[t, :, :, None] * update[:, None, :]
        ys.append((state * Ch[t, :, :, None]).sum(1) + D[:, None] * x[t])
    return rnd(torch.stack(ys))


def mamba2_mixer(s_in, w, prefix, cfg, rnd, linear):
    """One Mamba2 mixer on a whole sequence.

    python/logssms/layers/mamba2.py:118-149 (projection split z | xBC | dt, gate
    and output projection) and
    python/logssms/layers/linear_attention_backend/mamba2.py:36-57 (conv with
    the per-region input scales, then the scan)."""
    nh, P = cfg["mamba_n_heads"], cfg["mamba_d_head"]
    N, G, K = cfg["mamba_d_state"], cfg["mamba_n_groups"], cfg["mamba_d_conv"]
    inner = nh * P
    m = cfg["ssm_multipliers"]
    proj = linear(s_in, w[prefix + "in_proj.weight"], w.get(prefix + "in_proj.bias"))
    z, xbc, dt_raw = proj.split([inner, inner + 2 * G * N, nh], -1)
    # per-region scale of the conv input, each product rounded (packed_conv.py:24-29)
    scale = torch.cat([torch.full((inner,), m[1]), torch.full((G * N,), m[2]), torch.full((G * N,), m[3])])
    u = rnd(xbc * scale.to(xbc.dtype))
    conv = causal_conv_silu(u, w[prefix + "conv1d.weight"][:, 0, :], w.get(prefix + "conv1d.bias"), rnd)
    x, B, C = conv.split([inner, G * N, G * N], -1)
    T = x.shape[0]
    y = ssm_recurrence(x.reshape(T, nh, P), dt_raw, w[prefix + "A_log"], w[prefix + "dt_bias"],
                       B.reshape(T, G, N), C.reshape(T, G, N), w[prefix + "D"], m[4], rnd)
    y = y.reshape(T, inner)
    if cfg["mamba_rms_norm"]:
        y = gated_group_norm(y, z, w[prefix + "norm.weight"], cfg["rms_norm_eps"], G,
                             cfg["mamba_norm_before_gate"], m[0], rnd)
    else:
        y = silu_gate(y, z, m[0], rnd)
    return linear(y, w[prefix + "out_proj.weight"], w.get(prefix + "out_proj.bias"))


# --------------------------------------------------------------------------- feed-forward
def gated_mlp(h, w_gate, w_up, w_down, act_scale, out_scale, rnd, linear):
    """down(silu(gate * s0) * up) * s1.
    python/logssms/layers/mlp.py:50-61 and python/logssms/kernel/fused.py:32-50
    (scaled gate rounded, its SiLU rounded, product rounded)."""
    g, u = linear(h, w_gate), linear(h, w_up)
    a = rnd(rnd(silu(rnd(g * act_scale))) * u)
    return rnd(linear(a, w_down) * out_scale)


# --------------------------------------------------------------------------- whole model
def falcon_h1_logits(cfg: Mapping, tensors: Mapping[str, torch.Tensor], ids, *,
                     compute=torch.float64, act=None, window=None):
    """Logits [T, vocab] of every position of one sequence.

    Layer wiring: python/logssms/models/falcon_h1.py:152-185 (shared input norm
    with two scaled outputs; attention and Mamba2 side by side; their scaled sum
    joins the residual inside the pre-feed-forward norm; the MLP output joins it
    inside the next layer's norm), :210-222 (embedding multiplier, final norm),
    :235-237 (lm_head multiplier)."""
    rnd = _rounder(act)
    w = {k: v.to(compute) for k, v in tensors.items()}

    def linear(x, weight, bias=None):
        y = x @ weight.T
        if bias is not None:
            y = y + bias
        return rnd(y)

    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.numel()
    positions = torch.arange(T)
    H = cfg["hidden_size"]
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or Hq
    hd = cfg.get("head_dim") or H // Hq
    eps = cfg["rms_norm_eps"]
    rotary_dim = int(hd * float(cfg.get("partial_rotary_factor", 1.0)))
    inv_freq = rope_inv_freq(rotary_dim, cfg["rope_theta"], cfg.get("rope_scaling"))

    x = rnd(w["model.embed_tokens.weight"][ids] * cfg["embedding_multiplier"])
    residual = None
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        (a_in, s_in), residual = rms_norm_branches(
            x, w[p + "input_layernorm.weight"], eps, residual,
            out_scales=(cfg["attention_in_multiplier"], cfg["ssm_in_multiplier"]), rnd=rnd)
        # attention (python/logssms/layers/attention.py:115-167: key scaled before the rotation)
        q = linear(a_in, w[p + "self_attn.q_proj.weight"]).reshape(T, Hq, hd)
        k = linear(a_in, w[p + "self_attn.k_proj.weight"]).reshape(T, Hkv, hd)
        v = linear(a_in, w[p + "self_attn.v_proj.weight"]).reshape(T, Hkv, hd)
        k = rnd(k * cfg["key_multiplier"])
        q = rope_apply(q, positions, inv_freq, rotary_dim, rnd)
        k = rope_apply(k, positions, inv_freq, rotary_dim, rnd)
        attn = causal_attention(q, k, v, hd ** -0.5, window, rnd).reshape(T, Hq * hd)
        attn = linear(attn, w[p + "self_attn.o_proj.weight"])
        ssm = mamba2_mixer(s_in, w, p + "mamba.", cfg, rnd, linear)
        (h,), residual = rms_norm_branches(
            attn, w[p + "pre_ff_layernorm.weight"], eps, residual, other=ssm,
            in_scales=(cfg["attention_out_multiplier"], cfg["ssm_out_multiplier"]), rnd=rnd)
        x = gated_mlp(h, w[p + "feed_forward.gate_proj.weight"], w[p + "feed_forward.up_proj.weight"],
                      w[p + "feed_forward.down_proj.weight"], cfg["mlp_multipliers"][0],
                      cfg["mlp_multipliers"][1], rnd, linear)
    (hN,), _ = rms_norm_branches(x, w["model.final_layernorm.weight"], eps, residual, rnd=rnd)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return rnd(linear(hN, head) * cfg["lm_head_multiplier"]).to(torch.float32 if compute != torch.float64 else compute)
