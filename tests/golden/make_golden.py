#!/usr/bin/env python3
"""Run the parts of dakingffo/LogSSMs that can run on a CPU and store their outputs.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/LogSSMs

What runs here without a GPU (the reference's Triton kernels under the Triton interpreter, and its
pure-PyTorch code): `rms_norm_branches`, `grouped_rms_norm_gated`, `silu_and_mul`,
`scaled_silu_and_mul` (python/logssms/kernel/norm.py, fused.py), `packed_causal_conv1d`
(python/logssms/kernel/linear_attention/packed_conv.py), the cos/sin table of `RotaryEmbedding` and
the llama3 / yarn frequency post-processing (python/logssms/layers/rotary.py), and the recurrence
oracle of its own kernel tests (tests/kernel/test_mamba2.py:22-38).  What does NOT run on a CPU:
the whole model's forward pass (attention, embedding and the fused rope/store kernels assert CUDA),
the chunked Mamba2 prefill (its autotuner needs a driver) and `prepare_mamba2` (libdevice.log1p).
Those parts of tests/plain rest on the reference's formulas alone.

Note on the bfloat16 outputs: the interpreter converts float32 to bfloat16 by truncation, a GPU rounds
to nearest even, so they are good to a few units in the last place only; the float32 outputs are exact.

Inputs are drawn from seeded generators (`inputs()` below; tests/test_plain.py imports this file and
draws the same), outputs go to `reference_blocks.safetensors` next to this script.  The file that
is committed was made by this script from the reference checkout mounted at build time.
"""
from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "reference_blocks.safetensors")


def inputs() -> dict[str, torch.Tensor]:
    """Every input of every block, by name.  Deterministic."""
    g = torch.Generator().manual_seed(20261125)
    r = lambda *s, scale=1.0: torch.randn(*s, generator=g) * scale
    t: dict[str, torch.Tensor] = {}
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        t[f"norm.x.{tag}"] = r(5, 40).to(dt)
        t[f"norm.other.{tag}"] = r(5, 40).to(dt)
        t[f"norm.residual.{tag}"] = r(5, 40).to(dt)
        t[f"norm.weight.{tag}"] = (1 + r(40, scale=0.1)).to(dt)
        t[f"gated.y.{tag}"] = r(4, 48).to(dt)
        t[f"gated.gate.{tag}"] = r(4, 48).to(dt)
        t[f"gated.weight.{tag}"] = (1 + r(48, scale=0.1)).to(dt)
        t[f"mlp.gate_up.{tag}"] = r(3, 2 * 50).to(dt)
        t[f"conv.x.{tag}"] = r(75 + 9, 20).to(dt)                  # two requests: 75 and 9 tokens
        t[f"conv.weight.{tag}"] = r(20, 1, 4, scale=0.3).to(dt)
        t[f"conv.bias.{tag}"] = r(20, scale=0.1).to(dt)
    t["ssm.xbc"] = r(11, 2 * 8 + 2 * 1 * 16, scale=0.5).to(torch.bfloat16)        # 2 heads x 8, 1 group, state 16
    t["ssm.dt"] = (r(11, 2) - 2).to(torch.bfloat16)
    t["ssm.A_log"] = r(2, scale=0.1)
    t["ssm.dt_bias"] = r(2, scale=0.1)
    t["ssm.D"] = r(2, scale=0.1)
    return t


ROPE_CASES = {
    "default": (32, 32, 1e4, None),
    "partial": (48, 24, 1e11, None),
    "llama3": (32, 32, 1e5, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 64}),
    "yarn": (32, 32, 1e4, {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64}),
}
ROPE_POSITIONS = 200


def main(reference_root: str) -> None:
    os.environ.setdefault("TRITON_INTERPRET", "1")
    sys.path.insert(0, os.path.join(reference_root, "python"))
    sys.path.insert(0, reference_root)
    from types import SimpleNamespace

    from safetensors.torch import save_file

    from logssms.kernel.fused import scaled_silu_and_mul, silu_and_mul
    from logssms.kernel.linear_attention.packed_conv import packed_causal_conv1d
    from logssms.kernel.norm import grouped_rms_norm_gated, rms_norm_branches
    from logssms.layers import rotary
    from tests.kernel.test_mamba2 import reference as recurrence_oracle

    t = inputs()
    out: dict[str, torch.Tensor] = {}
    for tag in ("f32", "bf16"):
        x, other, res, w = (t[f"norm.{n}.{tag}"] for n in ("x", "other", "residual", "weight"))
        (o0, o1), r = rms_norm_branches(x, w, 1e-5, res.clone(), other=other, input_scales=(0.8, 0.7), output_scales=(1.5, 1.2))
        out[f"norm.two.out0.{tag}"], out[f"norm.two.out1.{tag}"], out[f"norm.two.residual.{tag}"] = o0, o1, r
        (o0,), r = rms_norm_branches(x, w, 1e-6, None, output_scales=(1.0,))
        out[f"norm.one.out0.{tag}"], out[f"norm.one.residual.{tag}"] = o0, r
        y, gate, gw = (t[f"gated.{n}.{tag}"] for n in ("y", "gate", "weight"))
        out[f"gated.before.{tag}"] = grouped_rms_norm_gated(y, gate, gw, 1e-5, 2, True, gate_scale=0.6)
        out[f"gated.after.{tag}"] = grouped_rms_norm_gated(y, gate, gw, 1e-5, 3, False, gate_scale=0.6)
        out[f"gated.none.{tag}"] = silu_and_mul(y, gate, 0.6)
        out[f"mlp.swiglu.{tag}"] = scaled_silu_and_mul(t[f"mlp.gate_up.{tag}"], 0.9)
        cx, cw, cb = (t[f"conv.{n}.{tag}"] for n in ("x", "weight", "bias"))
        history = torch.zeros(2, 20, 3, dtype=cx.dtype)
        cu = torch.tensor([0, 75, 84], dtype=torch.int32)
        chunks = torch.tensor([[0, 0], [0, 1], [1, 0]], dtype=torch.int32)         # (request, run of 64 tokens)
        out[f"conv.out.{tag}"] = packed_causal_conv1d(cx, cw, history, cu, chunks, cb, input_boundaries=(8, 14),
                                                      input_scales=(1.1, 0.9, 1.3))
    cfg = SimpleNamespace(value_dim=16, num_groups=1, state_dim=16, num_heads=2, head_dim=8)
    initial = torch.zeros(2, 16, 8)
    y, states = recurrence_oracle(t["ssm.xbc"], t["ssm.dt"], t["ssm.A_log"], t["ssm.dt_bias"], t["ssm.D"], cfg, initial)
    out["ssm.y"], out["ssm.final_state"] = y.contiguous(), states[-1].contiguous()
    for name, (hd, rd, theta, scaling) in ROPE_CASES.items():
        out[f"rope.{name}"] = rotary._get_rope(hd, rd, ROPE_POSITIONS, theta, scaling)._cos_sin_cache.contiguous()
    save_file({k: v.contiguous() for k, v in out.items()}, OUT)
    print(f"wrote {len(out)} tensors to {OUT} ({os.path.getsize(OUT)} bytes)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
