"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds config.json and model.safetensors and is read back through the
ordinary loader, so a random model takes the same path as a real one.  Every part
declares how each of its tensors is drawn (`ParamSpec.init`); the generator lives
on the CPU so that any reader — the engine on the GPU or a plain implementation
on the CPU — sees the same bits.

The reference's `--dummy-weight` (python/logssms/engine/engine.py:235-239) fills
every tensor with N(0,1); here the draw is structured so that the recurrence is
well-behaved: matrices N(0, 0.02), A_log = log U[1, 16], dt_bias = softplus^-1 of
a log-uniform step in [1e-3, 1e-1], D = 1, norm weights = 1 (`perturb` draws the
last two and all biases around these values so that tests see them act).
"""
from __future__ import annotations

import json
import os

import torch

from ..parts.base import TABLE, VECTOR


def random_tensors(model, seed: int, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    out = {}
    for name, spec in model.named_param_specs():
        t = spec.init(gen, tuple(spec.shape))
        if spec.role == TABLE:
            out[name] = t.to(torch.int32)
        else:
            out[name] = t.to(spec.store_dtype or dtype).contiguous()
    return out


def write_random_model(config, out_dir: str, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                       perturb: bool = False) -> str:
    """Create `out_dir` with config.json and model.safetensors for `config`
    (a typed architecture config).  Returns `out_dir`."""
    from safetensors.torch import save_file
    from ..models import build_model
    os.makedirs(out_dir, exist_ok=True)
    model = build_model(config, perturb_init=perturb)
    tensors = random_tensors(model, seed, dtype)
    raw = config.to_dict()
    raw["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir
