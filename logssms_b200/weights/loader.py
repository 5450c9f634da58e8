"""Weights from safetensors, by tensor name.

File discovery follows the reference (python/logssms/models/weight.py:52-88,
safetensors branch): `model.safetensors.index.json` (its weight_map order), else
`model.safetensors`, else `model-*.safetensors`, else any `*.safetensors` except
`consolidated.safetensors`.  Checking is stricter than the reference's per-tensor
asserts (python/logssms/layers/base.py:44-59): every problem of a checkpoint —
missing tensors, unexpected tensors, wrong shapes — is gathered into ONE
`WeightError` that lists them all.

Dtypes: a tensor is held as it is stored (bfloat16 stays bfloat16; a tensor
stored in 32-bit stays 32-bit; integer tables become int32).  Small per-channel
vectors are widened to float32 for the kernels (exact).  With
`dtype=torch.float32` every floating tensor is widened to float32.
"""
from __future__ import annotations

import glob
import json
import os

import torch

from ..parts.base import MATRIX, TABLE, VECTOR, Part


class WeightError(RuntimeError):
    def __init__(self, missing, unexpected, wrong_shape, source=""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"checkpoint {source} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: stored {tuple(got)}, model wants {tuple(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def checkpoint_files(model_dir: str) -> list[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        files = list(dict.fromkeys(weight_map.values()))
        return [os.path.join(model_dir, f) for f in files]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    sharded = sorted(glob.glob(os.path.join(model_dir, "model-*.safetensors")))
    if sharded:
        return sharded
    others = sorted(p for p in glob.glob(os.path.join(model_dir, "*.safetensors"))
                    if os.path.basename(p) != "consolidated.safetensors")
    if others:
        return others
    raise FileNotFoundError(f"no safetensors checkpoint in {model_dir}")


def read_checkpoint(model_dir: str) -> dict[str, torch.Tensor]:
    """All tensors of a model folder on the host, as stored."""
    from safetensors import safe_open
    tensors: dict[str, torch.Tensor] = {}
    for path in checkpoint_files(model_dir):
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name)
    return tensors


def _held(tensor: torch.Tensor, role: str, engine_dtype: torch.dtype) -> torch.Tensor:
    if role == TABLE:
        return tensor.to(torch.int32)
    if role == VECTOR or engine_dtype == torch.float32:
        return tensor.to(torch.float32)
    return tensor   # MATRIX in a bfloat16 engine: as stored


def check_and_place(model: Part, stored: dict[str, torch.Tensor], dtype: torch.dtype,
                    device, source: str = "") -> dict[str, torch.Tensor]:
    expected = dict(model.named_param_specs())
    missing = [n for n in expected if n not in stored]
    # a tensor the model shares with another one (a tied output head) may be stored all the same: it is dropped
    # when it equals the tensor it is tied to (the reference drops it unseen, python/logssms/layers/embedding.py:60-76)
    # and stays an error when it differs, since the model could not honour it
    twins = getattr(model, "duplicate_names", dict)()
    unexpected = [n for n in stored if n not in expected
                  and not (n in twins and twins[n] in stored and stored[n].shape == stored[twins[n]].shape
                           and torch.equal(stored[n], stored[twins[n]]))]
    wrong = [(n, stored[n].shape, expected[n].shape) for n in expected
             if n in stored and tuple(stored[n].shape) != tuple(expected[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, source)
    return {n: _held(stored[n], spec.role, dtype).to(device).contiguous() for n, spec in expected.items()}


def load_weights(model: Part, model_dir: str, dtype: torch.dtype, device) -> None:
    """Read, check and bind the weights of `model` from `model_dir`."""
    stored = read_checkpoint(model_dir)
    model.bind_tree(check_and_place(model, stored, dtype, device, model_dir))
