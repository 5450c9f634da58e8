"""Weight loading errors and the random-weights mode (CPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import save_file

from logssms_b200.config import make_model_config
from logssms_b200.models import build_model
from logssms_b200.weights import WeightError, check_and_place, checkpoint_files, read_checkpoint, write_random_model

from tiny import TINY_A, TINY_B, make_model_dir


def test_random_model_folder_is_complete_and_seeded(tmp_path):
    d1 = make_model_dir(tmp_path / "a", TINY_B, seed=3, dtype=torch.bfloat16)
    d2 = make_model_dir(tmp_path / "b", TINY_B, seed=3, dtype=torch.bfloat16)
    d3 = make_model_dir(tmp_path / "c", TINY_B, seed=4, dtype=torch.bfloat16)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    t1, t2, t3 = read_checkpoint(d1), read_checkpoint(d2), read_checkpoint(d3)
    assert t1.keys() == t2.keys() and all(torch.equal(t1[k], t2[k]) for k in t1)
    assert any(not torch.equal(t1[k], t3[k]) for k in t1)
    # names are the checkpoint's own (unmerged) names
    for name in ("model.embed_tokens.weight", "lm_head.weight", "model.final_layernorm.weight",
                 "model.layers.2.self_attn.q_proj.weight", "model.layers.0.mamba.in_proj.bias",
                 "model.layers.0.mamba.conv1d.weight", "model.layers.1.mamba.A_log",
                 "model.layers.1.mamba.norm.weight", "model.layers.0.mamba.out_proj.bias",
                 "model.layers.0.feed_forward.gate_proj.weight", "model.layers.0.pre_ff_layernorm.weight"):
        assert name in t1, name
    assert t1["model.layers.0.mamba.conv1d.weight"].shape == (272, 1, 3)
    assert t1["model.layers.0.mamba.A_log"].dtype == torch.float32          # stored in 32-bit
    assert t1["model.embed_tokens.weight"].dtype == torch.bfloat16
    a = t1["model.layers.0.mamba.A_log"]
    assert (a >= 0).all() and (a <= torch.log(torch.tensor(16.0))).all()
    dt = torch.nn.functional.softplus(t1["model.layers.0.mamba.dt_bias"].float())
    assert (dt > 9e-4).all() and (dt < 1.1e-1).all()
    tied = read_checkpoint(make_model_dir(tmp_path / "t", TINY_A))
    assert "lm_head.weight" not in tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_B)
    stored = read_checkpoint(d)
    del stored["model.layers.1.mamba.D"]
    del stored["model.layers.0.self_attn.k_proj.weight"]
    stored["model.layers.0.extra.weight"] = torch.zeros(2)
    stored["model.layers.2.mamba.conv1d.weight"] = torch.zeros(272, 1, 4)
    stored["model.final_layernorm.weight"] = torch.zeros(95)
    model = build_model(make_model_config(TINY_B))
    with pytest.raises(WeightError) as info:
        check_and_place(model, stored, torch.float32, "cpu", d)
    e = info.value
    assert e.missing == ["model.layers.0.self_attn.k_proj.weight", "model.layers.1.mamba.D"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.final_layernorm.weight", "model.layers.2.mamba.conv1d.weight"]
    msg = str(e)
    for part in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "stored (95,), model wants (96,)"):
        assert part in msg


def test_dtypes_are_kept(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_A, dtype=torch.bfloat16)
    stored = read_checkpoint(d)
    stored["model.layers.0.self_attn.o_proj.weight"] = stored["model.layers.0.self_attn.o_proj.weight"].float()
    model = build_model(make_model_config(TINY_A))
    placed = check_and_place(model, stored, torch.bfloat16, "cpu")
    assert placed["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert placed["model.layers.0.self_attn.o_proj.weight"].dtype == torch.float32     # stored in 32-bit: stays
    assert placed["model.layers.0.mamba.A_log"].dtype == torch.float32
    assert placed["model.layers.0.input_layernorm.weight"].dtype == torch.float32       # small vectors: widened, exact
    placed32 = check_and_place(model, stored, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in placed32.values())


def test_checkpoint_discovery_order(tmp_path):
    t = {"x": torch.zeros(1)}
    with pytest.raises(FileNotFoundError):
        checkpoint_files(str(tmp_path))
    save_file(t, str(tmp_path / "other.safetensors"))
    save_file(t, str(tmp_path / "consolidated.safetensors"))
    assert [os.path.basename(p) for p in checkpoint_files(str(tmp_path))] == ["other.safetensors"]
    save_file(t, str(tmp_path / "model-00002-of-00002.safetensors"))
    save_file(t, str(tmp_path / "model-00001-of-00002.safetensors"))
    assert [os.path.basename(p) for p in checkpoint_files(str(tmp_path))] == [
        "model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    save_file(t, str(tmp_path / "model.safetensors"))
    assert [os.path.basename(p) for p in checkpoint_files(str(tmp_path))] == ["model.safetensors"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"b": "model-00002-of-00002.safetensors", "a": "model-00001-of-00002.safetensors",
                        "c": "model-00002-of-00002.safetensors"}}))
    assert [os.path.basename(p) for p in checkpoint_files(str(tmp_path))] == [
        "model-00002-of-00002.safetensors", "model-00001-of-00002.safetensors"]


def test_sharded_checkpoint_reads_like_a_single_file(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_A)
    stored = read_checkpoint(d)
    names = sorted(stored)
    os.remove(os.path.join(d, "model.safetensors"))
    save_file({n: stored[n] for n in names[::2]}, os.path.join(d, "model-00001-of-00002.safetensors"))
    save_file({n: stored[n] for n in names[1::2]}, os.path.join(d, "model-00002-of-00002.safetensors"))
    again = read_checkpoint(d)
    assert again.keys() == stored.keys() and all(torch.equal(again[k], stored[k]) for k in stored)


def test_a_tied_checkpoint_may_store_the_output_head_if_it_equals_the_embedding(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_A, seed=4)               # TINY_A ties its embeddings
    model = build_model(make_model_config(TINY_A))
    stored = read_checkpoint(d)
    assert "lm_head.weight" not in stored
    same = {**stored, "lm_head.weight": stored["model.embed_tokens.weight"].clone()}
    placed = check_and_place(model, same, torch.float32, "cpu")
    assert "lm_head.weight" not in placed
    other = {**stored, "lm_head.weight": stored["model.embed_tokens.weight"] + 1.0}
    with pytest.raises(WeightError) as err:
        check_and_place(model, other, torch.float32, "cpu")
    assert err.value.unexpected == ["lm_head.weight"]
    # an untied model needs the tensor and never drops it
    untied = build_model(make_model_config(TINY_B))
    d2 = make_model_dir(tmp_path / "m2", TINY_B, seed=4)
    assert "lm_head.weight" in check_and_place(untied, read_checkpoint(d2), torch.float32, "cpu")
