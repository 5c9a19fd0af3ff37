"""Weights: the safetensors container, loading by name, one error for everything that is
wrong with a folder, the storage policy, and the random-weights mode."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import kvcache_b200  # noqa: F401
from kvcache_b200.config import config_from_dict
from kvcache_b200.engine.loading import load_model
from kvcache_b200.models.qwen2 import build_qwen2
from kvcache_b200.weights import (SafetensorsError, SafetensorsFile, TensorSpec, WeightError, load_tensors,
                                  write_random_model, write_safetensors)
from tiny_configs import TINY_A, TINY_B, make_model_folder


def test_container_round_trip_both_ways(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
               "d": torch.randn(2, 2).to(torch.float16), "e": torch.tensor(3.5)}
    mine = os.path.join(tmp_path, "mine.safetensors")
    write_safetensors(mine, tensors, {"note": "x"})
    theirs = load_file(mine)                       # the safetensors package reads what we wrote
    for k, v in tensors.items():
        assert torch.equal(theirs[k], v)
    other = os.path.join(tmp_path, "theirs.safetensors")
    save_file(tensors, other)
    f = SafetensorsFile(other)                     # and we read what it wrote
    assert set(f.names()) == set(tensors)
    for k, v in tensors.items():
        assert torch.equal(f.tensor(k), v) and f.dtype(k) == v.dtype and f.shape(k) == tuple(v.shape)


def test_truncated_or_corrupt_file(tmp_path):
    path = os.path.join(tmp_path, "model.safetensors")
    write_safetensors(path, {"a": torch.randn(64, 64)})
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:len(blob) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    open(path, "wb").write(b"\x05\x00\x00")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(65)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(128, 64)     # transposed
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    save_file(tensors, path)
    with pytest.raises(WeightError) as err:
        load_model(folder, "float32", "cpu")
    e = err.value
    assert set(e.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["model.layers.7.extra.weight"]
    assert {n for n, _, _ in e.wrong_shape} == {"model.layers.0.self_attn.q_proj.bias", "model.layers.0.mlp.down_proj.weight"}
    assert [n for n, _, _ in e.wrong_kind] == ["model.embed_tokens.weight"]
    text = str(e)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "expected [64, 128] found [128, 64]"):
        assert word in text, text


def test_untied_model_needs_lm_head_and_tied_model_refuses_it(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    head = tensors.pop("lm_head.weight")
    save_file(tensors, path)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_model(folder, "float32", "cpu")
    folder = make_model_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(64)      # a tensor this architecture has no place for
    save_file(tensors, path)
    with pytest.raises(WeightError, match="unexpected"):
        load_model(folder, "float32", "cpu")
    model = load_model(folder, "float32", "cpu", strict=False)                # on request: a warning, not an error
    assert model.head is model.embed


def test_tensors_a_checkpoint_may_carry_unused(tmp_path, capsys):
    """The reference's exporter stores the embedding a second time as lm_head.weight when the head is tied
    (tools/dump_weights.py:24-26), and checkpoints carry the rotation's frequencies as a buffer: both are left
    alone, named in a warning, and the tied head stays the embedding's own buffer."""
    folder = make_model_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(tensors, path)
    model = load_model(folder, "float32", "cpu")
    assert model.head is model.embed
    warning = capsys.readouterr().err
    assert "lm_head.weight" in warning and "inv_freq" in warning and "2 tensors" in warning
    ignored = []
    load_tensors(folder, model.tensor_specs(), ignorable=model.ignorable_tensors, ignored=ignored)
    assert sorted(ignored) == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    # An untied model does use lm_head.weight; for it the name is not ignorable.
    assert "lm_head.weight" not in build_qwen2(config_from_dict(TINY_B), dtype="float32").ignorable_tensors


def test_sharded_checkpoint_through_its_index(tmp_path):
    """A checkpoint in several files: model.safetensors.index.json maps every tensor to its file."""
    folder = make_model_folder(tmp_path, "B")
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    whole = load_model(folder, "float32", "cpu")
    os.remove(path)
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[:len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for file, members in shards.items():
        save_file({n: tensors[n] for n in members}, os.path.join(folder, file))
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        json.dump({"metadata": {}, "weight_map": {n: file for file, members in shards.items() for n in members}}, fh)
    sharded = load_model(folder, "float32", "cpu")
    assert torch.equal(sharded.embed, whole.embed) and torch.equal(sharded.head, whole.head)
    assert torch.equal(sharded.blocks[2].mixer.w_qkv, whole.blocks[2].mixer.w_qkv)
    assert torch.equal(sharded.blocks[0].ffn.w_down, whole.blocks[0].ffn.w_down)
    # A tensor missing from every shard is reported like any missing tensor; a shard the index names but the folder
    # lacks is an error of its own.
    os.remove(os.path.join(folder, "model-00002-of-00002.safetensors"))
    with pytest.raises(WeightError, match="model-00002-of-00002.safetensors"):
        load_model(folder, "float32", "cpu")


def test_missing_file(tmp_path):
    with open(os.path.join(tmp_path, "config.json"), "w") as fh:
        json.dump(TINY_A, fh)
    with pytest.raises(WeightError, match="model.safetensors"):
        load_model(str(tmp_path), "float32", "cpu")


def test_storage_policy(tmp_path):
    path = os.path.join(tmp_path, "model.safetensors")
    write_safetensors(path, {"h": torch.randn(4).to(torch.float16), "b": torch.randn(4).to(torch.bfloat16),
                             "f": torch.randn(4), "d": torch.randn(4, dtype=torch.float64),
                             "i": torch.arange(4, dtype=torch.int64)})
    specs = {k: TensorSpec((4,)) for k in "hbfd"}
    specs["i"] = TensorSpec((4,), kind="int")
    got = load_tensors(str(tmp_path), specs)
    assert got["h"].dtype == torch.bfloat16 and got["b"].dtype == torch.bfloat16    # 16-bit -> bfloat16
    assert got["f"].dtype == torch.float32 and got["d"].dtype == torch.float32      # 32-bit stays 32-bit
    assert got["i"].dtype == torch.int32                                            # integer tables -> int32


def test_bound_dtypes(tmp_path):
    folder = make_model_folder(tmp_path, "A", dtype=torch.bfloat16)
    for dtype, want in (("bfloat16", torch.bfloat16), ("float32", torch.float32)):
        model = load_model(folder, dtype, "cpu")
        mixer = model.blocks[0].mixer
        assert model.embed.dtype == want and mixer.w_qkv.dtype == want and model.blocks[0].ffn.w_down.dtype == want
        assert mixer.b_qkv.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32
        assert model.head is model.embed          # tied: one buffer
        assert mixer.w_qkv.shape == (4 * 16 + 2 * 2 * 16, 64)


def test_random_mode_is_seeded_and_shaped(tmp_path):
    a1 = load_file(os.path.join(make_model_folder(tmp_path / "x", "B", seed=3), "model.safetensors"))
    a2 = load_file(os.path.join(make_model_folder(tmp_path / "y", "B", seed=3), "model.safetensors"))
    b = load_file(os.path.join(make_model_folder(tmp_path / "z", "B", seed=4), "model.safetensors"))
    assert all(torch.equal(a1[k], a2[k]) for k in a1)
    assert not torch.equal(a1["lm_head.weight"], b["lm_head.weight"])
    model = build_qwen2(config_from_dict(TINY_B), dtype="float32")
    assert {k: tuple(v.shape) for k, v in a1.items()} == {k: s.shape for k, s in model.tensor_specs().items()}
    w = a1["model.layers.0.mlp.gate_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = a1["model.layers.2.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.02
    with open(os.path.join(tmp_path / "x", "tiny_B_3", "config.json")) as fh:
        assert config_from_dict(json.load(fh)) == config_from_dict(TINY_B)
