"""Weights: reading by name, kept dtypes, one error for everything that does not line up, the random mode."""
import json

import pytest
import torch

from qwenforge_b200.config import config_from_dict
from qwenforge_b200.engine import Model
from qwenforge_b200.parts import TensorSpec
from qwenforge_b200.weights import (SafetensorsFile, WeightsError, load_weights, resolve_model_dir, save_safetensors,
                                    write_random_model)
from tests import plain_qwen2 as plain
from tests.helpers import TINY_A, TINY_B, make_model_dir


def specs_of(config):
    return Model.tensor_specs_of(config_from_dict(config).model_spec())


def test_names_are_the_files_own():
    for config in (TINY_A, TINY_B):
        ours = {(s.name, tuple(s.shape)) for s in specs_of(config)}
        theirs = {(n, tuple(s)) for n, s, _ in plain.tensor_names_and_shapes(config)}
        assert ours == theirs


def test_round_trip_and_kept_dtypes(tmp_path):
    folder, weights = make_model_dir(TINY_B, 1, tmp_path, store_dtype=torch.float32)
    as_bf16 = load_weights(folder, specs_of(TINY_B), torch.bfloat16, "cpu")
    as_f32 = load_weights(folder, specs_of(TINY_B), torch.float32, "cpu")
    for name, t in weights.items():
        assert as_f32[name].dtype == torch.float32 and torch.equal(as_f32[name], t)
        assert as_bf16[name].dtype == torch.bfloat16 and torch.equal(as_bf16[name], t.to(torch.bfloat16))
    # a bfloat16 file widens exactly on the 32-bit path
    folder2, _ = make_model_dir(TINY_B, 1, tmp_path / "b", store_dtype=torch.bfloat16)
    widened = load_weights(folder2, specs_of(TINY_B), torch.float32, "cpu")
    assert torch.equal(widened["model.norm.weight"], weights["model.norm.weight"].to(torch.bfloat16).float())


def test_stored_and_integer_tensors_keep_their_type(tmp_path):
    save_safetensors(tmp_path / "model.safetensors", {
        "a": torch.randn(3, 4), "b": torch.randn(5).to(torch.bfloat16), "t": torch.arange(6, dtype=torch.int64)})
    specs = [TensorSpec("a", (3, 4), keep="stored"), TensorSpec("b", (5,), keep="stored"), TensorSpec("t", (6,), keep="int32")]
    got = load_weights(tmp_path, specs, torch.bfloat16, "cpu")
    assert got["a"].dtype == torch.float32      # stored in 32-bit: stays so
    assert got["b"].dtype == torch.bfloat16
    assert got["t"].dtype == torch.int32 and got["t"].tolist() == list(range(6))
    with pytest.raises(WeightsError, match="wrong dtype"):
        load_weights(tmp_path, [TensorSpec("a", (3, 4), keep="int32"), specs[1], specs[2]], torch.bfloat16, "cpu")


def test_one_error_lists_everything(tmp_path):
    folder, weights = make_model_dir(TINY_A, 0, tmp_path)
    broken = dict(weights)
    del broken["model.layers.1.mlp.up_proj.weight"]
    del broken["model.norm.weight"]
    broken["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    broken["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    save_safetensors(folder / "model.safetensors", broken)
    with pytest.raises(WeightsError) as info:
        load_weights(folder, specs_of(TINY_A), torch.float32, "cpu")
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(e.wrong_shape) == 1 and "k_proj.weight" in e.wrong_shape[0] and "[32, 64]" in e.wrong_shape[0]
    text = str(e)
    assert "missing (2)" in text and "unexpected (1)" in text and "wrong shape (1)" in text


def test_tied_and_untied_heads(tmp_path):
    folder, weights = make_model_dir(TINY_A, 0, tmp_path)          # tied: no lm_head tensor wanted
    extra = dict(weights, **{"lm_head.weight": torch.zeros(256, 64)})
    save_safetensors(folder / "model.safetensors", extra)
    with pytest.raises(WeightsError, match="unexpected.*lm_head.weight"):
        load_weights(folder, specs_of(TINY_A), torch.float32, "cpu")
    folder_b, weights_b = make_model_dir(TINY_B, 0, tmp_path / "b")  # untied: lm_head tensor required
    del weights_b["lm_head.weight"]
    save_safetensors(folder_b / "model.safetensors", weights_b)
    with pytest.raises(WeightsError, match="missing.*lm_head.weight"):
        load_weights(folder_b, specs_of(TINY_B), torch.float32, "cpu")


def test_a_stored_copy_of_a_tied_head_and_files_that_do_not_say(tmp_path):
    """The reference takes lm_head.weight if the files hold it and the embedding table otherwise, whatever config.json
    says (student_engine.py:359). Here a tied model accepts a stored head that IS the embedding table and refuses
    one that differs; and a config.json without `tie_word_embeddings` lets the files decide."""
    spec = config_from_dict(TINY_A).model_spec()
    folder, weights = make_model_dir(TINY_A, 0, tmp_path)
    save_safetensors(folder / "model.safetensors", dict(weights, **{"lm_head.weight": weights["model.embed_tokens.weight"].clone()}))
    got = load_weights(folder, specs_of(TINY_A), torch.float32, "cpu", spec.redundant_tensors)
    assert "lm_head.weight" not in got and torch.equal(got["model.embed_tokens.weight"], weights["model.embed_tokens.weight"])
    save_safetensors(folder / "model.safetensors", dict(weights, **{"lm_head.weight": torch.zeros(256, 64)}))
    with pytest.raises(WeightsError, match="lm_head.weight.*differs"):
        load_weights(folder, specs_of(TINY_A), torch.float32, "cpu", spec.redundant_tensors)
    # no tie_word_embeddings key at all
    silent = {k: v for k, v in TINY_B.items() if k != "tie_word_embeddings"}
    assert config_from_dict(silent).tie_word_embeddings is None
    folder_b, weights_b = make_model_dir(silent, 1, tmp_path / "b")
    with_head = load_weights(folder_b, specs_of(silent), torch.float32, "cpu")
    assert torch.equal(with_head["lm_head.weight"], weights_b["lm_head.weight"])
    del weights_b["lm_head.weight"]
    save_safetensors(folder_b / "model.safetensors", weights_b)
    without = load_weights(folder_b, specs_of(silent), torch.float32, "cpu")
    assert torch.equal(without["lm_head.weight"], weights_b["model.embed_tokens.weight"])
    assert without["lm_head.weight"] is without["model.embed_tokens.weight"]     # one tensor, not a second copy


def test_shards_index_and_duplicates(tmp_path):
    _, weights = make_model_dir(TINY_A, 0, tmp_path / "whole")
    names = sorted(weights)
    half = len(names) // 2
    folder = tmp_path / "sharded"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    save_safetensors(folder / "model-00001-of-00002.safetensors", {n: weights[n] for n in names[:half]})
    save_safetensors(folder / "model-00002-of-00002.safetensors", {n: weights[n] for n in names[half:]})
    got = load_weights(folder, specs_of(TINY_A), torch.float32, "cpu")
    assert all(torch.equal(got[n], weights[n]) for n in names)
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
        for i, n in enumerate(names)}}))
    assert set(load_weights(folder, specs_of(TINY_A), torch.float32, "cpu")) == set(names)
    save_safetensors(folder / "model-00002-of-00002.safetensors", {n: weights[n] for n in names[half - 1:]})
    with pytest.raises(WeightsError, match="more than one file"):
        load_weights(folder, specs_of(TINY_A), torch.float32, "cpu")
    with pytest.raises(FileNotFoundError):
        load_weights(tmp_path / "nowhere", specs_of(TINY_A), torch.float32, "cpu")
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="No safetensors"):
        load_weights(empty, specs_of(TINY_A), torch.float32, "cpu")


def test_random_mode_writes_a_loadable_folder(tmp_path):
    config = config_from_dict(TINY_B)
    a = write_random_model(config, 7, tmp_path / "a", torch.float32)
    b = write_random_model(config, 7, tmp_path / "b", torch.float32)
    c = write_random_model(config, 8, tmp_path / "c", torch.bfloat16)
    wa = load_weights(a, specs_of(TINY_B), torch.float32, "cpu")
    wb = load_weights(b, specs_of(TINY_B), torch.float32, "cpu")
    wc = load_weights(c, specs_of(TINY_B), torch.float32, "cpu")
    assert all(torch.equal(wa[n], wb[n]) for n in wa)                 # same seed, same weights
    assert not torch.equal(wa["lm_head.weight"], wc["lm_head.weight"])  # other seed
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    w = wa["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(wa["model.norm.weight"].mean()) - 1.0) < 0.05
    with SafetensorsFile(c / "model.safetensors") as f:
        assert f.info("lm_head.weight")[0] == torch.bfloat16


def test_resolve_model_dir(tmp_path, monkeypatch):
    assert resolve_model_dir(tmp_path) == tmp_path
    with pytest.raises(FileNotFoundError, match="Model path not found"):
        resolve_model_dir("no_such_local_name")
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path))
    with pytest.raises(FileNotFoundError, match="Model cache not found"):
        resolve_model_dir("org/name")
    snap = tmp_path / "models--org--name" / "snapshots"
    (snap / "aaa").mkdir(parents=True)
    (snap / "bbb").mkdir()
    assert resolve_model_dir("org/name") == snap / "bbb"
