"""Configuration: typed reads, defaults, errors that name the key, the registry, the presets."""
import json

import pytest
import torch

from qwenforge_b200.config import (ModelConfig, Qwen2Config, config_from_dict, load_config, preset_config, preset_names,
                                   register_architecture, registered_architectures, resolve_dtype)
from tests.helpers import TINY_A, TINY_B, TINY_W


def test_reads_and_defaults():
    c = config_from_dict(TINY_B)
    assert isinstance(c, Qwen2Config)
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (120, 5, 1, 24)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    minimal = dict(model_type="qwen2", vocab_size=10, hidden_size=8, intermediate_size=16, num_hidden_layers=1,
                   num_attention_heads=2)
    d = config_from_dict(minimal)
    # the reference's defaults (student_engine.py:336-342)
    assert d.num_key_value_heads == 2 and d.head_dim == 4 and d.rms_norm_eps == 1e-6 and d.rope_theta == 10000.0
    assert d.max_position_embeddings == 32768 and d.layer_window(0) == 0


def test_round_trip_through_dict():
    c = config_from_dict(TINY_W)
    assert config_from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change,word", [
    (dict(num_attention_heads=None), "num_attention_heads"),
    (dict(vocab_size=None), "vocab_size"),
    (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(head_dim=15), "head_dim"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
    (dict(model_type="llama", architectures=["Qwen2ForCausalLM"]), "model_type"),
    (dict(hidden_size=65, head_dim=None), "hidden_size"),
])
def test_errors_name_the_key(change, word):
    data = dict(TINY_A)
    data.update(change)
    data = {k: v for k, v in data.items() if not (v is None and k in ("num_attention_heads", "vocab_size", "head_dim"))}
    with pytest.raises(ValueError, match=word):
        config_from_dict(data)


def test_registry():
    assert "Qwen2ForCausalLM" in registered_architectures()
    with pytest.raises(ValueError, match="registered: .*Qwen2ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["NoSuchModel"]))
    # without an `architectures` key the model_type decides
    data = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert isinstance(config_from_dict(data), Qwen2Config)

    class Other(ModelConfig):
        @classmethod
        def from_dict(cls, data):
            return cls()

    register_architecture("OtherForTest", Other)
    assert isinstance(config_from_dict({"architectures": ["OtherForTest"]}), Other)
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen2ForCausalLM", Other)


def test_load_config_from_folder(tmp_path):
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert load_config(tmp_path).hidden_size == 64


def test_spec_is_data():
    spec = config_from_dict(TINY_W).model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert [layer.part("mixer").params["window"] for layer in spec.layers] == [0, 37, 37]
    assert spec.layers[0].part("mixer").params["position"].params["theta"] == 50000.0
    assert spec.head.tensors["weight"] == "lm_head.weight"
    tied = config_from_dict(TINY_A).model_spec()
    assert tied.head.tensors["weight"] == tied.embedding.tensors["weight"]


def test_presets_cover_the_measured_sizes():
    assert {"tiny-a", "tiny-b", "qwen2.5-0.5b", "qwen2.5-3b", "qwen2.5-7b"} <= set(preset_names())
    c = preset_config("qwen2.5-0.5b")
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size, c.tie_word_embeddings) == (896, 24, 14, 2, 64, 4864, 151936, True)
    with pytest.raises(ValueError, match="unknown preset"):
        preset_config("nope")


def test_dtype_names():
    assert resolve_dtype("bf16") == torch.bfloat16 and resolve_dtype("float32") == torch.float32
    assert resolve_dtype("auto", "float32") == torch.float32 and resolve_dtype("auto", "float16") == torch.bfloat16
    with pytest.warns(UserWarning, match="bfloat16"):   # the reference's default name is served by the 16-bit path there is
        assert resolve_dtype("float16") == torch.bfloat16
    assert resolve_dtype("auto", "float16") == torch.bfloat16
    with pytest.raises(ValueError, match="Unsupported dtype"):
        resolve_dtype("int8")
