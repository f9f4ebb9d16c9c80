"""Typed configuration of the dense grouped-query Qwen2 decoder (`Qwen2ForCausalLM`).

Keys and defaults follow the reference's reads (student_engine.py:327-349):
`hidden_size`, `intermediate_size`, `num_hidden_layers`, `num_attention_heads`
(required), `num_key_value_heads` (default: the head count), `rms_norm_eps` (1e-6),
`rope_theta` (10000.0), `max_position_embeddings` (32768), `torch_dtype`; the three
checks there (width divisible by heads, heads by kv heads, even head size) are kept.

The reference never reads `vocab_size`, `tie_word_embeddings`, `head_dim`,
`hidden_act`, `rope_scaling` or the sliding-window keys. They are read here so that no
size stands in code and so that a file that asks for something this library does not
compute is refused instead of silently computed differently:
  vocab_size            required (sizes the tables of random weights and is checked
                        against the file's tensors)
  tie_word_embeddings   default false: true means the head is the embedding table
  head_dim              default hidden_size // num_attention_heads
  hidden_act            must be "silu" (the reference's fixed activation, :663-666)
  rope_scaling          must be null
  use_sliding_window, sliding_window, max_window_layers
                        layers with index >= max_window_layers attend to the last
                        `sliding_window` positions only, when use_sliding_window is
                        true (every published Qwen2.5 file has it false, which is
                        what the reference computes)
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Mapping, Optional

from .registry import ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _need(data: Mapping[str, Any], key: str):
    if key not in data or data[key] is None:
        raise ValueError(f"config.json: required key {key!r} is missing")
    return data[key]


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: Optional[bool] = False   # None: the key is absent; the files decide (student_engine.py:359)
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen2Config":
        model_type = data.get("model_type", cls.model_type)
        if str(model_type) != cls.model_type:
            raise ValueError(f"config.json: model_type is {model_type!r}, expected {cls.model_type!r}")
        hidden = int(_need(data, "hidden_size"))
        heads = int(_need(data, "num_attention_heads"))
        if heads <= 0 or hidden <= 0:
            raise ValueError("config.json: hidden_size and num_attention_heads must be positive")
        kv_heads = int(data.get("num_key_value_heads") or heads)
        if hidden % heads != 0 and data.get("head_dim") is None:
            raise ValueError(f"config.json: hidden_size {hidden} is not divisible by "
                             f"num_attention_heads {heads} and no head_dim is given")
        head_dim = int(data.get("head_dim") or hidden // heads)
        eos = data.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        config = cls(
            vocab_size=int(_need(data, "vocab_size")),
            hidden_size=hidden,
            intermediate_size=int(_need(data, "intermediate_size")),
            num_hidden_layers=int(_need(data, "num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(data.get("rms_norm_eps", 1e-6)),
            rope_theta=float(data.get("rope_theta", 10000.0)),
            max_position_embeddings=int(data.get("max_position_embeddings", 32768)),
            tie_word_embeddings=None if data.get("tie_word_embeddings") is None else bool(data["tie_word_embeddings"]),
            hidden_act=str(data.get("hidden_act", "silu")),
            use_sliding_window=bool(data.get("use_sliding_window", False)),
            sliding_window=None if data.get("sliding_window") is None else int(data["sliding_window"]),
            max_window_layers=None if data.get("max_window_layers") is None else int(data["max_window_layers"]),
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
            bos_token_id=None if data.get("bos_token_id") is None else int(data["bos_token_id"]),
            eos_token_id=None if eos is None else int(eos),
        )
        config.validate(rope_scaling=data.get("rope_scaling"))
        return config

    def validate(self, rope_scaling=None) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError(f"config.json: num_attention_heads {self.num_attention_heads} is not divisible "
                             f"by num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ValueError(f"config.json: head_dim {self.head_dim} is odd; rotary embedding needs an even head size")
        if self.hidden_act != "silu":
            raise ValueError(f"config.json: hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if rope_scaling not in (None, {}):
            raise ValueError(f"config.json: rope_scaling {rope_scaling!r} is not supported (must be null)")
        for key in ("vocab_size", "intermediate_size", "num_hidden_layers", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ValueError(f"config.json: {key} must be positive, got {getattr(self, key)}")
        if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
            raise ValueError("config.json: rms_norm_eps and rope_theta must be positive")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ValueError("config.json: use_sliding_window is true but sliding_window is not a positive integer")

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture], "model_type": self.model_type}
        for f in fields(self):
            out[f.name] = getattr(self, f.name)
        return out

    # ------------------------------------------------------------------ derived
    def layer_window(self, index: int) -> int:
        """Attention window of layer `index`; 0 means all earlier keys."""
        if not self.use_sliding_window or self.sliding_window is None:
            return 0
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return int(self.sliding_window) if index >= first else 0

    def model_spec(self) -> ModelSpec:
        """Tensor names are the files' own (student_engine.py:357-359, :498-528)."""
        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": self.hidden_size, "eps": self.rms_norm_eps}, {"weight": name})

        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            mixer = PartSpec(
                "gqa_attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "qkv_bias": True,
                    "out_bias": False,
                    "scale": float(self.head_dim) ** -0.5,
                    "window": self.layer_window(i),
                    "position": PartSpec("rotary_half", {"head_dim": self.head_dim, "theta": self.rope_theta}),
                },
                {
                    "q_weight": p + "self_attn.q_proj.weight", "q_bias": p + "self_attn.q_proj.bias",
                    "k_weight": p + "self_attn.k_proj.weight", "k_bias": p + "self_attn.k_proj.bias",
                    "v_weight": p + "self_attn.v_proj.weight", "v_bias": p + "self_attn.v_proj.bias",
                    "o_weight": p + "self_attn.o_proj.weight",
                },
            )
            ffn = PartSpec(
                "swiglu",
                {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size},
                {"gate_weight": p + "mlp.gate_proj.weight", "up_weight": p + "mlp.up_proj.weight",
                 "down_weight": p + "mlp.down_proj.weight"},
            )
            layers.append(LayerSpec("pre_norm", {
                "mixer_norm": norm(p + "input_layernorm.weight"), "mixer": mixer,
                "feed_forward_norm": norm(p + "post_attention_layernorm.weight"), "feed_forward": ffn}))
        if self.tie_word_embeddings:
            head_tensors = {"weight": "model.embed_tokens.weight"}
        elif self.tie_word_embeddings is None:   # config.json does not say: lm_head.weight if the files hold it
            head_tensors = {"weight": "lm_head.weight", "weight_fallback": "model.embed_tokens.weight"}
        else:
            head_tensors = {"weight": "lm_head.weight"}
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "width": self.hidden_size},
                               {"weight": "model.embed_tokens.weight"}),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=norm("model.norm.weight"),
            head=PartSpec("linear_head",
                          {"vocab_size": self.vocab_size, "width": self.hidden_size,
                           "tied": bool(self.tie_word_embeddings)},
                          head_tensors),
            stop_token_ids=() if self.eos_token_id is None else (self.eos_token_id,),
            # a tied model whose files also store the head: taken if it is the embedding table, as the reference
            # takes it (student_engine.py:359)
            redundant_tensors={"lm_head.weight": "model.embed_tokens.weight"} if self.tie_word_embeddings else {},
        )
        spec.validate()
        return spec


register_architecture(Qwen2Config.architecture, Qwen2Config, Qwen2Config.model_type)
