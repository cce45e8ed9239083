"""LlamaConfig: the typed configuration of the Llama / DeepSeek-LLM dense decoder.

Keys, aliases and defaults are those fastllm-py reads for this architecture
(fastllm_py/config.py:87-104 and :121): hidden_size|n_embd,
num_attention_heads|n_head, head_dim (default hidden // heads),
num_hidden_layers|n_layer, num_key_value_heads (default heads),
intermediate_size (default 4 * hidden), vocab_size, rope_theta (10000.0),
rms_norm_eps|layer_norm_epsilon (1e-6), max_position_embeddings (32768),
tie_word_embeddings (false), rope_scaling {type|rope_type, factor}.

Where the reference silently accepts what it cannot compute (an activation
other than silu is parsed but ignored, config.py:122 and ops.py:157; an unknown
rope_scaling type falls through to unscaled rope, model.py:331-339), this
configuration refuses with an error that names the key.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class LinearRopeScaling:
    """Position interpolation: positions are divided by `factor` (model.py:337-338)."""
    factor: float


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    num_layers: int
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rope_scaling: LinearRopeScaling | None
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool

    @classmethod
    def from_hf(cls, raw: dict) -> "LlamaConfig":
        r = KeyReader(raw)
        hidden = r.integer("hidden_size", "n_embd")
        heads = r.integer("num_attention_heads", "n_head")
        head_dim = r.integer("head_dim", default=None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        kv_heads = r.integer("num_key_value_heads", default=heads)
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary pairs")
        act = r.string("hidden_act", default="silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        if r.boolean("attention_bias", "qkv_bias", default=False):
            raise ConfigError("config.json: attention_bias is true; this architecture has no biases")
        if r.boolean("mlp_bias", default=False):
            raise ConfigError("config.json: mlp_bias is true; this architecture has no biases")
        scaling = None
        sc = r.mapping("rope_scaling")
        if sc is not None:
            kind = sc.get("type") or sc.get("rope_type")
            if kind == "linear":
                factor = sc.get("factor")
                if isinstance(factor, bool) or not isinstance(factor, (int, float)) or not factor > 0:
                    raise ConfigError(f"config.json: rope_scaling.factor must be > 0, got {factor!r}")
                scaling = LinearRopeScaling(float(factor))
            elif kind in (None, "default"):
                scaling = None
            else:
                raise ConfigError(
                    f"config.json: rope_scaling type {kind!r} is not supported (only 'linear')")
        arch = raw.get("architectures")
        arch = arch[0] if isinstance(arch, list) and arch else "LlamaForCausalLM"
        return cls(
            architecture=arch,
            num_layers=r.integer("num_hidden_layers", "n_layer"),
            hidden_size=hidden,
            num_heads=heads,
            num_kv_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=r.integer("intermediate_size", default=4 * hidden),
            vocab_size=r.integer("vocab_size"),
            rope_theta=r.number("rope_theta", default=10000.0),
            rope_scaling=scaling,
            rms_norm_eps=r.number("rms_norm_eps", "layer_norm_epsilon", default=1e-6),
            max_position_embeddings=r.integer("max_position_embeddings", default=32768),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
        )

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.rope_scaling is not None:
            out["rope_scaling"] = {"type": "linear", "factor": self.rope_scaling.factor}
        return out
