"""Llama / DeepSeek-LLM dense decoder as a plan of parts.

Every layer is a pre-norm block of grouped-query attention with rotary position
encoding and a SwiGLU feed-forward; layers run once each, in order, each with a
cache of its own.  Tensor names are the checkpoint's
(fastllm_py/model.py:196-231): `model.embed_tokens.weight`,
`model.layers.<i>.{input_layernorm, post_attention_layernorm}.weight`,
`model.layers.<i>.self_attn.{q,k,v,o}_proj.weight`,
`model.layers.<i>.mlp.{gate,up,down}_proj.weight`, `model.norm.weight`,
`lm_head.weight`.  The `model.` prefix is dropped when the checkpoint has none
(model.py:194).  With tie_word_embeddings the head uses the embedding table
(model.py:228-231); an untied model without `lm_head.weight` is reported as a
missing tensor instead of being tied silently.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerRun, LayerSpec, ModelPlan, PartSpec


def make_plan(cfg: LlamaConfig, tensor_names=None) -> ModelPlan:
    prefix = "model."
    if tensor_names is not None and "model.embed_tokens.weight" not in tensor_names \
            and "embed_tokens.weight" in tensor_names:
        prefix = ""
    scaling = ("linear", cfg.rope_scaling.factor) if cfg.rope_scaling is not None else None
    position = PartSpec("rotary", dict(rot_dim=cfg.head_dim, theta=cfg.rope_theta, scaling=scaling))

    def norm(name):
        return PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps), {"weight": name})

    layers = []
    for i in range(cfg.num_layers):
        base = f"{prefix}layers.{i}."
        mixer = PartSpec(
            "attention",
            dict(hidden_size=cfg.hidden_size, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
                 head_dim=cfg.head_dim, position=position, window=None),
            {s: f"{base}self_attn.{s}_proj.weight" for s in ("q", "k", "v", "o")})
        ffn = PartSpec(
            "swiglu", dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size),
            {s: f"{base}mlp.{s}_proj.weight" for s in ("gate", "up", "down")})
        layers.append(LayerSpec("prenorm", mixer, ffn, {
            "mixer": norm(base + "input_layernorm.weight"),
            "feed_forward": norm(base + "post_attention_layernorm.weight")}))
    embed_name = f"{prefix}embed_tokens.weight"
    io = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size)
    head_name = embed_name if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("table", io, {"weight": embed_name}),
        layers=layers,
        order=[LayerRun(i) for i in range(cfg.num_layers)],
        final_norm=norm(f"{prefix}norm.weight"),
        head=PartSpec("linear", io, {"weight": head_name}),
        # buffers that older checkpoints carry, and the copy of the table a tied model may store
        ignorable=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if cfg.tie_word_embeddings else ()))


register_architecture("LlamaForCausalLM", LlamaConfig, make_plan, model_types=("llama",))
