"""Configuration, registry, weight loading errors and the random-weights mode (no GPU)."""
import json

import pytest
import torch

import tiny
from fastllm_py_b200.config import (ConfigError, LinearRopeScaling, LlamaConfig, load_config,
                                    register_architecture)
from fastllm_py_b200.config.registry import architecture_names
from fastllm_py_b200.parts import BuildContext, Decoder
from fastllm_py_b200.weights import (RandomStore, SafetensorsStore, WeightError, check_store,
                                     write_model_folder)

BASE = {"architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_attention_heads": 6,
        "num_hidden_layers": 3, "vocab_size": 320}


def write_config(tmp_path, raw):
    (tmp_path / "config.json").write_text(json.dumps(raw))
    return tmp_path


def test_defaults_are_the_references(tmp_path):
    arch, cfg = load_config(write_config(tmp_path, BASE))
    assert arch.name == "LlamaForCausalLM"
    assert cfg.num_kv_heads == 6 and cfg.head_dim == 16          # heads; hidden // heads
    assert cfg.intermediate_size == 4 * 96
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.max_position_embeddings == 32768 and cfg.tie_word_embeddings is False
    assert cfg.rope_scaling is None


def test_aliases_text_config_and_model_type(tmp_path):
    raw = {"model_type": "llama", "text_config": {"n_embd": 64, "n_head": 4, "n_layer": 2,
                                                   "vocab_size": 100, "layer_norm_epsilon": 1e-5}}
    arch, cfg = load_config(write_config(tmp_path, raw))
    assert (cfg.hidden_size, cfg.num_heads, cfg.num_layers, cfg.rms_norm_eps) == (64, 4, 2, 1e-5)


def test_every_key_is_read(tmp_path):
    raw = dict(BASE, num_key_value_heads=2, head_dim=32, intermediate_size=264, rope_theta=1e5,
               rope_scaling={"rope_type": "linear", "factor": 4}, rms_norm_eps=1e-5,
               max_position_embeddings=256, tie_word_embeddings=True)
    _, cfg = load_config(write_config(tmp_path, raw))
    assert cfg == LlamaConfig("LlamaForCausalLM", 3, 96, 6, 2, 32, 264, 320, 1e5,
                              LinearRopeScaling(4.0), 1e-5, 256, True)
    assert LlamaConfig.from_hf(cfg.to_hf()) == cfg                # round trip


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "big"}, "vocab_size"),
    ({"num_key_value_heads": 4}, "num_key_value_heads"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 2}}, "rope_scaling"),
    ({"rope_scaling": {"type": "linear", "factor": 0}}, "factor"),
    ({"attention_bias": True}, "attention_bias"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"architectures": ["NoSuchModel"]}, "NoSuchModel"),
])
def test_bad_configs_name_the_key(tmp_path, patch, word):
    with pytest.raises(ConfigError, match=word):
        load_config(write_config(tmp_path, dict(BASE, **patch)))


def test_registry_takes_new_architectures(tmp_path):
    class OtherConfig(LlamaConfig):
        pass

    register_architecture("OtherForCausalLM", OtherConfig, lambda cfg, names: None, ("other",))
    assert "OtherForCausalLM" in architecture_names()
    arch, cfg = load_config(write_config(tmp_path, dict(BASE, architectures=["OtherForCausalLM"])))
    assert isinstance(cfg, OtherConfig)
    raw = dict(BASE, model_type="other")
    raw.pop("architectures")
    arch, _ = load_config(write_config(tmp_path, raw))
    assert arch.name == "OtherForCausalLM"


def expected_of(name, names=None):
    from fastllm_py_b200.config.registry import architecture_of

    cfg = tiny.CONFIGS[name]["config"]
    plan = architecture_of(cfg.to_hf()).make_plan(cfg, names)
    return plan, Decoder(plan, BuildContext(torch.device("cpu"), torch.float32, 16, 8)).expected_tensors()


def test_random_mode_writes_a_loadable_folder(model_folders):
    for name in tiny.CONFIGS:
        store = SafetensorsStore(model_folders[name])
        plan, expected = expected_of(name, set(store.names()))
        check_store(expected, store)
        cfg = tiny.CONFIGS[name]["config"]
        assert ("lm_head.weight" in expected) == (not cfg.tie_word_embeddings)
        shape, dtype = store.describe("model.layers.0.mlp.down_proj.weight")
        assert shape == (cfg.hidden_size, cfg.intermediate_size) and dtype == torch.bfloat16
        assert load_config(model_folders[name])[1] == cfg


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    a = RandomStore({"x": (4, 6), "n": (6,)}, seed=1)
    b = RandomStore({"n": (6,), "other": (3, 3), "x": (4, 6)}, seed=1)
    c = RandomStore({"x": (4, 6)}, seed=2)
    assert torch.equal(a.get("x", "cpu"), b.get("x", "cpu"))
    assert not torch.equal(a.get("x", "cpu"), c.get("x", "cpu"))
    assert abs(float(a.get("n", "cpu").float().mean()) - 1.0) < 0.1      # norm weights are 1 + noise


def test_one_error_lists_everything_wrong(model_folders, tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(model_folders["tiny_a"] / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.bool)
    (tmp_path / "config.json").write_text((model_folders["tiny_a"] / "config.json").read_text())
    save_file(tensors, str(tmp_path / "model.safetensors"))
    store = SafetensorsStore(tmp_path)
    _, expected = expected_of("tiny_a", set(store.names()))
    with pytest.raises(WeightError) as e:
        check_store(expected, store, str(tmp_path))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (64, 64), (32, 64))]
    assert err.wrong_dtype[0][0] == "model.layers.0.input_layernorm.weight"
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "[32, 64]", "[64, 64]"):
        assert word in str(err)


def test_untied_model_without_head_is_an_error(model_folders, tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(model_folders["tiny_a"] / "model.safetensors"))
    del tensors["lm_head.weight"]
    save_file(tensors, str(tmp_path / "model.safetensors"))
    store = SafetensorsStore(tmp_path)
    _, expected = expected_of("tiny_a", set(store.names()))
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_store(expected, store)


def test_prefix_and_ignorable_names(model_folders, tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(model_folders["tiny_b"] / "model.safetensors"))
    bare = {k[len("model."):] if k.startswith("model.") else k: v for k, v in tensors.items()}
    bare["lm_head.weight"] = bare["embed_tokens.weight"].clone()       # a tied model may store a copy
    bare["layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(bare, str(tmp_path / "model.safetensors"))
    store = SafetensorsStore(tmp_path)
    plan, expected = expected_of("tiny_b", set(store.names()))
    assert "embed_tokens.weight" in expected
    check_store(expected, store, ignorable=plan.ignorable)


def test_stored_dtypes_are_kept(tmp_path):
    from safetensors.torch import save_file

    save_file({"a": torch.ones(2, 2, dtype=torch.bfloat16), "b": torch.ones(2, dtype=torch.float32),
               "c": torch.ones(2, dtype=torch.float16), "d": torch.ones(2, dtype=torch.int64)},
              str(tmp_path / "model.safetensors"))
    store = SafetensorsStore(tmp_path)
    got = {n: store.get(n, "cpu").dtype for n in "abcd"}
    assert got == {"a": torch.bfloat16, "b": torch.float32, "c": torch.float32, "d": torch.int32}


def test_no_safetensors_is_an_error(tmp_path):
    with pytest.raises(FileNotFoundError):
        SafetensorsStore(tmp_path)
