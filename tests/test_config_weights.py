"""Configuration, registry, command-line grammar, weight loading errors, random-weights mode."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from plain_llama import tiny_configs
from tokasaurus_b200.config import (ConfigError, EngineConfig, LlamaConfig, OptionError, UnknownArchitectureError,
                                    known_architectures, lookup_architecture, parse_overrides)
from tokasaurus_b200.weights import WeightLoadError, load_weights, write_model_folder


def test_config_reads_its_keys_and_derives_nothing_else():
    for d in tiny_configs():
        c = LlamaConfig.from_dict(d)
        assert c.hidden_size == d["hidden_size"] and c.head_dim == d["hidden_size"] // d["num_attention_heads"]
        assert c.num_key_value_heads == d["num_key_value_heads"] and c.rms_norm_eps == d["rms_norm_eps"]
        assert (c.rope_scaling is None) == (d["rope_scaling"] is None)
        again = LlamaConfig.from_dict(c.to_dict())
        assert again == c
    c = LlamaConfig.from_dict(dict(hidden_size=64, num_attention_heads=4, num_hidden_layers=1, intermediate_size=8,
                                   vocab_size=10))
    assert c.num_key_value_heads == 4 and c.rope_theta == 10000.0 and not c.tie_word_embeddings


@pytest.mark.parametrize("change, word", [
    (dict(hidden_size=65), "multiple"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=99), "head_dim"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_type"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "lacks"),
    (dict(attention_bias=True), "bias"),
    (dict(hidden_act="gelu"), "silu"),
    (dict(vocab_size=0), "positive"),
])
def test_config_errors(change, word):
    d = dict(tiny_configs()[0])
    d.update(change)
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(d)


def test_missing_required_key():
    d = dict(tiny_configs()[0])
    del d["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_dict(d)


def test_registry():
    assert "LlamaForCausalLM" in known_architectures()
    assert lookup_architecture({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert lookup_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(UnknownArchitectureError, match="LlamaForCausalLM"):
        lookup_architecture({"architectures": ["NopeForCausalLM"], "model_type": "nope"})


def test_command_line_grammar():
    cfg, extra = parse_overrides(["model=/x", "dtype=float32", "kv_cache_num_tokens=(1024*8)", "use_cudagraphs=F",
                                  "greedy_prefill=T", "page_size=32", "temperature=0.7"], EngineConfig,
                                 {"temperature": float})
    assert cfg.model == "/x" and cfg.dtype == "float32" and cfg.kv_cache_num_tokens == 8192
    assert cfg.use_cudagraphs is False and cfg.greedy_prefill is True and cfg.page_size == 32
    assert extra == {"temperature": 0.7}
    assert cfg.kv_cache_num_blocks() == 256
    for bad in (["nokey=1"], ["page_size=abc"], ["use_cudagraphs=maybe"], ["justaword"],
                ["page_size=(__import__('os').getpid())"]):
        with pytest.raises(OptionError):
            parse_overrides(bad)
    with pytest.raises(OptionError):
        EngineConfig(page_size=16, kv_cache_num_tokens=100).finalize()
    with pytest.raises(OptionError):
        EngineConfig(dtype="float16").finalize()


def _specs(cfg_dict):
    arch = lookup_architecture(cfg_dict)
    return arch.build_model(arch.parse_config(cfg_dict)).weight_specs()


def test_random_weights_folder_roundtrip(tmp_path):
    d = tiny_configs()[1]
    folder = write_model_folder(tmp_path / "m", d, seed=1, std=0.05, norm_init="uniform")
    assert json.load(open(folder / "config.json"))["hidden_size"] == 96
    again = write_model_folder(tmp_path / "m2", d, seed=1, std=0.05, norm_init="uniform")
    a, b = load_file(str(folder / "model.safetensors")), load_file(str(again / "model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    other = load_file(str(write_model_folder(tmp_path / "m3", d, seed=2, std=0.05) / "model.safetensors"))
    assert not torch.equal(a["lm_head.weight"], other["lm_head.weight"])
    assert "lm_head.weight" in a and a["lm_head.weight"].dtype == torch.bfloat16
    w = load_weights(folder, _specs(d), torch.bfloat16, "cpu")
    assert w["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert w["model.norm.weight"].dtype == torch.float32  # norm weights are used in 32-bit arithmetic
    w32 = load_weights(folder, _specs(d), torch.float32, "cpu")
    assert w32["lm_head.weight"].dtype == torch.float32
    tied = write_model_folder(tmp_path / "t", tiny_configs()[0], seed=0)
    assert "lm_head.weight" not in load_file(str(tied / "model.safetensors"))


def test_weight_errors_are_listed_together(tmp_path):
    d = tiny_configs()[0]
    folder = write_model_folder(tmp_path / "m", d, seed=0)
    t = load_file(str(folder / "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(7, 64, dtype=torch.bfloat16)
    t["model.layers.9.mlp.up_proj.weight"] = torch.zeros(2, 2)
    save_file(t, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError) as e:
        load_weights(folder, _specs(d), torch.bfloat16, "cpu")
    err = e.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.9.mlp.up_proj.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (7, 64), (32, 64))]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "model.norm.weight", "[7, 64]", "[32, 64]"):
        assert word in msg


def test_tensors_that_llama_checkpoints_may_carry_are_passed_over(tmp_path):
    """The reference reads only the names it wants (tokasaurus/model/safetensors_utils.py:72-95): an older export
    with rotary inverse frequencies, or a tied model that also stores its head, loads there.  Here such names are
    declared by the architecture and passed over with a warning; any other extra tensor is still an error."""
    from tokasaurus_b200.config import lookup_architecture

    d = tiny_configs()[0]  # tied embeddings
    folder = write_model_folder(tmp_path / "m", d, seed=0)
    t = load_file(str(folder / "model.safetensors"))
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, str(folder / "model.safetensors"))
    arch = lookup_architecture(d)
    model = arch.build_model(arch.parse_config(d))
    assert set(model.ignored_weight_patterns) == {"*.rotary_emb.inv_freq", "lm_head.weight"}
    with pytest.warns(UserWarning, match="are not used"):
        w = load_weights(folder, model.weight_specs(), torch.bfloat16, "cpu", ignore=model.ignored_weight_patterns)
    assert "lm_head.weight" not in w and "model.embed_tokens.weight" in w
    with pytest.raises(WeightLoadError) as e:
        load_weights(folder, model.weight_specs(), torch.bfloat16, "cpu")
    assert e.value.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    # an untied model does read lm_head.weight, so it is not on its list
    d1 = tiny_configs()[1]
    arch1 = lookup_architecture(d1)
    assert set(arch1.build_model(arch1.parse_config(d1)).ignored_weight_patterns) == {"*.rotary_emb.inv_freq"}


def test_no_weight_files(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs()[0]))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_weights(tmp_path, _specs(tiny_configs()[0]), torch.bfloat16, "cpu")


def test_sharded_checkpoint(tmp_path):
    d = tiny_configs()[0]
    folder = write_model_folder(tmp_path / "m", d, seed=0)
    t = load_file(str(folder / "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    save_file({k: t[k] for k in names[:half]}, str(folder / "a.safetensors"))
    save_file({k: t[k] for k in names[half:]}, str(folder / "b.safetensors"))
    (folder / "model.safetensors").unlink()
    idx = {"weight_map": {k: ("a.safetensors" if i < half else "b.safetensors") for i, k in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(idx))
    w = load_weights(folder, _specs(d), torch.float32, "cpu")
    assert all(torch.equal(w[k], t[k].float()) for k in names)


def test_stored_32bit_policy(tmp_path):
    from tokasaurus_b200.parts.base import WeightSpec
    from tokasaurus_b200.weights import target_dtype

    keep = WeightSpec("a", (2,), keep_32bit=True)
    assert target_dtype(keep, torch.float32, torch.bfloat16) == torch.float32
    assert target_dtype(keep, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert target_dtype(WeightSpec("m", (2, 2)), torch.float32, torch.bfloat16) == torch.bfloat16
    assert target_dtype(WeightSpec("t", (2,), role="table"), torch.int64, torch.bfloat16) == torch.int32
    assert target_dtype(WeightSpec("v", (2,), role="vector"), torch.bfloat16, torch.bfloat16) == torch.float32


def test_command_line_help_lists_every_option(capsys):
    from dataclasses import fields

    from tokasaurus_b200.config.engine_config import EngineConfig
    from tokasaurus_b200.engine import cli

    assert cli.main(["--help"]) == 0
    out = capsys.readouterr().out
    for f in fields(EngineConfig):
        assert f"  {f.name}=" in out
    for k in cli.RUN_OPTIONS:
        assert f"  {k}=<" in out
    assert "greedy_prefill=True" in out and "page_size=16" in out
